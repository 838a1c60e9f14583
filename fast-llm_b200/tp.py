"""Tensor-parallel partition of the Llama-shape decode step over the GPUs of one
box (one process per GPU). The reference has no multi-GPU path; the partition
follows its decode graph (src/model/decoder.cpp:639-672): tensors whose outputs
are per head or per FFN row are split by rows, the two projections back to the
hidden size (O, down) by columns, and the replicated hidden state is rebuilt by
summing the ranks' partial vectors.

Everything here is layout arithmetic on packed GGUF tensors ``[rows, row_bytes]``
(numpy arrays or torch tensors alike) and the set-up handshake; the arithmetic
runs in the CUDA library.
"""
import ctypes as C

from . import capi

ROW_SPLIT = ("wq", "wk", "wv", "gate", "up", "output")
COL_SPLIT = ("wo", "down")


def local_dims(cfg, world):
    """Per-rank sizes: query heads, KV heads, FFN rows, vocabulary rows."""
    if cfg["n_kv_head"] % world or cfg["n_ff"] % (256 * world) or cfg["n_vocab"] % world:
        raise ValueError("%d ranks do not divide n_kv_head=%d, n_ff=%d/256, n_vocab=%d"
                         % (world, cfg["n_kv_head"], cfg["n_ff"], cfg["n_vocab"]))
    return dict(n_head=cfg["n_head"] // world, n_kv_head=cfg["n_kv_head"] // world, n_ff=cfg["n_ff"] // world,
                n_vocab=cfg["n_vocab"] // world)


def slice_of(name, cfg, rank, world):
    """(axis, start, count) of tensor `name` owned by `rank`: axis 0 = rows, 1 = columns
    (in weights, a multiple of 256). KV head h lives on rank h // (n_kv_head / world) with
    its 4 query heads, so row and column ranges of wq / wo and wk / wv line up."""
    loc = local_dims(cfg, world)
    d = cfg["head_dim"]
    n = {"wq": loc["n_head"] * d, "wk": loc["n_kv_head"] * d, "wv": loc["n_kv_head"] * d, "wo": loc["n_head"] * d,
         "gate": loc["n_ff"], "up": loc["n_ff"], "down": loc["n_ff"], "output": loc["n_vocab"]}[name]
    return (1 if name in COL_SPLIT else 0), rank * n, n


def pitch_of(fmt, cols):
    """Row pitch of a column slice: its row bytes rounded up to 16 (the library's rule)."""
    return (capi.row_bytes(fmt, cols) + 15) // 16 * 16


def slice_rows(w, start, count):
    return w[start:start + count]


def slice_cols(w, fmt, start, count):
    """Blocks [start/256, (start+count)/256) of every row, each row zero-padded to
    a multiple of 16 bytes. Works on numpy arrays and torch tensors."""
    bb = capi.BLK_BYTES[fmt]
    be = capi.BLK_ELEMS[fmt]
    if start % be or count % be:
        raise ValueError("column slice not block aligned")
    part = w[:, start // be * bb:(start + count) // be * bb]
    pad = pitch_of(fmt, count) - part.shape[1]
    if hasattr(part, "numpy") or type(part).__module__.startswith("torch"):
        import torch
        part = part.contiguous()
        if pad:
            part = torch.nn.functional.pad(part, (0, pad))
        return part.contiguous()
    import numpy as np
    out = np.zeros((part.shape[0], part.shape[1] + pad), dtype=np.uint8)
    out[:, :part.shape[1]] = part
    return out


def shard_tensor(name, w, fmt, cfg, rank, world):
    axis, start, count = slice_of(name, cfg, rank, world)
    return slice_cols(w, fmt, start, count) if axis else slice_rows(w, start, count)


def merge_top(records):
    """Host restatement of the cross-rank argmax merge (records in rank order,
    each (best, global index, runner-up)): highest value, lowest index on ties,
    margin = best - runner-up (src/model/decoder.cpp:1253-1264)."""
    b, i, s = float("-inf"), 2 ** 32 - 1, float("-inf")
    for yb, yi, ys in records:
        if yb > b or (yb == b and yi < i):
            b, i, s = yb, yi, max(b, s, ys)
        else:
            s = max(yb, s, ys)
    return i, b - s


def merge_lse(records):
    """Host restatement of the cross-rank attention merge: records in rank order, each
    (context[128] normalised over the rank's keys, max score, sum of exp(score - max));
    returns the context over all keys."""
    import numpy as np
    M = max(m for _, m, _ in records)
    acc, W = np.zeros_like(np.asarray(records[0][0], dtype=np.float64)), 0.0
    for o, m, l in records:
        w = 0.0 if (l == 0 or m == float("-inf")) else l * np.exp(m - M)
        acc += w * np.asarray(o, dtype=np.float64)
        W += w
    return acc / W


def connect(dec, dist, group=None):
    """Maps every rank's exchange buffer into this process and hands the pointers
    to the decoder. `dist` is torch.distributed with an initialised process group
    (any backend: only Python objects travel)."""
    lib, ctx = dec.lib, dec.ctx
    buf, nbytes = C.c_void_p(), C.c_size_t()
    capi._ck(lib.fl_b200_decoder_comm(dec._h, C.byref(buf), C.byref(nbytes)))
    handle = (C.c_uint8 * 64)()
    capi._ck(lib.fl_b200_ipc_export(ctx._h, buf, handle))
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle), group=group)
    ptrs = (C.c_void_p * world)()
    opened = []
    for r in range(world):
        if r == rank:
            ptrs[r] = buf.value
        else:
            h = (C.c_uint8 * 64).from_buffer_copy(handles[r])
            p = C.c_void_p()
            capi._ck(lib.fl_b200_ipc_open(ctx._h, h, C.byref(p)))
            ptrs[r] = p.value
            opened.append(p.value)
    capi._ck(lib.fl_b200_decoder_set_peers(dec._h, ptrs, C.c_uint32(world)))
    dec._peer_maps = opened
    return opened


class SeqParallel:
    """Cross-GPU merge of sequence-parallel decode attention (the long-context
    configuration): every rank attends its contiguous slice of the keys with
    Context.attn_decode_lse, then combine() merges the ranks' (context, max, sum)
    records through peer memory; all ranks get identical results."""

    def __init__(self, ctx, dist, max_records, group=None):
        self.ctx, self.lib = ctx, ctx.lib
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_seqpar_create(ctx._h, C.c_uint32(self.rank), C.c_uint32(self.world),
                                                C.c_uint32(max_records), C.byref(self._h)))
        buf, nbytes = C.c_void_p(), C.c_size_t()
        capi._ck(self.lib.fl_b200_seqpar_comm(self._h, C.byref(buf), C.byref(nbytes)))
        handle = (C.c_uint8 * 64)()
        capi._ck(self.lib.fl_b200_ipc_export(ctx._h, buf, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        ptrs = (C.c_void_p * self.world)()
        self._maps = []
        for r in range(self.world):
            if r == self.rank:
                ptrs[r] = buf.value
            else:
                p = C.c_void_p()
                capi._ck(self.lib.fl_b200_ipc_open(ctx._h, (C.c_uint8 * 64).from_buffer_copy(handles[r]), C.byref(p)))
                ptrs[r] = p.value
                self._maps.append(p.value)
        capi._ck(self.lib.fl_b200_seqpar_set_peers(self._h, ptrs, C.c_uint32(self.world)))

    def combine(self, out_local, lse_local, n_records, out):
        capi._ck(self.lib.fl_b200_seqpar_combine(self._h, capi._p(out_local), capi._p(lse_local),
                                                 C.c_uint32(n_records), capi._p(out)))

    def close(self):
        if self._h and self.ctx._h:
            for p in self._maps:
                self.lib.fl_b200_ipc_close(self.ctx._h, C.c_void_p(p))
            self.lib.fl_b200_seqpar_destroy(self._h)
        self._h = C.c_void_p()
        self._maps = []
