"""Host-side mirror of the reference's ``Decoder`` interface
(src/model/decoder.h:52-81) for the Llama shape, over the C ABI decoder
(``fl_b200_decoder_*``): ``step``, ``n_past``, ``rewind_to``, ``logits``,
``last_margin``. All arithmetic happens in the CUDA library."""
import ctypes as C

import numpy as np

from . import capi


class Decoder:
    def __init__(self, ctx, cfg, tp=None):
        """cfg: dict with n_layer, n_embd, n_head, n_kv_head, head_dim, n_ff,
        n_vocab, max_kv, rope_base, eps (the whole model). tp = (rank, world)
        makes this the decoder of one rank of a tensor-parallel group: tensors are
        then handed over sliced (fast_llm_b200.tp) and fast_llm_b200.tp.connect
        must run before finalize."""
        self.ctx = ctx
        self.lib = ctx.lib
        self.cfg = dict(cfg)
        self.rank, self.world = tp if tp else (0, 1)
        c = capi.LlamaCfg(**{k: cfg[k] for k in ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim",
                                                  "n_ff", "n_vocab", "max_kv", "rope_base", "eps")})
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_decoder_create_tp(ctx._h, C.byref(c), C.c_uint32(self.rank), C.c_uint32(self.world),
                                                    C.byref(self._h)))
        # this rank's share of the sizes that are split
        self.loc = dict(self.cfg)
        for k in ("n_head", "n_kv_head", "n_ff", "n_vocab"):
            self.loc[k] = cfg[k] // self.world
        self._keep = []   # device tensors the decoder points into
        self._peer_maps = []

    @classmethod
    def from_gguf(cls, ctx, gguf, max_kv, tp=None):
        """The decoder of a "llama" GGUF file (fast_llm_b200.gguf.Gguf), weights
        uploaded by the library (DecoderImpl::load, src/model/decoder.cpp:277-321).
        Not finalized: with tp = (rank, world) run fast_llm_b200.tp.connect first."""
        self = cls.__new__(cls)
        self.ctx, self.lib = ctx, ctx.lib
        self.rank, self.world = tp if tp else (0, 1)
        c = gguf.llama_cfg(max_kv)
        self.cfg = {k: getattr(c, k) for k, _ in capi.LlamaCfg._fields_}
        self.loc = dict(self.cfg)
        for k in ("n_head", "n_kv_head", "n_ff", "n_vocab"):
            self.loc[k] = self.cfg[k] // self.world
        self._keep, self._peer_maps = [], []
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_decoder_create_gguf(ctx._h, gguf._h, C.c_uint32(max_kv), C.c_uint32(self.rank),
                                                      C.c_uint32(self.world), C.byref(self._h)))
        return self

    def close(self):
        if self._h and not self.ctx._h:
            self._h = C.c_void_p()   # the context is gone already (teardown order): nothing left to free safely
        if self._h:
            self.lib.fl_b200_decoder_destroy(self._h)
            self._h = C.c_void_p()
            self._keep = []
            for p in self._peer_maps:
                self.lib.fl_b200_ipc_close(self.ctx._h, C.c_void_p(p))
            self._peer_maps = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- model set-up --
    def set_layer_tensor(self, layer, which, fmt, w):
        self._keep.append(w)
        capi._ck(self.lib.fl_b200_decoder_set_layer_tensor(self._h, C.c_uint32(layer), which, fmt, capi._p(w)))

    def set_layer_norms(self, layer, attn_norm, ffn_norm):
        self._keep += [attn_norm, ffn_norm]
        capi._ck(self.lib.fl_b200_decoder_set_layer_norms(self._h, C.c_uint32(layer), capi._p(attn_norm),
                                                          capi._p(ffn_norm)))

    def set_layer_moe(self, layer, block):
        """A fast_llm_b200.moe.MoeBlock in place of the layer's gate / up / down (a Mixtral-shape layer)."""
        self._keep.append(block)
        capi._ck(self.lib.fl_b200_decoder_set_layer_moe(self._h, C.c_uint32(layer), block._h))

    def set_global(self, which, fmt, w):
        self._keep.append(w)
        capi._ck(self.lib.fl_b200_decoder_set_global(self._h, which, fmt, capi._p(w)))

    def set_out_norm(self, w):
        self._keep.append(w)
        capi._ck(self.lib.fl_b200_decoder_set_out_norm(self._h, capi._p(w)))

    def kv_ptrs(self, layer):
        k, v = C.c_void_p(), C.c_void_p()
        capi._ck(self.lib.fl_b200_decoder_kv(self._h, C.c_uint32(layer), C.byref(k), C.byref(v)))
        return k.value, v.value

    def step_batch(self, tokens):
        """Decoder::step_batch: feeds len(tokens) <= 8 tokens in one pass; returns
        (greedy token after each position, its top1 - top2 margin)."""
        m = len(tokens)
        toks = (C.c_int32 * m)(*[int(t) for t in tokens])
        outs, margins = (C.c_int32 * m)(), (C.c_float * m)()
        capi._ck(self.lib.fl_b200_decoder_step_batch(self._h, toks, C.c_uint32(m), outs, margins))
        return list(outs), list(margins)

    # -- independent sequences in lock step --
    def seqs_init(self, n_seq):
        capi._ck(self.lib.fl_b200_decoder_seqs_init(self._h, C.c_uint32(n_seq)))
        self.n_seq = n_seq

    def seqs_kv_ptrs(self, layer, seq):
        k, v = C.c_void_p(), C.c_void_p()
        capi._ck(self.lib.fl_b200_decoder_seqs_kv(self._h, C.c_uint32(layer), C.c_uint32(seq), C.byref(k), C.byref(v)))
        return k.value, v.value

    def seqs_set_pos(self, seq, n_past):
        capi._ck(self.lib.fl_b200_decoder_seqs_set_pos(self._h, C.c_uint32(seq), C.c_int32(n_past)))

    def seqs_pos(self, seq):
        out = C.c_int32()
        capi._ck(self.lib.fl_b200_decoder_seqs_pos(self._h, C.c_uint32(seq), C.byref(out)))
        return out.value

    def seqs_step(self, tokens):
        """One token per sequence; returns (greedy token of every sequence, its top1 - top2 margin)."""
        m = self.n_seq
        assert len(tokens) == m
        toks = (C.c_int32 * m)(*[int(t) for t in tokens])
        outs, margins = (C.c_int32 * m)(), (C.c_float * m)()
        capi._ck(self.lib.fl_b200_decoder_seqs_step(self._h, toks, outs, margins))
        return list(outs), list(margins)

    def batch_logits(self, index):
        out = np.empty(self.loc["n_vocab"], dtype=np.float32)
        capi._ck(self.lib.fl_b200_decoder_batch_logits(self._h, C.c_uint32(index), out.ctypes.data_as(C.c_void_p)))
        return out

    def finalize(self):
        capi._ck(self.lib.fl_b200_decoder_finalize(self._h))

    # -- Decoder interface --
    def step(self, token):
        out = C.c_int32()
        capi._ck(self.lib.fl_b200_decoder_step(self._h, C.c_int32(int(token)), C.byref(out)))
        return out.value

    def run(self, first_token, n):
        """n greedy steps with the argmax fed back on the device."""
        toks = np.zeros(n, dtype=np.int32)
        capi._ck(self.lib.fl_b200_decoder_run(self._h, C.c_int32(int(first_token)), C.c_uint32(n),
                                              C.c_void_p(toks.ctypes.data)))
        return toks

    def verify(self, first_token, draft):
        """Greedy verification of a draft: (number of accepted draft tokens, the model's next token)."""
        arr = (C.c_int32 * len(draft))(*[int(t) for t in draft])
        acc, nxt = C.c_uint32(), C.c_int32()
        capi._ck(self.lib.fl_b200_decoder_verify(self._h, C.c_int32(int(first_token)), arr, C.c_uint32(len(draft)),
                                                 C.byref(acc), C.byref(nxt)))
        return acc.value, nxt.value

    def n_past(self):
        v = C.c_int32()
        capi._ck(self.lib.fl_b200_decoder_n_past(self._h, C.byref(v)))
        return v.value

    def rewind_to(self, pos):
        capi._ck(self.lib.fl_b200_decoder_set_n_past(self._h, C.c_int32(int(pos))))

    def logits(self):
        out = np.empty(self.loc["n_vocab"], dtype=np.float32)   # this rank's slice of the vocabulary
        capi._ck(self.lib.fl_b200_decoder_logits(self._h, C.c_void_p(out.ctypes.data)))
        return out

    def last_margin(self):
        v = C.c_float()
        capi._ck(self.lib.fl_b200_decoder_margin(self._h, C.byref(v)))
        return v.value

    def tap(self, which):
        c = self.loc
        n = {0: c["n_embd"], 1: c["n_embd"], 2: c["n_head"] * c["head_dim"], 3: c["n_kv_head"] * c["head_dim"],
             4: c["n_head"] * c["head_dim"], 5: c["n_embd"], 6: c["n_ff"], 7: c["n_ff"]}[which]
        out = np.empty(n, dtype=np.float32)
        capi._ck(self.lib.fl_b200_decoder_tap(self._h, which, C.c_void_p(out.ctypes.data)))
        return out

    def time_class(self, kernel_class, reps):
        """(ms per step, launches per step) of one kernel class replayed alone:
        1 matvec, 2 attention, 4 small operators, 8 exchange steps (tensor parallel), 15 all."""
        ms, n = C.c_float(), C.c_uint32()
        capi._ck(self.lib.fl_b200_decoder_time_class(self._h, C.c_uint32(kernel_class), C.c_uint32(reps),
                                                     C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def trace(self):
        """Per-launch device timestamps of the last step (FLB_TRACE=1): array [n, 4] of ns."""
        cap = 16 + 8 * self.cfg["n_layer"]
        buf = np.zeros((cap, 4), dtype=np.uint64)
        n = C.c_uint32()
        capi._ck(self.lib.fl_b200_decoder_trace(self._h, C.c_void_p(buf.ctypes.data), C.c_uint32(cap), C.byref(n)))
        return buf[:n.value]

    def launches_per_step(self):
        v = C.c_uint32()
        capi._ck(self.lib.fl_b200_decoder_launches_per_step(self._h, C.byref(v)))
        return v.value

    def bytes_per_step(self, pos):
        w, kv = C.c_uint64(), C.c_uint64()
        capi._ck(self.lib.fl_b200_decoder_bytes_per_step(self._h, C.c_int32(int(pos)), C.byref(w), C.byref(kv)))
        return w.value, kv.value
