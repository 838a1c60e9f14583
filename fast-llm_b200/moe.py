"""Mixture-of-experts feed-forward block over the C ABI (``fl_b200_moe_*``): single
GPU or expert parallel over the GPUs of one box (one process per GPU)."""
import ctypes as C

import numpy as np

from . import capi


class MoeCfg(C.Structure):
    """Image of fl_b200_moe_cfg."""
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_expert", C.c_uint32), ("top_k", C.c_uint32),
                ("norm", C.c_uint32), ("scale", C.c_float), ("fmt_gate_up", C.c_int32), ("fmt_down", C.c_int32),
                ("max_tokens", C.c_uint32)]


def local_experts(n_expert, rank, world):
    """[first, first + count) of the experts rank `rank` holds."""
    if n_expert % world:
        raise ValueError("%d ranks do not divide %d experts" % (world, n_expert))
    n = n_expert // world
    return rank * n, n


class MoeBlock:
    def __init__(self, ctx, n_embd, n_ff, n_expert, top_k, norm=1, scale=1.0, fmt_gate_up=capi.Q4_K, fmt_down=capi.Q4_K,
                 max_tokens=16, ep=None):
        self.ctx, self.lib = ctx, ctx.lib
        self.rank, self.world = ep if ep else (0, 1)
        self.cfg = MoeCfg(n_embd, n_ff, n_expert, top_k, norm, scale, fmt_gate_up, fmt_down, max_tokens)
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_moe_create(ctx._h, C.byref(self.cfg), C.c_uint32(self.rank), C.c_uint32(self.world),
                                             C.byref(self._h)))
        self._keep, self._maps = [], []

    def set_weights(self, router, gate, up, down):
        """Device tensors: router f32 [n_expert][n_embd]; this rank's experts stacked row-wise."""
        self._keep = [router, gate, up, down]
        capi._ck(self.lib.fl_b200_moe_set_weights(self._h, capi._p(router), capi._p(gate), capi._p(up), capi._p(down)))

    def connect(self, dist, group=None):
        """Maps every rank's exchange buffer into this process (as fast_llm_b200.tp.connect does for the decoder)."""
        buf, nbytes = C.c_void_p(), C.c_size_t()
        capi._ck(self.lib.fl_b200_moe_comm(self._h, C.byref(buf), C.byref(nbytes)))
        handle = (C.c_uint8 * 64)()
        capi._ck(self.lib.fl_b200_ipc_export(self.ctx._h, buf, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        ptrs = (C.c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                ptrs[r] = buf.value
            else:
                p = C.c_void_p()
                capi._ck(self.lib.fl_b200_ipc_open(self.ctx._h, (C.c_uint8 * 64).from_buffer_copy(handles[r]), C.byref(p)))
                ptrs[r] = p.value
                self._maps.append(p.value)
        capi._ck(self.lib.fl_b200_moe_set_peers(self._h, ptrs, C.c_uint32(self.world)))

    def forward(self, x, n_tok, y):
        capi._ck(self.lib.fl_b200_moe_forward(self._h, capi._p(x), C.c_uint32(n_tok), capi._p(y)))

    def routing(self, n_tok):
        k = self.cfg.top_k
        ids, gates = np.zeros((n_tok, k), dtype=np.uint32), np.zeros((n_tok, k), dtype=np.float32)
        capi._ck(self.lib.fl_b200_moe_routing(self._h, C.c_uint32(n_tok), ids.ctypes.data_as(C.c_void_p),
                                              gates.ctypes.data_as(C.c_void_p)))
        return ids, gates

    def close(self):
        if self._h and self.ctx._h:
            for p in self._maps:
                self.lib.fl_b200_ipc_close(self.ctx._h, C.c_void_p(p))
            self.lib.fl_b200_moe_destroy(self._h)
        self._h = C.c_void_p()
        self._maps = []
