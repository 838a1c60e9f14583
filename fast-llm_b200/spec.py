"""Speculative decoding: bindings of the library's draft source, draft-length
controller and generation loop (``fl_b200_suffix_*``, ``fl_b200_spec_*``,
``fl_b200_decoder_generate_spec``), the counterparts of SuffixIndex
(src/spec/suffix_index.h), SpecController (src/spec/spec_controller.h) and the
speculative loop of tools/decode_main.cpp:329-400 in the reference."""
import ctypes as C

import numpy as np

from . import capi


class SpecCfg(C.Structure):
    """Image of fl_b200_spec_cfg."""
    _fields_ = [("n_max", C.c_int32), ("alpha0", C.c_double), ("alpha_decay", C.c_double), ("lat_decay", C.c_double),
                ("probe_iv", C.c_int32), ("probe_n", C.c_int32), ("seed_slope", C.c_double)]


class SpecStats(C.Structure):
    """Image of fl_b200_spec_stats."""
    _fields_ = [("passes", C.c_uint32), ("drafted", C.c_uint32), ("accepted", C.c_uint32), ("emitted", C.c_uint32),
                ("n_hist", C.c_uint32 * 17), ("pass_ms", C.c_double)]


class SuffixIndex:
    def __init__(self, chain_cap=64, min_match=3):
        self.lib = capi.load()
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_suffix_create(C.c_uint32(chain_cap), C.c_uint32(min_match), C.byref(self._h)))

    def close(self):
        if self._h:
            self.lib.fl_b200_suffix_destroy(self._h)
        self._h = C.c_void_p()

    __del__ = close

    def reset(self):
        self.lib.fl_b200_suffix_reset(self._h)

    def push(self, token):
        self.lib.fl_b200_suffix_push(self._h, C.c_int32(int(token)))

    def size(self):
        return self.lib.fl_b200_suffix_size(self._h)

    def draft(self, n_max, diag=False):
        """The proposed continuation (a list, possibly empty); with diag=True also
        (tail gram indexed, candidates compared, longest match, entries walked)."""
        out = (C.c_int32 * max(n_max, 1))()
        dg = (C.c_int32 * 4)()
        n = self.lib.fl_b200_suffix_draft(self._h, C.c_int32(n_max), out, dg)
        toks = list(out[:n])
        return (toks, tuple(dg)) if diag else toks


class SpecController:
    def __init__(self, **cfg):
        self.lib = capi.load()
        c = SpecCfg()
        self.lib.fl_b200_spec_cfg_default(C.byref(c))
        for k, v in cfg.items():
            setattr(c, k, v)
        self.cfg = c
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_spec_create(C.byref(c), C.byref(self._h)))

    def close(self):
        if self._h:
            self.lib.fl_b200_spec_destroy(self._h)
        self._h = C.c_void_p()

    __del__ = close

    def choose(self):
        return self.lib.fl_b200_spec_choose(self._h)

    def observe(self, n_drafted, n_accepted, pass_ms):
        self.lib.fl_b200_spec_observe(self._h, C.c_int32(n_drafted), C.c_int32(n_accepted), C.c_double(pass_ms))

    def alpha(self):
        return self.lib.fl_b200_spec_alpha(self._h)

    def lat_est(self, n):
        return self.lib.fl_b200_spec_lat_est(self._h, C.c_int32(n))

    def expected_emitted(self, n):
        return self.lib.fl_b200_spec_expected_emitted(self._h, C.c_int32(n))


def generate(dec, first_token, n_gen, index, ctrl=None, spec_max=7, spec_fixed=-1):
    """n_gen tokens (first_token first) from a fast_llm_b200.decoder.Decoder with
    speculation; returns (tokens, SpecStats)."""
    out = np.zeros(n_gen, dtype=np.int32)
    st = SpecStats()
    capi._ck(dec.lib.fl_b200_decoder_generate_spec(dec._h, C.c_int32(int(first_token)), C.c_uint32(n_gen),
                                                   C.c_int32(spec_max), C.c_int32(spec_fixed), index._h,
                                                   ctrl._h if ctrl else None, C.c_void_p(out.ctypes.data), C.byref(st)))
    return [int(t) for t in out], st
