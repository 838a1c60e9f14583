"""ctypes binding of the C ABI declared in ``include/fl_b200.h``.

Every call goes through ``libfl_b200.so``; a missing library, a missing symbol
or a missing CUDA device raises. Nothing here computes on the CPU.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfl_b200.so")

F32, Q8_0, Q5_0, Q4_K, Q6_K = 0, 1, 2, 3, 4
FMT_NAMES = {F32: "F32", Q8_0: "Q8_0", Q5_0: "Q5_0", Q4_K: "Q4_K", Q6_K: "Q6_K"}
# TaskKind values (include/fastllm/fastllm.h:17-45 of the reference; 13 and 14 are appended here)
K_STREAM_DOT, K_MERGE, K_SIGNAL, K_ACT_Q8, K_STREAM_DOT_IDX, K_RMSNORM, K_ADD2, K_ROPE_DS2, K_KV_APPEND = range(9)
K_ATTN_HEAD, K_ROUTER_SEL, K_SILU_MUL, K_WMERGE, K_ATTN_GQA_F16, K_ROPE_KV_APPEND_F16 = range(9, 15)
BLK_ELEMS = {F32: 1, Q8_0: 32, Q5_0: 32, Q4_K: 256, Q6_K: 256}
BLK_BYTES = {F32: 4, Q8_0: 34, Q5_0: 22, Q4_K: 144, Q6_K: 210}

T_WQ, T_WK, T_WV, T_WO, T_GATE, T_UP, T_DOWN = range(7)
G_TOK_EMBD, G_OUTPUT = 0, 1

# Every symbol include/fl_b200.h declares (the CPU test suite checks the
# library exports each of them).
SYMBOLS = [
    "fl_b200_abi_version", "fl_b200_last_error", "fl_b200_create", "fl_b200_destroy", "fl_b200_sync",
    "fl_b200_device_status", "fl_b200_sm_count", "fl_b200_set_wait_limit", "fl_b200_stream", "fl_b200_malloc", "fl_b200_free",
    "fl_b200_upload", "fl_b200_download", "fl_b200_memset", "fl_b200_ipc_export", "fl_b200_ipc_open", "fl_b200_ipc_close", "fl_b200_timer_start", "fl_b200_timer_stop",
    "fl_b200_dequant", "fl_b200_matvec", "fl_b200_matvec_assign", "fl_b200_matvec_expert", "fl_b200_matvec_pitched", "fl_b200_matvec_host",
    "fl_b200_attn_decode", "fl_b200_attn_decode_lse", "fl_b200_seqpar_create", "fl_b200_seqpar_destroy",
    "fl_b200_seqpar_comm", "fl_b200_seqpar_set_peers", "fl_b200_seqpar_combine", "fl_b200_attn_verify", "fl_b200_attn_decode_static", "fl_b200_attn_decode_host", "fl_b200_rmsnorm", "fl_b200_add2",
    "fl_b200_silu_mul", "fl_b200_router_sel", "fl_b200_wmerge", "fl_b200_rope_kv_append", "fl_b200_argmax", "fl_b200_exec_task", "fl_b200_plan_create", "fl_b200_plan_run", "fl_b200_plan_info", "fl_b200_plan_destroy",
    "fl_b200_decoder_create", "fl_b200_decoder_create_tp", "fl_b200_decoder_comm", "fl_b200_decoder_set_peers",
    "fl_b200_decoder_destroy", "fl_b200_decoder_set_layer_tensor",
    "fl_b200_decoder_set_layer_norms", "fl_b200_decoder_set_layer_moe", "fl_b200_decoder_set_global", "fl_b200_decoder_set_out_norm",
    "fl_b200_decoder_kv", "fl_b200_decoder_finalize", "fl_b200_decoder_set_n_past",
    "fl_b200_decoder_n_past", "fl_b200_decoder_step", "fl_b200_decoder_run", "fl_b200_decoder_verify", "fl_b200_decoder_step_batch", "fl_b200_decoder_batch_logits", "fl_b200_decoder_seqs_init", "fl_b200_decoder_seqs_kv", "fl_b200_decoder_seqs_set_pos", "fl_b200_decoder_seqs_pos", "fl_b200_decoder_seqs_step", "fl_b200_decoder_logits",
    "fl_b200_decoder_margin", "fl_b200_decoder_tap", "fl_b200_decoder_time_class", "fl_b200_decoder_trace", "fl_b200_decoder_launches_per_step",
    "fl_b200_decoder_bytes_per_step",
    "fl_b200_gguf_open", "fl_b200_gguf_close", "fl_b200_gguf_counts", "fl_b200_gguf_tensor_at", "fl_b200_gguf_find",
    "fl_b200_gguf_has", "fl_b200_gguf_kv_i", "fl_b200_gguf_kv_f", "fl_b200_gguf_kv_s", "fl_b200_gguf_kv_sarr_count",
    "fl_b200_gguf_kv_sarr_at", "fl_b200_gguf_llama_cfg", "fl_b200_decoder_create_gguf",
    "fl_b200_suffix_create", "fl_b200_suffix_destroy", "fl_b200_suffix_reset", "fl_b200_suffix_push", "fl_b200_suffix_size",
    "fl_b200_suffix_draft", "fl_b200_spec_cfg_default", "fl_b200_spec_create", "fl_b200_spec_destroy", "fl_b200_spec_choose",
    "fl_b200_spec_observe", "fl_b200_spec_alpha", "fl_b200_spec_lat_est", "fl_b200_spec_expected_emitted",
    "fl_b200_decoder_generate_spec",
    "fl_b200_moe_create", "fl_b200_moe_destroy", "fl_b200_moe_set_weights", "fl_b200_moe_comm", "fl_b200_moe_set_peers",
    "fl_b200_moe_forward", "fl_b200_moe_routing",
]


def row_bytes(fmt, cols):
    return cols // BLK_ELEMS[fmt] * BLK_BYTES[fmt]


class Fl200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("fl_b200 error %d: %s" % (code, msg))
        self.code = code


class LlamaCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim", "n_ff", "n_vocab", "max_kv")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)]


class Task(C.Structure):
    """Image of fl_b200_task (= fastllm::Task, include/fastllm/fastllm.h:65-97)."""
    _fields_ = [
        ("id", C.c_uint32), ("kind", C.c_uint8), ("affinity", C.c_uint8), ("fmt", C.c_uint8),
        ("n_consumers", C.c_uint16), ("consumers", C.c_uint32 * 6), ("w", C.c_void_p),
        ("w_bytes", C.c_uint64), ("x", C.c_void_p), ("y", C.c_void_p), ("rows", C.c_uint32),
        ("cols", C.c_uint32), ("dep_init", C.c_int32), ("dep_count", C.c_int32), ("epoch", C.c_uint32),
        ("handoff_ts", C.c_uint64), ("aux", C.c_void_p), ("aux2", C.c_uint64), ("nx", C.c_uint32),
        ("xstride", C.c_uint32), ("ystride", C.c_uint32), ("_pad", C.c_uint8 * 124),
    ]


_lib = None


def load():
    """Loads the library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "%s is missing: build it with `python -m fast_llm_b200.build` "
            "(there is no fallback path)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for s in SYMBOLS:
        getattr(lib, s)   # AttributeError if the ABI is incomplete
    lib.fl_b200_last_error.restype = C.c_char_p
    lib.fl_b200_stream.restype = C.c_void_p
    lib.fl_b200_destroy.restype = None
    lib.fl_b200_decoder_destroy.restype = None
    lib.fl_b200_seqpar_destroy.restype = None
    lib.fl_b200_plan_destroy.restype = None
    lib.fl_b200_gguf_close.restype = None
    lib.fl_b200_moe_destroy.restype = None
    for name in ("fl_b200_suffix_destroy", "fl_b200_suffix_reset", "fl_b200_suffix_push", "fl_b200_spec_cfg_default",
                 "fl_b200_spec_destroy", "fl_b200_spec_observe"):
        getattr(lib, name).restype = None
    lib.fl_b200_suffix_size.restype = C.c_uint64
    for name in ("fl_b200_spec_alpha", "fl_b200_spec_lat_est", "fl_b200_spec_expected_emitted"):
        getattr(lib, name).restype = C.c_double
    lib.fl_b200_gguf_kv_i.restype = C.c_int64
    lib.fl_b200_gguf_kv_f.restype = C.c_double
    lib.fl_b200_gguf_kv_sarr_count.restype = C.c_int64
    _lib = lib
    return lib


def _ck(rc):
    if rc != 0:
        raise Fl200Error(rc, load().fl_b200_last_error().decode())


def _p(t):
    """Device pointer of a torch tensor, or pass integers / None through."""
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


class Context:
    """One device, one stream (fl_b200_ctx)."""

    def __init__(self, device=0):
        lib = load()
        self._h = C.c_void_p()
        _ck(lib.fl_b200_create(C.c_int(device), C.byref(self._h)))
        self.lib = lib
        self.device = device

    def close(self):
        if self._h:
            self.lib.fl_b200_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- plumbing --
    def sync(self):
        _ck(self.lib.fl_b200_sync(self._h))

    def status(self):
        v = C.c_uint32()
        _ck(self.lib.fl_b200_device_status(self._h, C.byref(v)))
        return v.value

    def sm_count(self):
        return self.lib.fl_b200_sm_count(self._h)

    def set_wait_limit(self, nanoseconds):
        """Limit of the exchange kernels' waits for another rank (0 = one second)."""
        _ck(self.lib.fl_b200_set_wait_limit(self._h, C.c_uint64(nanoseconds)))

    def stream(self):
        return self.lib.fl_b200_stream(self._h)

    def timer_start(self):
        _ck(self.lib.fl_b200_timer_start(self._h))

    def timer_stop(self):
        ms = C.c_float()
        _ck(self.lib.fl_b200_timer_stop(self._h, C.byref(ms)))
        return ms.value

    # -- operators (torch CUDA tensors or raw device pointers) --
    def dequant(self, fmt, w, rows, cols, out):
        _ck(self.lib.fl_b200_dequant(self._h, fmt, _p(w), C.c_uint64(rows), C.c_uint32(cols), _p(out)))

    def matvec(self, fmt, w, rows, cols, x, y, nx=1, xstride=0, ystride=0):
        """STREAM_DOT semantics: y += W x."""
        _ck(self.lib.fl_b200_matvec(self._h, fmt, _p(w), C.c_uint32(rows), C.c_uint32(cols), _p(x),
                                    C.c_uint32(nx), C.c_uint32(xstride), _p(y), C.c_uint32(ystride)))

    def matvec_assign(self, fmt, w, rows, cols, x, y):
        _ck(self.lib.fl_b200_matvec_assign(self._h, fmt, _p(w), C.c_uint32(rows), C.c_uint32(cols), _p(x), _p(y)))

    def matvec_expert(self, fmt, w, rows, cols, expert_id, expert_stride, x, y, nx=1, xstride=0, ystride=0):
        """STREAM_DOT_IDX: accumulates W[expert] x into y; expert_id is a device uint32."""
        _ck(self.lib.fl_b200_matvec_expert(self._h, fmt, _p(w), C.c_uint32(rows), C.c_uint32(cols), _p(expert_id),
                                           C.c_uint64(expert_stride), _p(x), C.c_uint32(nx), C.c_uint32(xstride),
                                           _p(y), C.c_uint32(ystride)))

    def router_sel(self, logits, ids, gates, n_expert, top_k, norm, scale):
        _ck(self.lib.fl_b200_router_sel(self._h, _p(logits), _p(ids), _p(gates), C.c_uint32(n_expert),
                                        C.c_uint32(top_k), C.c_uint32(norm), C.c_float(scale)))

    def wmerge(self, parts, gates, add1, add2, y, scale, n_parts, n, n_full=0):
        _ck(self.lib.fl_b200_wmerge(self._h, _p(parts), _p(gates), _p(add1), _p(add2), _p(y), C.c_float(scale),
                                    C.c_uint32(n_parts), C.c_uint32(n), C.c_uint32(n_full)))

    def matvec_pitched(self, fmt, w, rows, cols, pitch, x, y):
        _ck(self.lib.fl_b200_matvec_pitched(self._h, fmt, _p(w), C.c_uint32(rows), C.c_uint32(cols), C.c_uint32(pitch),
                                            _p(x), _p(y)))

    def matvec_host(self, fmt, w, rows, cols, x_host, y_host):
        """x_host / y_host: numpy float32 arrays (or pinned torch CPU tensors)."""
        _ck(self.lib.fl_b200_matvec_host(self._h, fmt, _p(w), C.c_uint32(rows), C.c_uint32(cols),
                                         _hp(x_host), _hp(y_host)))

    def attn_decode(self, q, k, v, n_q_head, n_kv_head, head_dim, kv_len, kv_stride, batch, scale, out):
        _ck(self.lib.fl_b200_attn_decode(self._h, _p(q), _p(k), _p(v), C.c_uint32(n_q_head),
                                         C.c_uint32(n_kv_head), C.c_uint32(head_dim), C.c_uint32(kv_len),
                                         C.c_uint32(kv_stride), C.c_uint32(batch), C.c_float(scale), _p(out)))

    def attn_decode_lse(self, q, k, v, n_q_head, n_kv_head, head_dim, kv_len, kv_stride, batch, scale, out, lse):
        _ck(self.lib.fl_b200_attn_decode_lse(self._h, _p(q), _p(k), _p(v), C.c_uint32(n_q_head), C.c_uint32(n_kv_head),
                                             C.c_uint32(head_dim), C.c_uint32(kv_len), C.c_uint32(kv_stride),
                                             C.c_uint32(batch), C.c_float(scale), _p(out), _p(lse)))

    def attn_verify(self, q, k, v, n_q_head, n_kv_head, head_dim, base_len, kv_stride, n_draft, scale, out):
        """Causal-within-draft attention: query b sees keys 0 .. base_len + b - 1 of one shared cache."""
        _ck(self.lib.fl_b200_attn_verify(self._h, _p(q), _p(k), _p(v), C.c_uint32(n_q_head), C.c_uint32(n_kv_head),
                                         C.c_uint32(head_dim), C.c_uint32(base_len), C.c_uint32(kv_stride),
                                         C.c_uint32(n_draft), C.c_float(scale), _p(out)))

    def attn_decode_static(self, q, k, v, n_q_head, n_kv_head, head_dim, kv_len, kv_stride, batch, scale, out):
        """attn_decode with its scratch in a fixed array of the library (no allocation at call time)."""
        _ck(self.lib.fl_b200_attn_decode_static(self._h, _p(q), _p(k), _p(v), C.c_uint32(n_q_head),
                                                C.c_uint32(n_kv_head), C.c_uint32(head_dim), C.c_uint32(kv_len),
                                                C.c_uint32(kv_stride), C.c_uint32(batch), C.c_float(scale), _p(out)))

    def attn_decode_host(self, q_host, k, v, n_q_head, n_kv_head, head_dim, kv_len, kv_stride, batch, scale,
                         out_host):
        _ck(self.lib.fl_b200_attn_decode_host(self._h, _hp(q_host), _p(k), _p(v), C.c_uint32(n_q_head),
                                              C.c_uint32(n_kv_head), C.c_uint32(head_dim), C.c_uint32(kv_len),
                                              C.c_uint32(kv_stride), C.c_uint32(batch), C.c_float(scale),
                                              _hp(out_host)))

    def rmsnorm(self, x, w, y, eps, n):
        _ck(self.lib.fl_b200_rmsnorm(self._h, _p(x), _p(w), _p(y), C.c_float(eps), C.c_uint32(n)))

    def add2(self, a, b, y, n):
        _ck(self.lib.fl_b200_add2(self._h, _p(a), _p(b), _p(y), C.c_uint32(n)))

    def silu_mul(self, g, u, h, n):
        _ck(self.lib.fl_b200_silu_mul(self._h, _p(g), _p(u), _p(h), C.c_uint32(n)))

    def rope_kv_append(self, q, k, v, kcache, vcache, pos, n_q_head, n_kv_head, head_dim, kv_stride, freq_base):
        _ck(self.lib.fl_b200_rope_kv_append(self._h, _p(q), _p(k), _p(v), _p(kcache), _p(vcache), _p(pos),
                                            C.c_uint32(n_q_head), C.c_uint32(n_kv_head), C.c_uint32(head_dim),
                                            C.c_uint32(kv_stride), C.c_float(freq_base)))

    def argmax(self, logits, n, idx, margin):
        _ck(self.lib.fl_b200_argmax(self._h, _p(logits), C.c_uint32(n), _p(idx), _p(margin)))

    def exec_task(self, task):
        _ck(self.lib.fl_b200_exec_task(self._h, C.byref(task)))


def _hp(a):
    """Host pointer of a numpy array or a CPU torch tensor."""
    if hasattr(a, "ctypes"):
        return C.c_void_p(a.ctypes.data)
    return C.c_void_p(a.data_ptr())
