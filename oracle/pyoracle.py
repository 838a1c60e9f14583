"""Test infrastructure, not product code: ctypes access to the two CPU oracles.

  port       oracle/liboracle.so        plain-C restatement (oracle.c) + the
                                         Llama-step driver (llama_oracle.c)
  reference  oracle/_ref/libflref.so    the reference's own operators, compiled
                                         from the reference sources by
                                         oracle/Makefile

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``
import this module. The libraries are built on demand with ``make`` (gcc is part
of the image on both the build box and the GPU box); the reference one only
where the reference checkout is present, otherwise a prebuilt copy is used if
it travelled with the tree.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_LIB = os.path.join(HERE, "liboracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libflref.so")
# the same reference sources at -O3 -march=x86-64-v3 (AVX2 + FMA): a timed CPU baseline, never a checker
REF_O3_LIB = os.path.join(HERE, "_ref", "libflref_o3.so")
# the reference checkout: FLB_REFERENCE, else a directory named "reference" beside this repository
REF_SRC = os.environ.get("FLB_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

F32, Q8_0, Q5_0, Q4_K, Q6_K = 0, 1, 2, 3, 4
T_WQ, T_WK, T_WV, T_WO, T_GATE, T_UP, T_DOWN = range(7)
G_TOK_EMBD, G_OUTPUT = 0, 1


def _newer(a, b):
    return os.path.exists(a) and (not os.path.exists(b) or os.path.getmtime(a) > os.path.getmtime(b))


def host_has_avx2_fma():
    """True when this host's cores can run the x86-64-v3 build (libflref_o3.so)."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    return {"avx2", "fma", "bmi2", "f16c"} <= flags
    except OSError:
        pass
    return False


def build(which="all"):
    """Builds what is missing or stale. Returns (port_ok, ref_ok)."""
    srcs = [os.path.join(HERE, f) for f in ("oracle.c", "llama_oracle.c", "flo_ops.h")]
    if which in ("all", "port") and any(_newer(s, PORT_LIB) for s in srcs):
        subprocess.run(["make", "-C", HERE, "port"], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if which in ("all", "ref") and os.path.isdir(os.path.join(REF_SRC, "src", "runtime")):
        shim = [os.path.join(HERE, f) for f in ("ref_shim.cpp", "flo_ops.h", "abi_check.cpp")]
        if any(_newer(s, REF_LIB) for s in shim):
            subprocess.run(["make", "-C", HERE, "ref", "REF=" + REF_SRC], check=True, stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT)
        if any(_newer(s, REF_O3_LIB) for s in shim):
            subprocess.run(["make", "-C", HERE, "ref_o3", "REF=" + REF_SRC], check=True, stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT)
    return os.path.exists(PORT_LIB), os.path.exists(REF_LIB)


class LlamaCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim", "n_ff", "n_vocab", "max_kv")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)]


class Ops(C.Structure):
    _fields_ = [
        ("name", C.c_char_p),
        ("h2f", C.CFUNCTYPE(C.c_float, C.c_uint16)),
        ("f2h", C.CFUNCTYPE(C.c_uint16, C.c_float)),
        ("dequant", C.CFUNCTYPE(None, C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p)),
        ("stream_dot", C.CFUNCTYPE(None, C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32,
                                   C.c_uint32, C.c_void_p, C.c_uint32)),
        ("rmsnorm", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_uint32)),
        ("add2", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32)),
        ("rope", C.CFUNCTYPE(None, C.c_void_p, C.c_int32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float)),
        ("kv_append", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_uint32)),
        ("attn_head", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                  C.c_float, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32)),
        ("silu_mul", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32)),
        ("router_sel", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                   C.c_float)),
        ("wmerge", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                               C.c_uint32, C.c_uint32)),
    ]


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


class Oracle:
    """One of the two oracles, through the shared operator table."""

    def __init__(self, kind="port", ref_lib=None):
        """ref_lib: another build of the reference library (REF_O3_LIB) for kind == "reference"."""
        build()
        if not os.path.exists(PORT_LIB):
            raise RuntimeError("oracle/liboracle.so could not be built")
        self.port = C.CDLL(PORT_LIB)
        self.kind = kind
        if kind == "port":
            self.port.flo_port_ops.restype = C.POINTER(Ops)
            self.ops = self.port.flo_port_ops()
            self.ref = None
        elif kind == "reference":
            lib = ref_lib or REF_LIB
            if not os.path.exists(lib):
                raise RuntimeError("%s is not available (no reference checkout, no prebuilt copy)" % os.path.relpath(lib, HERE))
            self.ref = C.CDLL(lib)
            self.ref.flref_ops.restype = C.POINTER(Ops)
            self.ops = self.ref.flref_ops()
            self.ref.flref_dot_row.restype = C.c_float
            self.ref.flref_dot_row_fast.restype = C.c_float
            self.ref.flref_stream_dot_tasks.restype = C.c_uint64
        else:
            raise ValueError(kind)
        self.o = self.ops.contents
        p = self.port
        p.flo_row_bytes.restype = C.c_uint64
        p.flo_llama_create.restype = C.c_void_p
        p.flo_llama_step.restype = C.c_int32
        p.flo_llama_n_past.restype = C.c_int32
        p.flo_llama_logits.restype = C.POINTER(C.c_float)
        p.flo_llama_hidden.restype = C.POINTER(C.c_float)
        p.flo_llama_normed.restype = C.POINTER(C.c_float)
        p.flo_llama_margin.restype = C.c_float
        p.flo_llama_tap.restype = C.POINTER(C.c_float)
        p.flo_llama_moe_ids.restype = C.POINTER(C.c_uint32)

    @staticmethod
    def available(kind):
        build()
        return os.path.exists(PORT_LIB if kind == "port" else REF_LIB)

    # ---- scalar helpers ----
    def h2f(self, h):
        return self.o.h2f(int(h))

    def f2h(self, f):
        return self.o.f2h(float(f))

    def row_bytes(self, fmt, cols):
        return self.port.flo_row_bytes(fmt, C.c_uint32(cols))

    # ---- tensor-level ----
    def dequant(self, fmt, w, rows, cols):
        """Bulk dequantise (rows in parallel). w: uint8 array of packed rows."""
        w = np.ascontiguousarray(w, dtype=np.uint8)
        out = np.empty((rows, cols), dtype=np.float32)
        self.port.flo_dequant_rows(self.ops, fmt, _ptr(w), C.c_uint32(rows), C.c_uint32(cols), _ptr(out))
        return out

    def matvec(self, fmt, w, rows, cols, x):
        """y = W x through zeroed slots + STREAM_DOT tiles of 192 rows (multi-threaded, bit-exact)."""
        w = np.ascontiguousarray(w, dtype=np.uint8)
        x = _f32(x)
        y = np.empty(rows, dtype=np.float32)
        self.port.flo_matvec(self.ops, fmt, _ptr(w), C.c_uint32(rows), C.c_uint32(cols), _ptr(x), _ptr(y))
        return y

    def stream_dot(self, fmt, w, rows, cols, x, y, nx=1, xstride=0, ystride=0):
        """One STREAM_DOT tile, in place: y[p*ystride + r] += W[r] . x[p]."""
        w = np.ascontiguousarray(w, dtype=np.uint8)
        self.o.stream_dot(fmt, _ptr(w), rows, cols, _ptr(x), nx, xstride, _ptr(y), ystride)

    def rmsnorm(self, wnorm, x, eps):
        x = _f32(x); wnorm = _f32(wnorm)
        y = np.empty_like(x)
        self.o.rmsnorm(_ptr(wnorm), _ptr(x), _ptr(y), eps, x.size)
        return y

    def add2(self, a, b):
        a = _f32(a); b = _f32(b)
        y = np.empty_like(a)
        self.o.add2(_ptr(a), _ptr(b), _ptr(y), a.size)
        return y

    def silu_mul(self, g, u):
        g = _f32(g); u = _f32(u)
        h = np.empty_like(g)
        self.o.silu_mul(_ptr(g), _ptr(u), _ptr(h), g.size)
        return h

    def rope(self, buf, pos, n_head, head_stride, rot_off, n_rot, freq_base):
        out = _f32(buf).copy()
        self.o.rope(_ptr(out), pos, n_head, head_stride, rot_off, n_rot, freq_base)
        return out

    def router_sel(self, logits, top_k, norm, scale):
        logits = _f32(logits)
        ids = np.zeros(top_k, dtype=np.uint32)
        gates = np.zeros(top_k, dtype=np.float32)
        self.o.router_sel(_ptr(logits), _ptr(ids), _ptr(gates), logits.size, top_k, norm, scale)
        return ids, gates

    def wmerge(self, parts, gates, add1, add2, scale):
        parts = _f32(parts)
        n_parts, n = parts.shape
        y = np.empty(n, dtype=np.float32)
        g = None if gates is None else _f32(gates)
        a1 = None if add1 is None else _f32(add1)
        a2 = None if add2 is None else _f32(add2)
        self.o.wmerge(_ptr(parts), _ptr(g), _ptr(a1), _ptr(a2), _ptr(y), scale, n_parts, n)
        return y

    def attn_head_f32(self, q, kc, vc, pos, scale, head, n_head, dk, dv):
        """The one-head operator on an f32 cache [kv][n_head][d] (reference layout)."""
        q = _f32(q); kc = _f32(kc); vc = _f32(vc)
        max_kv = kc.shape[0]
        scratch = np.zeros(max_kv, dtype=np.float32)
        out = np.zeros(n_head * dv, dtype=np.float32)
        self.o.attn_head(_ptr(q), _ptr(kc), _ptr(vc), _ptr(scratch), _ptr(out), pos, scale, head, n_head, dk, dv,
                         max_kv)
        return out[head * dv:(head + 1) * dv].copy()

    def attn_gqa_f16(self, q, k16, v16, kv_len, scale):
        """q [n_head][d] f32; k16, v16 [n_kv_head][kv_stride][d] f16 -> out [n_head][d]."""
        q = _f32(q)
        k16 = np.ascontiguousarray(k16).view(np.uint16)
        v16 = np.ascontiguousarray(v16).view(np.uint16)
        n_head, d = q.shape
        n_kv, stride, _ = k16.shape
        out = np.zeros((n_head, d), dtype=np.float32)
        self.port.flo_attn_gqa_f16(self.ops, _ptr(q), _ptr(k16), _ptr(v16), C.c_uint64(stride), C.c_uint32(kv_len),
                                   C.c_float(scale), C.c_uint32(n_head), C.c_uint32(n_kv), C.c_uint32(d), _ptr(out))
        return out

    # ---- reference-only extras ----
    def ref_dot_row(self, fmt, row, x, fast=False):
        row = np.ascontiguousarray(row, dtype=np.uint8); x = _f32(x)
        f = self.ref.flref_dot_row_fast if fast else self.ref.flref_dot_row
        return f(fmt, _ptr(row), _ptr(x), C.c_uint32(x.size))

    def ref_stream_dot_tasks(self, fmt, w, rows, cols, x, threads, fast=False, rowsz=192):
        """y = W x through the reference's task graph (run_serial if threads <= 0,
        else its CPU worker pool). Returns (y, wall_ns of the run)."""
        w = np.ascontiguousarray(w, dtype=np.uint8); x = _f32(x)
        y = np.zeros(rows, dtype=np.float32)
        ns = self.ref.flref_stream_dot_tasks(fmt, _ptr(w), C.c_uint32(rows), C.c_uint32(cols), _ptr(x), 1, 0, _ptr(y),
                                             0, C.c_uint32(rowsz), C.c_int(threads), C.c_int(1 if fast else 0))
        return y, ns

    def ref_pool_shutdown(self):
        if self.ref is not None:
            self.ref.flref_pool_shutdown()


class LlamaOracle:
    """The Llama-step driver (llama_oracle.c) on one operator table."""

    def __init__(self, oracle, cfg):
        self.orc = oracle
        self.p = oracle.port
        self.cfg = dict(cfg)
        c = LlamaCfg(**{k: cfg[k] for k in ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim", "n_ff", "n_vocab",
                                            "max_kv", "rope_base", "eps")})
        self.h = C.c_void_p(self.p.flo_llama_create(C.byref(c)))
        self._keep = []

    def close(self):
        if self.h:
            self.p.flo_llama_destroy(self.h)
            self.h = None

    def set_layer_tensor(self, layer, which, fmt, w):
        w = np.ascontiguousarray(w, dtype=np.uint8)
        self._keep.append(w)
        self.p.flo_llama_set_layer_tensor(self.h, C.c_uint32(layer), which, fmt, _ptr(w))

    def set_layer_norms(self, layer, an, fn):
        an = _f32(an); fn = _f32(fn)
        self._keep += [an, fn]
        if layer == 0:
            self._attn_norm0 = an   # the live array the C side reads (one_ulp_move)
        self.p.flo_llama_set_layer_norms(self.h, C.c_uint32(layer), _ptr(an), _ptr(fn))

    def set_layer_moe(self, layer, n_expert, top_k, norm, scale, n_ff, router, fmt_gu, wg, wu, fmt_d, wd):
        """A mixture-of-experts feed-forward block in place of the layer's dense one (experts stacked row-wise)."""
        router = _f32(router)
        wg, wu, wd = (np.ascontiguousarray(a, dtype=np.uint8) for a in (wg, wu, wd))
        self._keep += [router, wg, wu, wd]
        self.p.flo_llama_set_layer_moe(self.h, C.c_uint32(layer), C.c_uint32(n_expert), C.c_uint32(top_k), C.c_uint32(norm),
                                       C.c_float(scale), C.c_uint32(n_ff), _ptr(router), fmt_gu, _ptr(wg), _ptr(wu), fmt_d, _ptr(wd))

    def set_global(self, which, fmt, w):
        w = np.ascontiguousarray(w, dtype=np.uint8)
        self._keep.append(w)
        self.p.flo_llama_set_global(self.h, which, fmt, _ptr(w))

    def set_out_norm(self, w):
        w = _f32(w)
        self._keep.append(w)
        self.p.flo_llama_set_out_norm(self.h, _ptr(w))

    def seed_kv(self, layer, k16, v16):
        k16 = np.ascontiguousarray(k16).view(np.uint16); v16 = np.ascontiguousarray(v16).view(np.uint16)
        n_pos = k16.shape[1]
        self.p.flo_llama_seed_kv(self.h, self.orc.ops, C.c_uint32(layer), _ptr(k16), _ptr(v16), C.c_uint32(n_pos),
                                 C.c_uint64(n_pos))

    def set_n_past(self, n):
        self.p.flo_llama_set_n_past(self.h, C.c_int32(n))

    def n_past(self):
        return self.p.flo_llama_n_past(self.h)

    def step(self, token):
        return self.p.flo_llama_step(self.h, self.orc.ops, C.c_int32(int(token)))

    def logits(self):
        return np.ctypeslib.as_array(self.p.flo_llama_logits(self.h), shape=(self.cfg["n_vocab"],)).copy()

    def one_ulp_move(self, token):
        """Conditioning of the step just taken (call right after step(token)): the step is repeated with every
        attn_norm weight of layer 0 one f32 ulp larger, then once more unperturbed (which restores the K/V rows
        and every tap). Returns max |logits' - logits| / RMS(logits): how far the ORACLE's own result moves for
        the smallest possible change of one input."""
        pos = self.n_past() - 1
        base = self.logits()
        an = self._attn_norm0
        keep = an.copy()
        an[:] = np.nextafter(an, np.float32(4.0))
        self.set_n_past(pos)
        self.step(token)
        moved = self.logits()
        an[:] = keep
        self.set_n_past(pos)
        self.step(token)
        assert np.array_equal(self.logits(), base)
        return float(np.max(np.abs(moved - base)) / (np.sqrt(np.mean(base.astype(np.float64) ** 2)) + 1e-30))

    def hidden(self):
        return np.ctypeslib.as_array(self.p.flo_llama_hidden(self.h), shape=(self.cfg["n_embd"],)).copy()

    def normed(self):
        return np.ctypeslib.as_array(self.p.flo_llama_normed(self.h), shape=(self.cfg["n_embd"],)).copy()

    def margin(self):
        return self.p.flo_llama_margin(self.h)

    def tap(self, which):
        c = self.cfg
        n = {0: c["n_embd"], 1: c["n_embd"], 2: c["n_head"] * c["head_dim"], 3: c["n_kv_head"] * c["head_dim"],
             4: c["n_head"] * c["head_dim"], 5: c["n_embd"], 6: c["n_ff"], 7: c["n_ff"]}[which]
        return np.ctypeslib.as_array(self.p.flo_llama_tap(self.h, which), shape=(n,)).copy()

    def kv_row(self, layer, pos):
        n = self.cfg["n_kv_head"] * self.cfg["head_dim"]
        k = np.zeros(n, dtype=np.uint16); v = np.zeros(n, dtype=np.uint16)
        self.p.flo_llama_get_kv_row(self.h, self.orc.ops, C.c_uint32(layer), C.c_uint32(pos), _ptr(k), _ptr(v))
        return k.view(np.float16), v.view(np.float16)
