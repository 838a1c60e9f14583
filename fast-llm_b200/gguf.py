"""GGUF model files: the binding of the library's reader (``fl_b200_gguf_*``, the
counterpart of class Gguf, src/model/gguf.h:28-79 of the reference) and a writer
for fixtures and synthetic models (the reference keeps its own in
tests/test_quants.cpp:131-182). The reader runs in the library; nothing here
parses a file.
"""
import ctypes as C
import struct

import numpy as np

from . import capi

GGML_F32, GGML_F16, GGML_Q5_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_IQ2_XXS, GGML_IQ3_XXS = 0, 1, 6, 8, 12, 14, 16, 18
GGML_OF_FMT = {capi.F32: GGML_F32, capi.Q8_0: GGML_Q8_0, capi.Q5_0: GGML_Q5_0, capi.Q4_K: GGML_Q4_K,
               capi.Q6_K: GGML_Q6_K}
# metadata value type ids
V_U8, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STR, V_ARR, V_U64, V_I64, V_F64 = range(13)
_SCALAR = {V_U8: "<B", V_I8: "<b", V_U16: "<H", V_I16: "<h", V_U32: "<I", V_I32: "<i", V_F32: "<f", V_BOOL: "<B",
           V_U64: "<Q", V_I64: "<q", V_F64: "<d"}


class TensorInfo(C.Structure):
    """Image of fl_b200_gguf_tensor."""
    _fields_ = [("fmt", C.c_int32), ("ggml_type", C.c_uint32), ("n_dims", C.c_uint32), ("shard", C.c_uint32),
                ("ne", C.c_uint64 * 4), ("offset", C.c_uint64), ("nbytes", C.c_uint64), ("data", C.c_void_p)]

    def bytes(self):
        """The payload, copied out of the mapping."""
        return C.string_at(self.data, self.nbytes)


class Gguf:
    """An open model file (all shards of a split one). Needs no GPU."""

    def __init__(self, path):
        self.lib = capi.load()
        self._h = C.c_void_p()
        capi._ck(self.lib.fl_b200_gguf_open(str(path).encode(), C.byref(self._h)))

    def close(self):
        if self._h:
            self.lib.fl_b200_gguf_close(self._h)
        self._h = C.c_void_p()

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def counts(self):
        """(tensors, shards, alignment of the file named)."""
        n, s, a = C.c_uint32(), C.c_uint32(), C.c_uint32()
        capi._ck(self.lib.fl_b200_gguf_counts(self._h, C.byref(n), C.byref(s), C.byref(a)))
        return n.value, s.value, a.value

    def tensor_at(self, i):
        name = C.create_string_buffer(256)
        info = TensorInfo()
        capi._ck(self.lib.fl_b200_gguf_tensor_at(self._h, C.c_uint32(i), name, C.c_size_t(256), C.byref(info)))
        return name.value.decode(), info

    def tensors(self):
        return [self.tensor_at(i) for i in range(self.counts()[0])]

    def find(self, name):
        info = TensorInfo()
        capi._ck(self.lib.fl_b200_gguf_find(self._h, name.encode(), C.byref(info)))
        return info

    def has(self, key):
        return bool(self.lib.fl_b200_gguf_has(self._h, key.encode()))

    def kv_i(self, key, dflt=0):
        return self.lib.fl_b200_gguf_kv_i(self._h, key.encode(), C.c_int64(dflt))

    def kv_f(self, key, dflt=0.0):
        return self.lib.fl_b200_gguf_kv_f(self._h, key.encode(), C.c_double(dflt))

    def kv_s(self, key, dflt=""):
        n = C.c_size_t()
        capi._ck(self.lib.fl_b200_gguf_kv_s(self._h, key.encode(), dflt.encode(), None, C.c_size_t(0), C.byref(n)))
        buf = C.create_string_buffer(n.value + 1)
        capi._ck(self.lib.fl_b200_gguf_kv_s(self._h, key.encode(), dflt.encode(), buf, C.c_size_t(n.value + 1), None))
        return buf.raw[:n.value].decode()

    def kv_sarr(self, key):
        """The string array under `key`, or None."""
        n = self.lib.fl_b200_gguf_kv_sarr_count(self._h, key.encode())
        if n < 0:
            return None
        out = []
        for i in range(n):
            ln = C.c_size_t()
            capi._ck(self.lib.fl_b200_gguf_kv_sarr_at(self._h, key.encode(), C.c_uint64(i), None, C.c_size_t(0), C.byref(ln)))
            buf = C.create_string_buffer(ln.value + 1)
            capi._ck(self.lib.fl_b200_gguf_kv_sarr_at(self._h, key.encode(), C.c_uint64(i), buf, C.c_size_t(ln.value + 1), None))
            out.append(buf.raw[:ln.value].decode())
        return out

    def llama_cfg(self, max_kv):
        cfg = capi.LlamaCfg()
        capi._ck(self.lib.fl_b200_gguf_llama_cfg(self._h, C.c_uint32(max_kv), C.byref(cfg)))
        return cfg


# ---- writer ----

def _str(s):
    b = s.encode() if isinstance(s, str) else bytes(s)
    return struct.pack("<Q", len(b)) + b


def _value(vtype, v):
    if vtype == V_STR:
        return _str(v)
    if vtype == V_ARR:
        etype, items = v
        return struct.pack("<IQ", etype, len(items)) + b"".join(_value(etype, x) for x in items)
    return struct.pack(_SCALAR[vtype], v)


def write_gguf(path, kv, tensors, alignment=None, version=3):
    """Writes one GGUF file. `kv`: list of (key, value type id, value), an array value being
    (element type id, items). `tensors`: list of (name, ggml type id, dims innermost first,
    payload bytes). `alignment`: written as general.alignment when given (32 otherwise applies)."""
    kv = list(kv)
    if alignment is not None:
        kv.append(("general.alignment", V_U32, alignment))
    align = alignment or 32
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv))
    for key, vtype, v in kv:
        head += _str(key) + struct.pack("<I", vtype) + _value(vtype, v)
    off, offsets = 0, []
    for name, gtype, dims, payload in tensors:
        off = (off + align - 1) // align * align
        offsets.append(off)
        head += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", gtype, off)
        off += len(payload)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (-len(head) % align))
        pos = 0
        for (name, gtype, dims, payload), o in zip(tensors, offsets):
            f.write(b"\0" * (o - pos))
            f.write(payload)
            pos = o + len(payload)


LAYER_TENSORS = (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"), ("gate", "ffn_gate"),
                 ("up", "ffn_up"), ("down", "ffn_down"))


def llama_records(cfg, model, tie_output=False):
    """(metadata, tensor records) of a "llama" file for a model in the layout of
    synth.host_llama: model["layers"][l][name] = (fmt, packed rows as a uint8 array), plus
    "attn_norm" / "ffn_norm" f32 arrays; model["tok_embd"], model["output"] likewise,
    model["out_norm"]."""
    kv = [("general.architecture", V_STR, "llama"), ("general.name", V_STR, "synthetic"),
          ("llama.block_count", V_U32, cfg["n_layer"]), ("llama.embedding_length", V_U32, cfg["n_embd"]),
          ("llama.attention.head_count", V_U32, cfg["n_head"]),
          ("llama.attention.head_count_kv", V_U32, cfg["n_kv_head"]),
          ("llama.feed_forward_length", V_U32, cfg["n_ff"]),
          ("llama.attention.layer_norm_rms_epsilon", V_F32, cfg.get("eps", 1e-5)),
          ("llama.rope.freq_base", V_F32, cfg.get("rope_base", 500000.0)),
          ("llama.rope.dimension_count", V_U32, cfg["head_dim"]),
          ("llama.vocab_size", V_U32, cfg["n_vocab"])]

    def mat(name, t):
        fmt, w = t
        w = np.ascontiguousarray(w)
        cols = w.shape[1] // capi.BLK_BYTES[fmt] * capi.BLK_ELEMS[fmt]
        return (name, GGML_OF_FMT[fmt], [cols, w.shape[0]], w.tobytes())

    def vec(name, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        return (name, GGML_F32, [a.size], a.tobytes())

    recs = [mat("token_embd.weight", model["tok_embd"])]
    for l, L in enumerate(model["layers"]):
        recs.append(vec("blk.%d.attn_norm.weight" % l, L["attn_norm"]))
        for key, gname in LAYER_TENSORS:
            recs.append(mat("blk.%d.%s.weight" % (l, gname), L[key]))
        recs.append(vec("blk.%d.ffn_norm.weight" % l, L["ffn_norm"]))
    recs.append(vec("output_norm.weight", model["out_norm"]))
    if not tie_output:
        recs.append(mat("output.weight", model["output"]))
    return kv, recs


def write_llama_gguf(path, cfg, model, tie_output=False, alignment=None):
    kv, recs = llama_records(cfg, model, tie_output)
    write_gguf(path, kv, recs, alignment=alignment)


def write_split(pattern_stem, kv, tensors, parts, alignment=None):
    """Writes `parts` shards "<stem>-0000i-of-0000N.gguf": all metadata in shard 1 (plus
    split.* keys in every shard), the tensors dealt out in order from shard 2 on when
    parts > 1 (shard 1 then holds none, as large published models do). Returns the paths."""
    paths = ["%s-%05d-of-%05d.gguf" % (pattern_stem, i + 1, parts) for i in range(parts)]
    holders = max(parts - 1, 1)
    per = (len(tensors) + holders - 1) // holders
    for i, p in enumerate(paths):
        mine = tensors if parts == 1 else ([] if i == 0 else tensors[(i - 1) * per:i * per])
        meta = (list(kv) if i == 0 else []) + [("split.no", V_U16, i), ("split.count", V_U16, parts),
                                                ("split.tensors.count", V_I32, len(tensors))]
        write_gguf(p, meta, mine, alignment=alignment)
    return paths
