"""CPU tests of the library's GGUF reader: against the reference's own reader
(class Gguf of the reference, compiled into oracle/_ref) on the same files, on
the fixture shape the reference's test writes (tests/test_quants.cpp:141-206),
and on the malformed files the reference aborts on. No GPU is used."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from fast_llm_b200 import capi, gguf, synth

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "..", "oracle", "_ref", "libflref.so")

SMALL = dict(n_layer=2, n_embd=512, n_head=4, n_kv_head=1, head_dim=128, n_ff=768, n_vocab=40, max_kv=32,
             rope_base=500000.0, eps=1e-5)


def small_model(cfg, seed, recipe=synth.Q4_K_M):
    layers = []
    for l in range(cfg["n_layer"]):
        L = {n: (recipe[n], synth.llama_tensor(cfg, seed, n, l, recipe)) for n in synth.LAYER_TENSORS}
        L["attn_norm"] = synth.llama_norm(cfg, seed, "attn_norm", l)
        L["ffn_norm"] = synth.llama_norm(cfg, seed, "ffn_norm", l)
        layers.append(L)
    return dict(layers=layers, tok_embd=(recipe["tok_embd"], synth.llama_tensor(cfg, seed, "tok_embd", None, recipe)),
                output=(recipe["output"], synth.llama_tensor(cfg, seed, "output", None, recipe)),
                out_norm=synth.llama_norm(cfg, seed, "out_norm"))


def fixture_records(seed=77):
    """The five tensors of the reference's reader test: one per format it maps."""
    rng = np.random.default_rng(seed)
    specs = [("t.q8", capi.Q8_0, 64, 3), ("t.q50", capi.Q5_0, 64, 2), ("t.q4k", capi.Q4_K, 256, 2),
             ("t.q6k", capi.Q6_K, 256, 1), ("t.f32", capi.F32, 16, 4)]
    recs = []
    for name, fmt, ne0, ne1 in specs:
        payload = rng.integers(0, 256, ne1 * capi.row_bytes(fmt, ne0), dtype=np.uint8).tobytes()
        recs.append((name, gguf.GGML_OF_FMT[fmt], [ne0, ne1], payload))
    return recs


RICH_KV = [
    ("general.architecture", gguf.V_STR, "llama"),
    ("a.u8", gguf.V_U8, 200), ("a.i8", gguf.V_I8, -100), ("a.u16", gguf.V_U16, 60000), ("a.i16", gguf.V_I16, -30000),
    ("a.u32", gguf.V_U32, 4000000000), ("a.i32", gguf.V_I32, -2000000000), ("a.u64", gguf.V_U64, 2 ** 40 + 7),
    ("a.i64", gguf.V_I64, -(2 ** 41)), ("a.f32", gguf.V_F32, 0.15625), ("a.f64", gguf.V_F64, 1e-9), ("a.true", gguf.V_BOOL, 1),
    ("a.false", gguf.V_BOOL, 0), ("a.empty", gguf.V_STR, ""),
    ("tokenizer.ggml.tokens", gguf.V_ARR, (gguf.V_STR, ["<s>", "", "hello", "wörld"])),
    ("tokenizer.ggml.scores", gguf.V_ARR, (gguf.V_F32, [0.0, -1.5, 2.25])),
    ("tokenizer.ggml.token_type", gguf.V_ARR, (gguf.V_I32, [1, 2, 3, 4])),
    ("nested", gguf.V_ARR, (gguf.V_ARR, [(gguf.V_U8, [1, 2, 3]), (gguf.V_STR, ["x", "yy"])])),
]
KEYS_I = ["a.u8", "a.i8", "a.u16", "a.i16", "a.u32", "a.i32", "a.u64", "a.i64", "a.f32", "a.true", "a.false", "absent",
          "general.alignment"]
KEYS_S = ["general.architecture", "a.empty", "a.u8", "absent"]
KEYS_SA = ["tokenizer.ggml.tokens", "tokenizer.ggml.scores", "nested", "absent"]


class RefGguf:
    """The reference's reader through oracle/_ref."""

    def __init__(self, path):
        self.lib = C.CDLL(REF_LIB)
        self.lib.flref_gguf_open.restype = C.c_void_p
        self.lib.flref_gguf_kv_i.restype = C.c_int64
        self.lib.flref_gguf_kv_f.restype = C.c_double
        self.lib.flref_gguf_find.restype = C.c_int64
        self.lib.flref_gguf_kv_sarr_count.restype = C.c_int64
        self.lib.flref_gguf_kv_s.restype = C.c_size_t
        self.lib.flref_gguf_kv_sarr_at.restype = C.c_size_t
        self.h = C.c_void_p(self.lib.flref_gguf_open(str(path).encode()))

    def close(self):
        if self.h:
            self.lib.flref_gguf_close(self.h)
        self.h = C.c_void_p()

    def counts(self):
        n, s, a = C.c_uint32(), C.c_uint32(), C.c_uint32()
        self.lib.flref_gguf_counts(self.h, C.byref(n), C.byref(s), C.byref(a))
        return n.value, s.value, a.value

    def tensor(self, i):
        name = C.create_string_buffer(256)
        typ, nd, sh, fmt = C.c_uint32(), C.c_int32(), C.c_int32(), C.c_int32()
        ne = (C.c_uint64 * 4)()
        off, nb = C.c_uint64(), C.c_uint64()
        data = C.c_void_p()
        self.lib.flref_gguf_tensor(self.h, C.c_uint32(i), name, C.c_size_t(256), C.byref(typ), C.byref(nd), ne,
                                   C.byref(off), C.byref(nb), C.byref(sh), C.byref(fmt), C.byref(data))
        return dict(name=name.value.decode(), type=typ.value, n_dims=nd.value, ne=list(ne), offset=off.value,
                    nbytes=nb.value, shard=sh.value, fmt=fmt.value, bytes=C.string_at(data.value, nb.value))

    def kv_s(self, key, dflt=""):
        buf = C.create_string_buffer(4096)
        n = self.lib.flref_gguf_kv_s(self.h, key.encode(), dflt.encode(), buf, C.c_size_t(4096))
        return buf.raw[:n].decode()

    def kv_sarr(self, key):
        n = self.lib.flref_gguf_kv_sarr_count(self.h, key.encode())
        if n < 0:
            return None
        out = []
        for i in range(n):
            buf = C.create_string_buffer(4096)
            ln = self.lib.flref_gguf_kv_sarr_at(self.h, key.encode(), C.c_uint64(i), buf, C.c_size_t(4096))
            out.append(buf.raw[:ln].decode())
        return out


def assert_same_view(path, names_to_find):
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref is not built")
    ref = RefGguf(path)
    assert ref.h
    with gguf.Gguf(path) as g:
        assert g.counts() == ref.counts()
        for i in range(g.counts()[0]):
            name, info = g.tensor_at(i)
            want = ref.tensor(i)
            got = dict(name=name, type=info.ggml_type, n_dims=info.n_dims, ne=list(info.ne), offset=info.offset,
                       nbytes=info.nbytes, shard=info.shard, fmt=info.fmt, bytes=info.bytes())
            assert got == want, (i, name)
        for nm in names_to_find:
            idx = ref.lib.flref_gguf_find(ref.h, nm.encode())
            if idx < 0:
                with pytest.raises(capi.Fl200Error):
                    g.find(nm)
            else:
                assert g.find(nm).offset == ref.tensor(idx)["offset"] and g.find(nm).shard == ref.tensor(idx)["shard"]
        for k in KEYS_I + KEYS_S + KEYS_SA + ["a.f64", "split.count", "split.no", "split.tensors.count"]:
            assert g.has(k) == bool(ref.lib.flref_gguf_has(ref.h, k.encode())), k
            assert g.kv_i(k, -5) == ref.lib.flref_gguf_kv_i(ref.h, k.encode(), C.c_int64(-5)), k
            assert g.kv_f(k, 2.5) == ref.lib.flref_gguf_kv_f(ref.h, k.encode(), C.c_double(2.5)), k
            assert g.kv_s(k, "dflt") == ref.kv_s(k, "dflt"), k
            assert g.kv_sarr(k) == ref.kv_sarr(k), k
    ref.close()


@pytest.mark.parametrize("version,alignment", [(3, None), (3, 32), (2, 64), (3, 256)])
def test_reader_equals_reference_reader(tmp_path, version, alignment):
    path = tmp_path / "rich.gguf"
    recs = fixture_records() + [("t.f16", gguf.GGML_F16, [8, 3], bytes(48)), ("t.unknown", 2, [32, 2], b""),
                                ("t.3d", gguf.GGML_Q4_K, [256, 2, 3], bytes(144 * 6)), ("t.vec", gguf.GGML_F32, [5], bytes(20)),
                                ("t.q4k", gguf.GGML_F32, [1], bytes(4))]   # a second tensor of a name already used
    gguf.write_gguf(path, RICH_KV, recs, alignment=alignment, version=version)
    assert_same_view(path, [r[0] for r in recs] + ["nope"])


def test_split_model_equals_reference_reader(tmp_path):
    recs = fixture_records()
    paths = gguf.write_split(str(tmp_path / "model"), RICH_KV, recs, parts=3, alignment=64)
    assert_same_view(paths[0], [r[0] for r in recs])
    with gguf.Gguf(paths[0]) as g:
        assert g.counts() == (5, 3, 64)
        assert g.kv_i("split.no", -1) == 0           # metadata of the shard named, not of the last one read
        assert [g.tensor_at(i)[1].shard for i in range(5)] == [1, 1, 1, 2, 2]
    # naming the second shard takes ITS metadata (which lacks the model's keys) and still maps all tensors
    assert_same_view(paths[1], [r[0] for r in recs])
    # a shard count the file names do not bear out
    os.remove(paths[2])
    with pytest.raises(capi.Fl200Error) as e:
        gguf.Gguf(paths[0])
    assert e.value.code == 5


def test_reference_fixture_shape(tmp_path):
    """What the reference's own reader test asserts (tests/test_quants.cpp:186-205)."""
    recs = fixture_records()
    path = tmp_path / "fixture.gguf"
    gguf.write_gguf(path, [], recs, alignment=32)
    with gguf.Gguf(path) as g:
        assert g.counts() == (5, 1, 32)
        for name, gtype, dims, payload in recs:
            t = g.find(name)
            assert t.ggml_type == gtype and list(t.ne)[:2] == dims and t.nbytes == len(payload)
            assert t.bytes() == payload
            assert t.fmt == {v: k for k, v in gguf.GGML_OF_FMT.items()}[gtype]


def test_malformed_files_return_a_status(tmp_path):
    good = tmp_path / "good.gguf"
    gguf.write_gguf(good, RICH_KV, fixture_records())
    blob = good.read_bytes()

    def code_of(data, name="bad.gguf"):
        p = tmp_path / name
        p.write_bytes(data)
        with pytest.raises(capi.Fl200Error) as e:
            gguf.Gguf(p)
        return e.value.code

    with pytest.raises(capi.Fl200Error) as e:
        gguf.Gguf(tmp_path / "missing.gguf")
    assert e.value.code == 5
    assert code_of(b"") == 5                                               # nothing to map
    assert code_of(b"GGUX" + blob[4:]) == 6                                # magic
    assert code_of(blob[:4] + struct.pack("<I", 1) + blob[8:]) == 6        # version 1
    assert code_of(blob[:4] + struct.pack("<I", 4) + blob[8:]) == 6
    with gguf.Gguf(good) as g:
        data_off = len(blob) - max(t.offset + t.nbytes for _, t in g.tensors())
    for cut in list(range(0, 64, 3)) + list(range(64, data_off, 17)) + [len(blob) - 1]:
        assert code_of(blob[:cut]) in (5, 6), cut                          # truncated anywhere: never a crash
    assert code_of(blob[:8] + struct.pack("<Q", 2 ** 60) + blob[16:]) == 6  # absurd tensor count
    assert code_of(blob[:16] + struct.pack("<Q", 2 ** 60) + blob[24:]) == 6  # absurd metadata count
    bad_type = bytearray()
    bad_type += struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 13)
    assert code_of(bytes(bad_type)) == 6                                   # value type 13 does not exist
    # arrays nested deeper than the reader follows (12 bytes per level: a few MB would otherwise overflow the stack)
    hdr = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 9)
    assert code_of(hdr + struct.pack("<IQ", 9, 1) * 400000 + struct.pack("<IQ", 4, 0)) == 6
    nested_ok = tmp_path / "nested_ok.gguf"                                # three levels are followed
    nested_ok.write_bytes(hdr + struct.pack("<IQ", 9, 1) * 2 + struct.pack("<IQ", 4, 2) + struct.pack("<II", 7, 8))
    with gguf.Gguf(nested_ok) as g:
        assert len(list(g.tensors())) == 0
    # dimensions whose byte size wraps around 64 bits must not pass the bounds check
    def one_tensor(ne, ggml_type=12):
        rec = struct.pack("<Q", 1) + b"t" + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", n) for n in ne)
        return struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + rec + struct.pack("<IQ", ggml_type, 0) + bytes(64)
    assert code_of(one_tensor([256, 2 ** 32, 2 ** 32])) == 6              # ne[1] * ne[2] wraps to 0
    assert code_of(one_tensor([256, 2 ** 62, 1, 1])) == 6                 # 144 * 2^62 wraps
    assert code_of(one_tensor([2 ** 32 + 256, 1])) == 6                   # a row longer than 32 bits of columns
    assert code_of(one_tensor([256, 2 ** 40])) == 6                       # honest but larger than the file
    p = tmp_path / "odd_align.gguf"
    gguf.write_gguf(p, [], [], alignment=48)
    with pytest.raises(capi.Fl200Error) as e:
        gguf.Gguf(p)
    assert e.value.code == 6


def test_llama_hyper_parameters(tmp_path):
    model = small_model(SMALL, seed=9)
    path = tmp_path / "llama.gguf"
    gguf.write_llama_gguf(path, SMALL, model)
    with gguf.Gguf(path) as g:
        c = g.llama_cfg(SMALL["max_kv"])
        for k in ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim", "n_ff", "n_vocab", "max_kv"):
            assert getattr(c, k) == SMALL[k], k
        assert c.rope_base == 500000.0 and abs(c.eps - 1e-5) < 1e-12
        t = g.find("blk.1.ffn_down.weight")
        assert t.fmt == capi.Q6_K and list(t.ne)[:2] == [SMALL["n_ff"], SMALL["n_embd"]]
        assert t.bytes() == model["layers"][1]["down"][1].tobytes()
    kv, recs = gguf.llama_records(SMALL, model)
    for bad_kv, extra in (
            ([(k, t, ("deepseek2" if k == "general.architecture" else v)) for k, t, v in kv], []),
            (kv + [("llama.rope.scaling.type", gguf.V_STR, "yarn")], []),
            (kv, [("rope_freqs.weight", gguf.GGML_F32, [64], bytes(256))]),
            ([x for x in kv if x[0] != "llama.block_count"], []),
            (kv + [("llama.attention.key_length", gguf.V_U32, 64)], [])):
        p = tmp_path / "bad_llama.gguf"
        gguf.write_gguf(p, bad_kv, recs + extra)
        with gguf.Gguf(p) as g, pytest.raises(capi.Fl200Error) as e:
            g.llama_cfg(16)
        assert e.value.code == 6
    # defaults: KV heads = heads, eps 1e-5, base 10000, head size = n_embd / n_head
    p = tmp_path / "defaults.gguf"
    keep = ("general.architecture", "llama.block_count", "llama.embedding_length", "llama.attention.head_count",
            "llama.feed_forward_length")
    gguf.write_gguf(p, [x for x in kv if x[0] in keep], recs)
    with gguf.Gguf(p) as g:
        c = g.llama_cfg(16)
        assert (c.n_kv_head, c.head_dim, c.rope_base) == (SMALL["n_head"], 128, 10000.0) and abs(c.eps - 1e-5) < 1e-12
