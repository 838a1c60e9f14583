"""CPU tests of the oracle itself: the plain-C port is pinned bit-for-bit to the
reference's own code (oracle/_ref, built from the reference sources), to the
reference's known-answer vectors, and to the committed golden fixtures."""
import os

import numpy as np
import pytest

from fast_llm_b200 import capi, synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_ops_golden.npz")
FMTS = [capi.Q8_0, capi.Q5_0, capi.Q4_K, capi.Q6_K]


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_f16_known_answers(port):
    # tests/test_runtime.cpp:540-544 of the reference
    kat = [(1.0, 0x3C00), (-2.0, 0xC000), (65504.0, 0x7BFF), (1e30, 0x7C00), (5.96e-8, 0x0001)]
    for f, h in kat:
        assert port.f2h(f) == h
    assert port.h2f(0x3C00) == 1.0 and port.h2f(0xC000) == -2.0 and port.h2f(0x7BFF) == 65504.0
    assert port.h2f(0x0001) == 2.0 ** -24


def test_f16_exhaustive_vs_reference(port, ref):
    for h in range(0, 65536):
        a, b = port.h2f(h), ref.h2f(h)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32) or (a != a and b != b)
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
                         np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 6.1e-5, 6.0e-5, 5.96e-8, 2.98e-8, 2.99e-8,
                                   np.inf, -np.inf], dtype=np.float32)]).astype(np.float32)
    for x in xs:
        assert port.f2h(x) == ref.f2h(x), x
    # round trip is the identity on every finite half
    for h in range(0, 0x7C00):
        assert port.f2h(port.h2f(h)) == h


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_and_dot_bitexact_vs_reference(port, ref, fmt):
    # shapes of the reference's own quant tests (tests/test_quants.cpp:292-295) plus block-count edge cases
    for seed, rows, cols in [(1, 3, 1408 if fmt in (capi.Q8_0, capi.Q5_0) else 2048), (2, 2, 2816 if fmt in (capi.Q8_0, capi.Q5_0) else 2816 // 256 * 256),
                             (3, 5, 256), (4, 1, 4096)]:
        rng = np.random.default_rng(seed)
        w = synth.quant_tensor(fmt, rng, rows, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        a, b = port.dequant(fmt, w, rows, cols), ref.dequant(fmt, w, rows, cols)
        assert np.array_equal(bits(a), bits(b))
        ya, yb = port.matvec(fmt, w, rows, cols, x), ref.matvec(fmt, w, rows, cols, x)
        assert np.array_equal(bits(ya), bits(yb))
        # the canonical dot is "dequantise, then dot ascending" in f32, one rounding per operation
        acc = np.zeros(rows, dtype=np.float32)
        for c in range(cols):
            acc = (acc + a[:, c] * x[c]).astype(np.float32)
        assert np.array_equal(bits(acc), bits(ya))
        # and it is close to the f64 value (the reference's own gate, tests/test_quants.cpp:82-107)
        y64 = a.astype(np.float64) @ x.astype(np.float64)
        assert np.all(np.abs(ya - y64) <= 1e-4 * (np.abs(y64) + 1))


def test_dequant_matches_independent_transcription(port):
    """Per-element formulas written directly from the block layout description."""
    rng = np.random.default_rng(11)
    w = synth.q4k_tensor(rng, 1, 512)[0]
    out = port.dequant(capi.Q4_K, w[None, :], 1, 512)[0]
    for e in rng.integers(0, 512, 64):
        b = w[(e // 256) * 144:(e // 256 + 1) * 144]
        d, dmin = b[0:2].view(np.float16)[0].astype(np.float32), b[2:4].view(np.float16)[0].astype(np.float32)
        i = e % 256
        j, l = i // 32, i % 32
        s = b[4:16]
        if j < 4:
            sc, mn = s[j] & 63, s[j + 4] & 63
        else:
            sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4)
            mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
        byte = b[16 + 32 * (j // 2) + l]
        q = (byte >> 4) if (j & 1) else (byte & 0xF)
        want = np.float32(np.float32(d * np.float32(sc)) * np.float32(q)) - np.float32(dmin * np.float32(mn))
        assert np.float32(want) == out[e]
    w = synth.q6k_tensor(rng, 1, 512)[0]
    out = port.dequant(capi.Q6_K, w[None, :], 1, 512)[0]
    for e in rng.integers(0, 512, 64):
        b = w[(e // 256) * 210:(e // 256 + 1) * 210]
        d = b[208:210].view(np.float16)[0].astype(np.float32)
        i = e % 256
        hf, g, l = i // 128, (i % 128) // 32, i % 32
        lo = b[64 * hf + 32 * (g & 1) + l]
        q4 = (lo & 0xF) if g < 2 else (lo >> 4)
        q = int(q4 | (((b[128 + 32 * hf + l] >> (2 * g)) & 3) << 4)) - 32
        sc = b[192:208].view(np.int8)[8 * hf + 2 * g + l // 16]
        want = np.float32(np.float32(d * np.float32(sc)) * np.float32(q))
        assert want == out[e]


def test_stream_dot_accumulates_and_multicolumn(port, ref):
    rng = np.random.default_rng(7)
    rows, cols, nx = 6, 512, 3
    w = synth.q4k_tensor(rng, rows, cols)
    x = rng.standard_normal((nx, cols)).astype(np.float32)
    for o in (port, ref):
        y = np.full((nx, rows), 0.5, dtype=np.float32)
        o.stream_dot(capi.Q4_K, w, rows, cols, x, y, nx=nx, xstride=cols, ystride=rows)
        for p in range(nx):
            single = o.matvec(capi.Q4_K, w, rows, cols, x[p])
            assert np.array_equal(bits(y[p]), bits((np.float32(0.5) + single).astype(np.float32)))


def test_small_ops_bitexact_vs_reference(port, ref):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(4096).astype(np.float32) * 3
    wn = rng.uniform(0.9, 1.1, 4096).astype(np.float32)
    assert np.array_equal(bits(port.rmsnorm(wn, x, 1e-5)), bits(ref.rmsnorm(wn, x, 1e-5)))
    y64 = x.astype(np.float64) / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5) * wn
    assert np.max(np.abs(port.rmsnorm(wn, x, 1e-5) - y64) / (np.abs(y64) + 1e-6)) < 1e-5
    u = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(bits(port.add2(x, u)), bits(ref.add2(x, u)))
    assert np.array_equal(bits(port.silu_mul(x, u)), bits(ref.silu_mul(x, u)))
    for pos in (0, 1, 17, 8191):
        buf = rng.standard_normal(8 * 128).astype(np.float32)
        a, b = port.rope(buf, pos, 8, 128, 0, 128, 500000.0), ref.rope(buf, pos, 8, 128, 0, 128, 500000.0)
        assert np.array_equal(bits(a), bits(b))
        if pos == 0:
            assert np.array_equal(bits(a), bits(buf))     # identity at position 0 (tests/test_decode_ops.cpp:37-82)
        pair = lambda z: z.reshape(-1, 2)
        assert np.allclose(np.sum(pair(a) ** 2, 1), np.sum(pair(buf) ** 2, 1), rtol=1e-5)
    # router known answer: ties go to the lower index (tests/test_decode_ops.cpp:84-102)
    logits = np.array([0.1, 2.0, -1.0, 2.0, 0.5, 1.5, -3.0, 0.0], dtype=np.float32)
    for o in (port, ref):
        ids, gates = o.router_sel(logits, 3, 1, 1.0)
        assert list(ids) == [1, 3, 5]
        assert abs(float(gates.sum()) - 1.0) < 1e-6
    ia, ga = port.router_sel(rng.standard_normal(8).astype(np.float32), 2, 1, 1.0)
    parts = rng.standard_normal((2, 64)).astype(np.float32)
    a1 = rng.standard_normal(64).astype(np.float32)
    assert np.array_equal(bits(port.wmerge(parts, ga, a1, None, 1.0)), bits(ref.wmerge(parts, ga, a1, None, 1.0)))


@pytest.mark.parametrize("dk,dv,n", [(128, 128, 1), (128, 128, 7), (128, 128, 400), (192, 128, 33), (50, 33, 7), (6, 3, 5)])
def test_attn_head_bitexact_vs_reference_and_f64(port, ref, dk, dv, n):
    # shapes of tests/test_runtime.cpp:866-937 and tests/test_decode_ops.cpp:179-232
    rng = np.random.default_rng(23)
    nh = 2
    q = rng.standard_normal(nh * dk).astype(np.float32)
    kc = rng.standard_normal((n, nh, dk)).astype(np.float32)
    vc = rng.standard_normal((n, nh, dv)).astype(np.float32)
    scale = 1.0 / np.sqrt(dk)
    for h in range(nh):
        a = port.attn_head_f32(q, kc, vc, n - 1, scale, h, nh, dk, dv)
        b = ref.attn_head_f32(q, kc, vc, n - 1, scale, h, nh, dk, dv)
        assert np.array_equal(bits(a), bits(b))
        s = (kc[:, h, :].astype(np.float64) @ q[h * dk:(h + 1) * dk].astype(np.float64)) * scale
        p = np.exp(s - s.max()); p /= p.sum()
        want = p @ vc[:, h, :].astype(np.float64)
        assert np.max(np.abs(a - want)) < 1e-5


def test_gqa_f16_adapter(port, ref):
    """Query head hq attends over KV head hq // 4 of the f16 cache."""
    rng = np.random.default_rng(9)
    n_head, n_kv, d, kv = 8, 2, 128, 70
    q = rng.standard_normal((n_head, d)).astype(np.float32)
    k = (rng.standard_normal((n_kv, kv + 5, d)) / np.sqrt(d)).astype(np.float16)
    v = (rng.standard_normal((n_kv, kv + 5, d)) / np.sqrt(d)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(d)))
    a, b = port.attn_gqa_f16(q, k, v, kv, scale), ref.attn_gqa_f16(q, k, v, kv, scale)
    assert np.array_equal(bits(a), bits(b))
    for hq in range(n_head):
        hk = hq // 4
        s = (k[hk, :kv].astype(np.float64) @ q[hq].astype(np.float64)) * scale
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.max(np.abs(a[hq] - p @ v[hk, :kv].astype(np.float64))) < 1e-5


def test_reference_task_graph_equals_serial(ref):
    """The reference's CPU worker pool and run_serial give the same bits as the
    tile loop used by the oracle driver (tests/test_quants.cpp:209-289)."""
    rng = np.random.default_rng(2)
    rows, cols = 1000, 2048
    w = synth.q6k_tensor(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    y0 = ref.matvec(capi.Q6_K, w, rows, cols, x)
    y1, _ = ref.ref_stream_dot_tasks(capi.Q6_K, w, rows, cols, x, threads=0)
    y2, _ = ref.ref_stream_dot_tasks(capi.Q6_K, w, rows, cols, x, threads=4)
    ref.ref_pool_shutdown()
    assert np.array_equal(bits(y0), bits(y1)) and np.array_equal(bits(y0), bits(y2))


def test_llama_step_port_equals_reference(port, ref):
    """Two decode steps of a tiny Llama-shape model: identical logits bit for bit."""
    from oracle import pyoracle
    cfg = dict(n_layer=2, n_embd=256, n_head=8, n_kv_head=2, head_dim=32, n_ff=512, n_vocab=300, max_kv=16,
               rope_base=10000.0, eps=1e-5)
    outs = []
    for o in (port, ref):
        m = pyoracle.LlamaOracle(o, cfg)
        for l in range(cfg["n_layer"]):
            for i, name in enumerate(synth.LAYER_TENSORS):
                m.set_layer_tensor(l, i, synth.Q4_K_M[name], synth.llama_tensor(cfg, 1, name, l))
            m.set_layer_norms(l, synth.llama_norm(cfg, 1, "attn_norm", l), synth.llama_norm(cfg, 1, "ffn_norm", l))
            k, v = synth.llama_kv(cfg, 1, l, 5)
            m.seed_kv(l, k, v)
        m.set_global(0, synth.Q4_K_M["tok_embd"], synth.llama_tensor(cfg, 1, "tok_embd"))
        m.set_global(1, synth.Q4_K_M["output"], synth.llama_tensor(cfg, 1, "output"))
        m.set_out_norm(synth.llama_norm(cfg, 1, "out_norm"))
        m.set_n_past(5)
        t1 = m.step(7)
        l1 = m.logits()
        t2 = m.step(t1)
        outs.append((t1, t2, l1, m.logits()))
        assert np.all(np.isfinite(l1))
        m.close()
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1]
    assert np.array_equal(bits(outs[0][2]), bits(outs[1][2])) and np.array_equal(bits(outs[0][3]), bits(outs[1][3]))


def test_port_matches_golden(port):
    """Fixtures generated from the reference build by tests/golden/make_golden.py."""
    g = np.load(GOLDEN)
    for name, fmt in (("q8_0", capi.Q8_0), ("q5_0", capi.Q5_0), ("q4_k", capi.Q4_K), ("q6_k", capi.Q6_K)):
        w, x = g[name + "_w"], g[name + "_x"]
        rows, cols = w.shape[0], x.size
        assert np.array_equal(bits(port.dequant(fmt, w, rows, cols)), bits(g[name + "_deq"]))
        assert np.array_equal(bits(port.matvec(fmt, w, rows, cols, x)), bits(g[name + "_y"]))
    out = port.attn_gqa_f16(g["attn_q"], g["attn_k"], g["attn_v"], int(g["attn_kv_len"]), float(g["attn_scale"]))
    assert np.array_equal(bits(out), bits(g["attn_out"]))
    assert np.array_equal(bits(port.rmsnorm(g["norm_w"], g["norm_x"], 1e-5)), bits(g["norm_y"]))
    assert np.array_equal(bits(port.silu_mul(g["norm_x"], g["norm_w"])), bits(g["silu_y"]))
    assert np.array_equal(bits(port.rope(g["rope_x"], 4097, 8, 128, 0, 128, 500000.0)), bits(g["rope_y"]))


def test_llama_oracle_moe_layer_equals_operator_chain(checker):
    """The step driver's mixture-of-experts layer (llama_oracle.c) against the same chain written out with the single
    operators: router matvec -> ROUTER_SEL -> per selected expert gate, up, SILU_MUL, down -> WMERGE with the residual
    (src/model/decoder.cpp:925-1045). One layer, so the hidden state after the step is the layer's output."""
    from oracle import pyoracle
    cfg = dict(n_layer=1, n_embd=512, n_head=4, n_kv_head=1, head_dim=128, n_ff=768, n_vocab=64, max_kv=8,
               rope_base=10000.0, eps=1e-5)
    NE, K, F, E = 4, 2, 256, 512
    rng = np.random.default_rng(41)
    orc = pyoracle.LlamaOracle(checker, cfg)
    shapes = synth.layer_shapes(cfg)
    tensors = {}
    for i, name in enumerate(synth.LAYER_TENSORS):
        tensors[name] = synth.quant_tensor(capi.Q4_K, rng, *shapes[name])
        orc.set_layer_tensor(0, i, capi.Q4_K, tensors[name])
    an, fn = rng.uniform(0.9, 1.1, E).astype(np.float32), rng.uniform(0.9, 1.1, E).astype(np.float32)
    orc.set_layer_norms(0, an, fn)
    emb = synth.quant_tensor(capi.Q6_K, rng, cfg["n_vocab"], E)
    orc.set_global(pyoracle.G_TOK_EMBD, capi.Q6_K, emb); orc.set_global(pyoracle.G_OUTPUT, capi.Q6_K, emb)
    orc.set_out_norm(np.ones(E, dtype=np.float32))
    wr = rng.standard_normal((NE, E)).astype(np.float32)
    wg = synth.q4k_tensor(rng, NE * F, E); wu = synth.q4k_tensor(rng, NE * F, E); wd = synth.q6k_tensor(rng, NE * E, F)
    orc.set_layer_moe(0, NE, K, 1, 1.0, F, wr, capi.Q4_K, wg, wu, capi.Q6_K, wd)
    orc.set_n_past(0)
    orc.step(5)
    x1 = orc.tap(5)                                   # residual after attention: the block's input and add1
    xn = checker.rmsnorm(fn, x1, cfg["eps"])
    logits = checker.matvec(capi.F32, wr.view(np.uint8).reshape(NE, -1), NE, E, xn)
    ids, gates = checker.router_sel(logits, K, 1, 1.0)
    assert list(ids) == [int(i) for i in np.ctypeslib.as_array(orc.p.flo_llama_moe_ids(orc.h), shape=(K,))]
    parts = np.zeros((K, E), dtype=np.float32)
    for k, e in enumerate(ids):
        g = checker.matvec(capi.Q4_K, wg[e * F:(e + 1) * F], F, E, xn)
        u = checker.matvec(capi.Q4_K, wu[e * F:(e + 1) * F], F, E, xn)
        parts[k] = checker.matvec(capi.Q6_K, wd[e * E:(e + 1) * E], E, F, checker.silu_mul(g, u))
    want = checker.wmerge(parts, np.asarray(gates, dtype=np.float32), x1, None, 1.0)
    assert np.array_equal(orc.hidden().view(np.uint32), want.view(np.uint32))
    orc.close()
