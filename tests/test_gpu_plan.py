"""A frozen task table through fl_b200_plan_*: one Llama-shape layer written as
the reference would (RMSNORM, row-tiled STREAM_DOTs, the appended RoPE/append and
GQA-attention kinds, ADD2, SILU_MUL, a terminal SIGNAL) replayed as one CUDA
graph, against the CPU oracle run operator by operator; and the freeze rules."""
import ctypes as C

import numpy as np
import pytest

from fast_llm_b200 import capi, synth
from fast_llm_b200.graph import Graph

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


class RmsNormP(C.Structure):
    _fields_ = [("wnorm", C.c_void_p), ("x", C.c_void_p), ("y", C.c_void_p), ("eps", C.c_float), ("n", C.c_uint32)]


class Add2P(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("y", C.c_void_p), ("n", C.c_uint32)]


class SiluMulP(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("h", C.c_void_p), ("n", C.c_uint32)]


class AttnP(C.Structure):
    _fields_ = [("q", C.c_void_p), ("kcache", C.c_void_p), ("vcache", C.c_void_p), ("out", C.c_void_p), ("pos", C.c_void_p),
                ("scale", C.c_float), ("n_q_head", C.c_uint32), ("n_kv_head", C.c_uint32), ("head_dim", C.c_uint32),
                ("kv_stride", C.c_uint32)]


class RopeAppendP(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("kcache", C.c_void_p), ("vcache", C.c_void_p),
                ("pos", C.c_void_p), ("n_q_head", C.c_uint32), ("n_kv_head", C.c_uint32), ("head_dim", C.c_uint32),
                ("kv_stride", C.c_uint32), ("freq_base", C.c_float)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(y, ref):
    ref = ref.astype(np.float64)
    return float(np.max(np.abs(y.astype(np.float64) - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


def fan_out(g, src, targets):
    """Edges src -> targets through SIGNAL tasks where the fan-out would exceed the reference's
    limit of 6 consumers per task (kMaxConsumers, include/fastllm/fastllm.h:59)."""
    targets = list(targets)
    while len(targets) > 6:
        nxt = []
        for i in range(0, len(targets), 6):
            s = g.add(capi.K_SIGNAL)
            for t in targets[i:i + 6]:
                g.edge(s, t)
            nxt.append(s)
        targets = nxt
    for t in targets:
        g.edge(src, t)
    return len(targets)


def test_layer_as_task_table(ctx, checker):
    rng = np.random.default_rng(41)
    E, NH, NKV, D, F, KV, POS = 2048, 16, 4, 128, 4096, 64, 37
    QD, KD = NH * D, NKV * D
    fm = {"wq": capi.Q4_K, "wk": capi.Q4_K, "wv": capi.Q6_K, "wo": capi.Q4_K, "gate": capi.Q4_K, "up": capi.Q4_K, "down": capi.Q6_K}
    shp = {"wq": (QD, E), "wk": (KD, E), "wv": (KD, E), "wo": (E, QD), "gate": (F, E), "up": (F, E), "down": (E, F)}
    w = {k: synth.quant_tensor(fm[k], rng, *shp[k]) for k in fm}
    x0 = rng.standard_normal(E).astype(np.float32)
    an = rng.uniform(0.9, 1.1, E).astype(np.float32); fn = rng.uniform(0.9, 1.1, E).astype(np.float32)
    kc = np.zeros((NKV, KV, D), dtype=np.float16); vc = np.zeros((NKV, KV, D), dtype=np.float16)
    kc[:, :POS] = (rng.standard_normal((NKV, POS, D)) * 0.1).astype(np.float16)
    vc[:, :POS] = (rng.standard_normal((NKV, POS, D)) * 0.1).astype(np.float16)
    scale = float(1.0 / np.sqrt(D))

    # ---- device buffers ----
    d = {k_: dev(v_) for k_, v_ in w.items()}
    xd, and_, fnd = dev(x0), dev(an), dev(fn)
    z = lambda n: torch.zeros(n, dtype=torch.float32, device="cuda")
    xn_d, q_d, k_d, v_d, att_d, o_d, x1_d, xn2_d, g_d, u_d, h_d, dn_d, x2_d = (z(E), z(QD), z(KD), z(KD), z(QD), z(E), z(E), z(E),
                                                                              z(F), z(F), z(F), z(E), z(E))
    kcd, vcd = dev(kc.view(np.int16)), dev(vc.view(np.int16))
    posd = torch.tensor([POS], dtype=torch.int32, device="cuda")
    g = Graph(ctx)
    t_norm = g.add(capi.K_RMSNORM, aux=g.param_block(RmsNormP(and_.data_ptr(), xd.data_ptr(), xn_d.data_ptr(), 1e-5, E)))

    def dots(name, x_t, y_t, rows, cols, tile):
        ids = []
        rb = capi.row_bytes(fm[name], cols)
        for r0 in range(0, rows, tile):
            n = min(tile, rows - r0)
            ids.append(g.add(capi.K_STREAM_DOT, fmt=fm[name], w=d[name].data_ptr() + r0 * rb, w_bytes=n * rb,
                             x=x_t.data_ptr(), y=y_t.data_ptr() + r0 * 4, rows=n, cols=cols))
        return ids

    tq = dots("wq", xn_d, q_d, QD, E, 512); tk = dots("wk", xn_d, k_d, KD, E, 192); tv = dots("wv", xn_d, v_d, KD, E, 192)
    fan_out(g, t_norm, tq + tk + tv)
    sig_qkv = g.add(capi.K_SIGNAL)                     # fan-in marker, as the reference uses between wide stages
    for t in tq + tk + tv:
        g.edge(t, sig_qkv)
    t_rope = g.add(capi.K_ROPE_KV_APPEND_F16, aux=g.param_block(RopeAppendP(q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(),
                   kcd.data_ptr(), vcd.data_ptr(), posd.data_ptr(), NH, NKV, D, KV, 500000.0)))
    g.edge(sig_qkv, t_rope)
    t_att = g.add(capi.K_ATTN_GQA_F16, aux=g.param_block(AttnP(q_d.data_ptr(), kcd.data_ptr(), vcd.data_ptr(), att_d.data_ptr(),
                  posd.data_ptr(), scale, NH, NKV, D, KV)))
    g.edge(t_rope, t_att)
    to = dots("wo", att_d, o_d, E, QD, 1024)
    t_add1 = g.add(capi.K_ADD2, aux=g.param_block(Add2P(xd.data_ptr(), o_d.data_ptr(), x1_d.data_ptr(), E)))
    fan_out(g, t_att, to)
    for t in to:
        g.edge(t, t_add1)
    t_norm2 = g.add(capi.K_RMSNORM, aux=g.param_block(RmsNormP(fnd.data_ptr(), x1_d.data_ptr(), xn2_d.data_ptr(), 1e-5, E)))
    g.edge(t_add1, t_norm2)
    tg = dots("gate", xn2_d, g_d, F, E, 1024); tu = dots("up", xn2_d, u_d, F, E, 1024)
    t_silu = g.add(capi.K_SILU_MUL, aux=g.param_block(SiluMulP(g_d.data_ptr(), u_d.data_ptr(), h_d.data_ptr(), F)))
    sig_gu = g.add(capi.K_SIGNAL)
    fan_out(g, t_norm2, tg + tu)
    for t in tg + tu:
        g.edge(t, sig_gu)
    g.edge(sig_gu, t_silu)
    td = dots("down", h_d, dn_d, E, F, 512)
    t_add2 = g.add(capi.K_ADD2, aux=g.param_block(Add2P(x1_d.data_ptr(), dn_d.data_ptr(), x2_d.data_ptr(), E)))
    fan_out(g, t_silu, td)
    for t in td:
        g.edge(t, t_add2)
    t_end = g.add(capi.K_SIGNAL)
    g.edge(t_add2, t_end)
    g.freeze()
    info = g.info()
    n_tiles = len(tq + tk + tv + to + tg + tu + td)
    assert info["tasks"] == len(g._tasks)
    # every tensor's tiles collapse into one launch: 7 matvecs + 2 norms + rope + attn + 2 adds + silu (two tensors
    # that happen to be adjacent in memory with adjacent outputs, e.g. gate and up, may merge further)
    assert 12 <= info["launches"] <= 14 and info["merged_tiles"] == n_tiles - (info["launches"] - 7)

    # ---- the oracle, operator by operator ----
    xn = checker.rmsnorm(an, x0, 1e-5)
    q = checker.matvec(fm["wq"], w["wq"], QD, E, xn); k = checker.matvec(fm["wk"], w["wk"], KD, E, xn)
    v = checker.matvec(fm["wv"], w["wv"], KD, E, xn)
    qr = checker.rope(q, POS, NH, D, 0, D, 500000.0); kr = checker.rope(k, POS, NKV, D, 0, D, 500000.0)
    kc2, vc2 = kc.copy(), vc.copy()
    kc2[:, POS] = kr.reshape(NKV, D).astype(np.float16); vc2[:, POS] = v.reshape(NKV, D).astype(np.float16)
    att = checker.attn_gqa_f16(qr.reshape(NH, D), kc2, vc2, POS + 1, scale).reshape(-1)
    x1 = checker.add2(x0, checker.matvec(fm["wo"], w["wo"], E, QD, att))

    for run in range(2):   # replay: the accumulate slots are zeroed per run, like the reference does
        for t_ in (q_d, k_d, v_d, o_d, g_d, u_d, dn_d):
            t_.zero_()
        torch.cuda.synchronize()
        g.run()
        ctx.sync()
        assert ctx.status() == 0
        assert rel(xn_d.cpu().numpy(), xn) < 1e-5
        assert rel(v_d.cpu().numpy(), v) < 1e-4
        x1g = x1_d.cpu().numpy()
        assert rel(x1g, x1) < 5e-3      # through the f16 append of this token's K / V
        # the FFN half from the device's own x1 (these synthetic weights amplify a 1e-3 input difference a hundredfold)
        xn2g = checker.rmsnorm(fn, x1g, 1e-5)
        hg = checker.silu_mul(checker.matvec(fm["gate"], w["gate"], F, E, xn2g), checker.matvec(fm["up"], w["up"], F, E, xn2g))
        x2g = checker.add2(x1g, checker.matvec(fm["down"], w["down"], E, F, hg))
        assert rel(x2_d.cpu().numpy(), x2g) < 2e-3
    g.close()


def test_freeze_rules(ctx):
    x = torch.zeros(256, device="cuda"); w = torch.zeros(144, dtype=torch.uint8, device="cuda")
    def dot(g):
        return g.add(capi.K_STREAM_DOT, fmt=capi.Q4_K, w=w.data_ptr(), w_bytes=144, x=x.data_ptr(), y=x.data_ptr(), rows=1, cols=256)
    g = Graph(ctx); a = dot(g); s = g.add(capi.K_SIGNAL); g.edge(a, s); g.freeze(); g.run(); ctx.sync(); g.close()
    g = Graph(ctx); a = dot(g); b = dot(g); g.edge(a, b); g.edge(b, a)          # cycle
    with pytest.raises(capi.Fl200Error): g.freeze()
    g = Graph(ctx); a = dot(g); s1 = g.add(capi.K_SIGNAL); s2 = g.add(capi.K_SIGNAL); g.edge(a, s1); g.edge(a, s2)   # two sinks
    with pytest.raises(capi.Fl200Error): g.freeze()
    g = Graph(ctx); a = dot(g)                                                   # sink is not a SIGNAL
    with pytest.raises(capi.Fl200Error): g.freeze()
    g = Graph(ctx); a = g.add(capi.K_STREAM_DOT, fmt=capi.Q4_K, w=w.data_ptr(), w_bytes=100, x=x.data_ptr(), y=x.data_ptr(), rows=1, cols=256)
    s = g.add(capi.K_SIGNAL); g.edge(a, s)                                       # w_bytes mismatch
    with pytest.raises(capi.Fl200Error): g.freeze()
    g = Graph(ctx); a = g.add(capi.K_RMSNORM); s = g.add(capi.K_SIGNAL); g.edge(a, s)   # decode op without aux
    with pytest.raises(capi.Fl200Error): g.freeze()
    g = Graph(ctx); a = g.add(9, aux=x.data_ptr()); s = g.add(capi.K_SIGNAL); g.edge(a, s)   # ATTN_HEAD (f32 MHA): no device kernel
    with pytest.raises(capi.Fl200Error): g.freeze()


def test_plan_survives_growth_of_the_attention_scratch(ctx, checker):
    """A recorded plan keeps the split-KV scratch address it was captured with. A later attention call that
    needs more scratch (more sequences) must not free that buffer: the plan is run again and checked."""
    shared = ctx   # the session's context may have grown its scratch already: use a fresh one
    ctx = capi.Context(0)
    rng = np.random.default_rng(5)
    NH, NKV, D, KV, POS = 8, 2, 128, 256, 200
    scale = float(1.0 / np.sqrt(D))
    q = rng.standard_normal((NH, D)).astype(np.float32)
    kc = (rng.standard_normal((NKV, KV, D)) * 0.1).astype(np.float16)
    vc = (rng.standard_normal((NKV, KV, D)) * 0.1).astype(np.float16)
    qd, kcd, vcd = dev(q), dev(kc.view(np.int16)), dev(vc.view(np.int16))
    out = torch.zeros((NH, D), dtype=torch.float32, device="cuda")
    posd = torch.tensor([POS], dtype=torch.int32, device="cuda")
    g = Graph(ctx)
    t_att = g.add(capi.K_ATTN_GQA_F16, aux=g.param_block(AttnP(qd.data_ptr(), kcd.data_ptr(), vcd.data_ptr(), out.data_ptr(),
                  posd.data_ptr(), scale, NH, NKV, D, KV)))
    g.edge(t_att, g.add(capi.K_SIGNAL))
    g.freeze()
    want = checker.attn_gqa_f16(q, kc, vc, POS + 1, scale)
    g.run(); ctx.sync()
    assert float(np.max(np.abs(out.cpu().numpy() - want))) <= 2e-3
    # a much larger call on the same context: 16 sequences x 32 heads, long enough for many splits
    B, NH2, NKV2, KV2 = 16, 32, 8, 4096
    q2 = torch.randn((B, NH2, D), device="cuda")
    k2 = (torch.randn((B, NKV2, KV2, D), device="cuda") * 0.1).half()
    v2 = (torch.randn((B, NKV2, KV2, D), device="cuda") * 0.1).half()
    o2 = torch.zeros((B, NH2, D), device="cuda")
    torch.cuda.synchronize()
    ctx.attn_decode(q2, k2.view(torch.int16), v2.view(torch.int16), NH2, NKV2, D, KV2, KV2, B, scale, o2)
    ctx.sync()
    junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(8)]   # reuse of freed memory would show
    out.zero_()
    torch.cuda.synchronize()
    g.run(); ctx.sync()
    assert ctx.status() == 0
    assert float(np.max(np.abs(out.cpu().numpy() - want))) <= 2e-3
    del junk
    g.close()
    ctx.close()
    assert shared.status() == 0
