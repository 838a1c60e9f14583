"""GPU parity tests of the mixture-of-experts operators of the decode graph
(ROUTER_SEL, STREAM_DOT_IDX, WMERGE; src/runtime/decode_params.h:234-295,
src/runtime/runtime_internal.h:149-152) and of one whole MoE feed-forward block
at the Mixtral shape (8 experts, top-2, hidden 4096) against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

from fast_llm_b200 import capi, synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(y, ref):
    ref = ref.astype(np.float64)
    floor = 0.1 * np.sqrt(np.mean(ref ** 2)) + 1e-30
    return float(np.max(np.abs(y.astype(np.float64) - ref) / np.maximum(np.abs(ref), floor)))


@pytest.mark.parametrize("n_expert,top_k,norm,scale", [(8, 2, 1, 1.0), (64, 6, 0, 16.0), (8, 8, 1, 2.5), (256, 1, 0, 1.0)])
def test_router_sel_vs_oracle(ctx, checker, n_expert, top_k, norm, scale):
    rng = np.random.default_rng(n_expert + top_k)
    for trial in range(4):
        logits = (rng.standard_normal(n_expert) * (0.02 if trial == 0 else 3.0)).astype(np.float32)
        if trial == 3:
            logits[:] = np.round(logits)            # ties: the lower index must win
        want_ids, want_gates = checker.router_sel(logits, top_k, norm, scale)
        ld = dev(logits)
        ids = torch.zeros(top_k, dtype=torch.int32, device="cuda")
        gates = torch.zeros(top_k, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        ctx.router_sel(ld, ids, gates, n_expert, top_k, norm, scale)
        ctx.sync()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), np.asarray(want_ids, dtype=np.uint32))
        # same order of operations; expf of the device is within 2 ulp of the host's
        assert np.allclose(gates.cpu().numpy(), want_gates, rtol=2e-6, atol=0)


def test_wmerge_vs_oracle(ctx, checker):
    rng = np.random.default_rng(5)
    n, n_parts = 4096, 2
    parts = rng.standard_normal((n_parts, n)).astype(np.float32)
    gates = rng.uniform(0.1, 0.9, n_parts).astype(np.float32)
    a1, a2 = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    for g, x1, x2, sc in ((gates, a1, a2, 1.0), (gates, a1, None, 2.5), (None, None, None, 1.0)):
        want = checker.wmerge(parts, g, x1, x2, sc)
        y = torch.zeros(n, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        ctx.wmerge(dev(parts), None if g is None else dev(g), None if x1 is None else dev(x1),
                   None if x2 is None else dev(x2), y, sc, n_parts, n)
        ctx.sync()
        # separate multiplies and adds in the reference's order: bit-exact
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt,rows,cols", [(capi.Q4_K, 512, 4096), (capi.Q6_K, 256, 2048), (capi.Q4_K, 130, 1024),
                                           (capi.Q8_0, 64, 512)])
def test_stream_dot_idx_vs_oracle(ctx, checker, fmt, rows, cols):
    """The expert is chosen by a device-side index written just before the launch."""
    rng = np.random.default_rng(rows + cols)
    n_expert = 4
    w = synth.quant_tensor(fmt, rng, n_expert * rows, cols)          # experts stacked row-wise
    x = rng.standard_normal(cols).astype(np.float32)
    wd, xd = dev(w), dev(x)
    stride = rows * capi.row_bytes(fmt, cols)
    idx = torch.zeros(1, dtype=torch.int32, device="cuda")
    for e in (2, 0, 3):
        y0 = rng.standard_normal(rows).astype(np.float32)
        yd = dev(y0)
        idx.fill_(e)
        torch.cuda.synchronize()
        ctx.matvec_expert(fmt, wd, rows, cols, idx, stride, xd, yd)
        ctx.sync()
        assert ctx.status() == 0
        want = y0 + checker.matvec(fmt, w[e * rows:(e + 1) * rows], rows, cols, x)   # STREAM_DOT_IDX accumulates
        assert rel_err(yd.cpu().numpy(), want) <= 1e-3
    with pytest.raises(capi.Fl200Error):
        ctx.matvec_expert(fmt, wd, rows, cols, idx, stride + 2, xd, yd)   # stride not a whole number of rows


def test_moe_ffn_block_mixtral_shape(ctx, checker):
    """Router -> top-2 experts (gate, up, SiLU*up, down through STREAM_DOT_IDX) -> WMERGE
    with the residual, for 3 tokens; experts Q4_K, router f32 ~ N(0, 0.02) as in the
    benchmark's MoE configuration (FFN width cut to 2048 to keep the CPU side quick)."""
    rng = np.random.default_rng(17)
    E, F, NE, K = 4096, 2048, 8, 2
    wg = synth.q4k_tensor(rng, NE * F, E); wu = synth.q4k_tensor(rng, NE * F, E); wd_ = synth.q4k_tensor(rng, NE * E, F)
    wr = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    wgd, wud, wdd, wrd = dev(wg), dev(wu), dev(wd_), dev(wr.view(np.uint8).reshape(NE, -1))
    sg, sd = F * capi.row_bytes(capi.Q4_K, E), E * capi.row_bytes(capi.Q4_K, F)
    for tok in range(3):
        x = rng.standard_normal(E).astype(np.float32)
        resid = rng.standard_normal(E).astype(np.float32)
        # oracle
        logits = checker.matvec(capi.F32, wr.view(np.uint8).reshape(NE, -1), NE, E, x)
        ids, gates = checker.router_sel(logits, K, 1, 1.0)
        parts = np.zeros((K, E), dtype=np.float32)
        for k, e in enumerate(ids):
            g = checker.matvec(capi.Q4_K, wg[e * F:(e + 1) * F], F, E, x)
            u = checker.matvec(capi.Q4_K, wu[e * F:(e + 1) * F], F, E, x)
            h = checker.silu_mul(g, u)
            parts[k] = checker.matvec(capi.Q4_K, wd_[e * E:(e + 1) * E], E, F, h)
        want = checker.wmerge(parts, np.asarray(gates, dtype=np.float32), resid, None, 1.0)
        # device: every index and gate stays on the device
        xd, rd = dev(x), dev(resid)
        lg = torch.zeros(NE, device="cuda"); idd = torch.zeros(K, dtype=torch.int32, device="cuda")
        gd = torch.zeros(K, device="cuda"); pd = torch.zeros((K, E), device="cuda")
        gt = torch.zeros(F, device="cuda"); ut = torch.zeros(F, device="cuda"); ht = torch.zeros(F, device="cuda")
        y = torch.zeros(E, device="cuda")
        torch.cuda.synchronize()
        ctx.matvec_assign(capi.F32, wrd, NE, E, xd, lg)
        ctx.router_sel(lg, idd, gd, NE, K, 1, 1.0)
        for k in range(K):
            ctx.lib.fl_b200_memset(ctx._h, capi._p(gt), 0, C.c_size_t(F * 4))
            ctx.lib.fl_b200_memset(ctx._h, capi._p(ut), 0, C.c_size_t(F * 4))
            ctx.matvec_expert(capi.Q4_K, wgd, F, E, idd[k:], sg, xd, gt)
            ctx.matvec_expert(capi.Q4_K, wud, F, E, idd[k:], sg, xd, ut)
            ctx.silu_mul(gt, ut, ht, F)
            ctx.matvec_expert(capi.Q4_K, wdd, E, F, idd[k:], sd, ht, pd[k])
        ctx.wmerge(pd, gd, rd, None, y, 1.0, K, E)
        ctx.sync()
        assert ctx.status() == 0
        assert list(idd.cpu().numpy()) == list(ids)
        assert rel_err(y.cpu().numpy(), want) <= 2e-3      # two chained matvecs


def test_exec_task_moe_kinds(ctx, checker):
    rng = np.random.default_rng(23)
    # ROUTER_SEL through a Task with its parameter block in device memory
    logits = rng.standard_normal(8).astype(np.float32)
    ld = dev(logits); ids = torch.zeros(2, dtype=torch.int32, device="cuda"); gates = torch.zeros(2, device="cuda")

    class RouterP(C.Structure):
        _fields_ = [("logits", C.c_void_p), ("ids", C.c_void_p), ("gates", C.c_void_p), ("n_expert", C.c_uint32),
                    ("top_k", C.c_uint32), ("norm", C.c_uint32), ("scale", C.c_float)]
    p = RouterP(ld.data_ptr(), ids.data_ptr(), gates.data_ptr(), 8, 2, 1, 1.0)
    pd = torch.from_numpy(np.frombuffer(bytes(p), dtype=np.uint8).copy()).cuda()
    t = capi.Task()
    t.kind = 10
    t.aux = pd.data_ptr()
    torch.cuda.synchronize()
    ctx.exec_task(t)
    ctx.sync()
    want_ids, want_gates = checker.router_sel(logits, 2, 1, 1.0)
    assert list(ids.cpu().numpy()) == list(want_ids)
    # STREAM_DOT_IDX through a Task: aux -> device expert id, aux2 = expert stride
    rows, cols = 64, 2048
    w = synth.q4k_tensor(rng, 3 * rows, cols); x = rng.standard_normal(cols).astype(np.float32)
    wd, xd = dev(w), dev(x); y = torch.zeros(rows, device="cuda")
    eid = torch.full((1,), 2, dtype=torch.int32, device="cuda")
    t = capi.Task()
    t.kind = 4; t.fmt = capi.Q4_K; t.w = wd.data_ptr(); t.w_bytes = rows * capi.row_bytes(capi.Q4_K, cols)
    t.x = xd.data_ptr(); t.y = y.data_ptr(); t.rows = rows; t.cols = cols; t.nx = 1
    t.aux = eid.data_ptr(); t.aux2 = rows * capi.row_bytes(capi.Q4_K, cols)
    torch.cuda.synchronize()
    ctx.exec_task(t)
    ctx.sync()
    assert rel_err(y.cpu().numpy(), checker.matvec(capi.Q4_K, w[2 * rows:], rows, cols, x)) <= 1e-3


@pytest.mark.parametrize("F", [1024, 2048])   # Q6_K rows of 1024 columns are not 16-byte pitched: the unfused path
def test_moe_block_vs_oracle(ctx, checker, F):
    """The whole block as one call (fl_b200_moe_forward) for several tokens, against the
    oracle's chain of operators; also what a second call leaves behind in the reused buffers."""
    from fast_llm_b200.moe import MoeBlock
    rng = np.random.default_rng(29)
    E, NE, K, T = 4096, 8, 2, 4
    wg = synth.q4k_tensor(rng, NE * F, E); wu = synth.q4k_tensor(rng, NE * F, E); wd_ = synth.q6k_tensor(rng, NE * E, F)
    wr = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    blk = MoeBlock(ctx, E, F, NE, K, norm=1, scale=1.0, fmt_gate_up=capi.Q4_K, fmt_down=capi.Q6_K, max_tokens=T)
    blk.set_weights(dev(wr), dev(wg), dev(wu), dev(wd_))
    for trial in range(2):
        x = rng.standard_normal((T, E)).astype(np.float32)
        xd = dev(x); y = torch.zeros((T, E), device="cuda")
        torch.cuda.synchronize()
        blk.forward(xd, T, y)
        ctx.sync()
        assert ctx.status() == 0
        ids, gates = blk.routing(T)
        got = y.cpu().numpy()
        for t in range(T):
            logits = checker.matvec(capi.F32, wr.view(np.uint8).reshape(NE, -1), NE, E, x[t])
            want_ids, want_gates = checker.router_sel(logits, K, 1, 1.0)
            assert list(ids[t]) == list(want_ids)
            assert np.allclose(gates[t], want_gates, rtol=1e-5)
            parts = np.zeros((K, E), dtype=np.float32)
            for k, e in enumerate(want_ids):
                g = checker.matvec(capi.Q4_K, wg[e * F:(e + 1) * F], F, E, x[t])
                u = checker.matvec(capi.Q4_K, wu[e * F:(e + 1) * F], F, E, x[t])
                parts[k] = checker.matvec(capi.Q6_K, wd_[e * E:(e + 1) * E], E, F, checker.silu_mul(g, u))
            want = checker.wmerge(parts, np.asarray(want_gates, dtype=np.float32), None, None, 1.0)
            assert rel_err(got[t], want) <= 2e-3, (trial, t)
    # a call that repeats the one before it is recorded as a CUDA graph, then replayed: same bits every time
    first = y.cpu().numpy().copy()
    for _ in range(3):
        y.zero_()
        torch.cuda.synchronize()
        blk.forward(xd, T, y)
        ctx.sync()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), first.view(np.uint32))
    with pytest.raises(capi.Fl200Error):
        blk.forward(xd, T + 1, y)
    blk.close()
