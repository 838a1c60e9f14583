"""GPU parity tests of the single operators, through the C ABI, against the CPU
oracle (the reference's own code where its build travelled, else the pinned
port) on identical seeded inputs.

Gates:
  dequantised weights    bit-exact
  matvec                 <= 1e-3 relative, error normalised by max(|ref|, 0.1 * RMS(ref))
                         (the reference's own GPU gate, tools/membench.cu:524-530)
  attention              <= 2e-3 max-abs
"""
import os

import numpy as np
import pytest

from fast_llm_b200 import capi, synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_ops_golden.npz")
MATVEC_RTOL = 1e-3
ATTN_ATOL = 2e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def rel_err(y, ref):
    ref = ref.astype(np.float64)
    floor = 0.1 * np.sqrt(np.mean(ref ** 2)) + 1e-30
    return float(np.max(np.abs(y.astype(np.float64) - ref) / np.maximum(np.abs(ref), floor)))


def gpu_dequant(ctx, fmt, w, rows, cols):
    wd = dev(w)
    out = torch.empty((rows, cols), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.dequant(fmt, wd, rows, cols, out)
    ctx.sync()
    return out.cpu().numpy()


def gpu_matvec(ctx, fmt, w, rows, cols, x):
    wd, xd = dev(w), dev(x)
    y = torch.full((rows + 8,), 7.0, dtype=torch.float32, device="cuda")   # canary tail
    torch.cuda.synchronize()
    ctx.matvec_assign(fmt, wd, rows, cols, xd, y)
    ctx.sync()
    assert ctx.status() == 0
    y = y.cpu().numpy()
    assert np.all(y[rows:] == 7.0), "matvec wrote past its output"
    return y[:rows]


@pytest.mark.parametrize("fmt,rows,cols", [
    (capi.Q4_K, 4096, 4096),       # configuration 0
    (capi.Q6_K, 1024, 4096),       # attn_v shape
    (capi.Q6_K, 64, 14336),        # ffn_down rows
    (capi.Q4_K, 3, 256), (capi.Q6_K, 3, 256), (capi.Q4_K, 5, 768), (capi.Q6_K, 5, 768),
    (capi.Q8_0, 7, 1408), (capi.Q5_0, 7, 1408), (capi.Q8_0, 1, 32), (capi.F32, 4, 64),
])
def test_dequant_bitexact(ctx, checker, fmt, rows, cols):
    w = synth.quant_tensor(fmt, np.random.default_rng(rows * 7 + cols + fmt), rows, cols)
    got = gpu_dequant(ctx, fmt, w, rows, cols)
    want = checker.dequant(fmt, w, rows, cols)
    assert np.array_equal(bits(got), bits(want))


def test_dequant_extreme_scales(ctx, checker):
    """Largest / smallest finite f16 scales, zero and subnormal scales, extreme quants."""
    rng = np.random.default_rng(1)
    w = synth.q4k_tensor(rng, 8, 512)
    blk = w.reshape(-1, 144)
    blk[0, 0:2] = np.array([0x7BFF], dtype=np.uint16).view(np.uint8)   # d = 65504
    blk[1, 0:2] = np.array([0x0001], dtype=np.uint16).view(np.uint8)   # d = smallest subnormal
    blk[2, 0:4] = 0                                                    # d = dmin = 0
    blk[3, 4:16] = 0xFF                                                # all scales / mins 63
    blk[4, 16:] = 0xFF                                                 # all quants 15
    blk[5, 2:4] = np.array([0x8400], dtype=np.uint16).view(np.uint8)   # negative dmin
    assert np.array_equal(bits(gpu_dequant(ctx, capi.Q4_K, w, 8, 512)), bits(checker.dequant(capi.Q4_K, w, 8, 512)))
    w = synth.q6k_tensor(rng, 8, 512)
    blk = w.reshape(-1, 210)
    blk[0, 208:210] = np.array([0x7BFF], dtype=np.uint16).view(np.uint8)
    blk[1, 208:210] = np.array([0x0001], dtype=np.uint16).view(np.uint8)
    blk[2, 192:208] = np.array([-128] * 16, dtype=np.int8).view(np.uint8)
    blk[3, 0:192] = 0xFF
    blk[4, 0:192] = 0
    assert np.array_equal(bits(gpu_dequant(ctx, capi.Q6_K, w, 8, 512)), bits(checker.dequant(capi.Q6_K, w, 8, 512)))


@pytest.mark.parametrize("fmt,rows,cols", [
    (capi.Q4_K, 4096, 4096),       # configuration 0 (streaming kernel)
    (capi.Q4_K, 1024, 4096),       # wk
    (capi.Q6_K, 1024, 4096),       # wv
    (capi.Q6_K, 512, 14336),       # rows of ffn_down
    (capi.Q4_K, 1026, 2048), (capi.Q6_K, 1029, 2048), (capi.Q4_K, 1, 2048), (capi.Q6_K, 3, 6144),   # ragged row counts
    (capi.Q4_K, 37, 768), (capi.Q6_K, 37, 1280),
    (capi.Q8_0, 1024, 4096), (capi.Q8_0, 37, 2048), (capi.Q8_0, 130, 768), (capi.Q8_0, 66, 6144),   # Q8_0 streaming path
    (capi.Q4_K, 64, 512), (capi.Q4_K, 101, 1792), (capi.Q4_K, 256, 7168), (capi.Q6_K, 64, 6144 + 2048),   # partial last segment
 (capi.Q8_0, 100, 1408), (capi.Q5_0, 33, 1408), (capi.F32, 50, 200),
])
def test_matvec_vs_oracle(ctx, checker, fmt, rows, cols):
    rng = np.random.default_rng(rows + 31 * cols + fmt)
    w = synth.quant_tensor(fmt, rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    got = gpu_matvec(ctx, fmt, w, rows, cols, x)
    want = checker.matvec(fmt, w, rows, cols, x)
    assert rel_err(got, want) <= MATVEC_RTOL
    # run-to-run reproducible (fixed summation order)
    assert np.array_equal(bits(got), bits(gpu_matvec(ctx, fmt, w, rows, cols, x)))


@pytest.mark.parametrize("fmt", [capi.Q4_K, capi.Q6_K, capi.Q8_0])
@pytest.mark.parametrize("case", ["outlier_1e3", "outlier_1e4", "zero_block", "denormal_block", "tiny_vector"])
def test_matvec_activation_outliers(ctx, checker, fmt, case):
    """The kernels keep the activation per 256-column block as scaled low-precision parts. Real residual
    streams hold single elements 1e3 - 1e4 times their neighbours: the small elements of such a block, an
    all-zero block, a block of denormal-scale values and a vector that is tiny throughout must all stay
    inside the 1e-3 gate (measured against the rows' own magnitude, not against the outlier)."""
    rows, cols = 256, 4096
    rng = np.random.default_rng(1000 + fmt)
    w = synth.quant_tensor(fmt, rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    if case.startswith("outlier"):
        # one huge element inside block 3; its own contribution is removed from both sides below so that the
        # comparison is about the OTHER elements of the block
        x[3 * 256 + 77] *= 1e3 if case == "outlier_1e3" else 1e4
    elif case == "zero_block":
        x[5 * 256:6 * 256] = 0.0
        x[9 * 256:10 * 256] = -0.0
    elif case == "denormal_block":
        x[7 * 256:8 * 256] = (rng.standard_normal(256) * 1e-40).astype(np.float32)
    else:
        x *= np.float32(1e-30)
    got = gpu_matvec(ctx, fmt, w, rows, cols, x)
    assert np.all(np.isfinite(got))
    if case.startswith("outlier"):
        # The f32 oracle is no yardstick here: once the huge term is in its running sum, every later addition
        # is rounded at that magnitude. The yardstick is the exact product of the (bit-exact) dequantised weights
        # in f64, and the error is measured against the rows' magnitude WITHOUT the outlier column.
        deq = checker.dequant(fmt, w, rows, cols).astype(np.float64)
        want = deq @ x.astype(np.float64)
        x0 = x.astype(np.float64); x0[3 * 256 + 77] = 0.0
        base = deq @ x0
        floor = 0.1 * np.sqrt(np.mean(base ** 2))
        err = float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(base), floor)))
        # one f32 rounding of the result itself, whose magnitude is the outlier term's
        slack = float(np.max(np.abs(want)) * 2.0 ** -23 / floor)
        assert err <= MATVEC_RTOL + slack, (err, slack)
    else:
        want = checker.matvec(fmt, w, rows, cols, x)
        assert rel_err(got, want) <= MATVEC_RTOL


@pytest.mark.parametrize("fmt,rows,cols,c0,n", [
    (capi.Q6_K, 4096, 14336, 7168, 7168),    # down, rank 1 of 2
    (capi.Q6_K, 512, 14336, 3584 * 3, 3584), # down, rank 3 of 4
    (capi.Q6_K, 300, 14336, 1792 * 5, 1792), # down, rank 5 of 8 (7 blocks: 1470-byte rows padded to 1472)
    (capi.Q4_K, 4096, 4096, 512 * 7, 512),   # O, rank 7 of 8
    (capi.Q4_K, 130, 4096, 1024, 1024),      # O, rank 1 of 4
])
def test_matvec_column_slice_with_pitch(ctx, checker, fmt, rows, cols, c0, n):
    """The tensor-parallel column slices of O / down: blocks [c0, c0+n) of every row,
    rows zero-padded to a multiple of 16 bytes, against the oracle on the packed slice."""
    from fast_llm_b200 import tp
    rng = np.random.default_rng(rows + cols + c0)
    w = synth.quant_tensor(fmt, rng, rows, cols)
    x = rng.standard_normal(n).astype(np.float32)
    ws = tp.slice_cols(w, fmt, c0, n)
    pitch = tp.pitch_of(fmt, n)
    assert ws.shape == (rows, pitch) and pitch % 16 == 0
    packed = np.ascontiguousarray(ws[:, :capi.row_bytes(fmt, n)])
    want = checker.matvec(fmt, packed, rows, n, x)
    wd, xd = dev(ws), dev(x)
    y = torch.full((rows + 8,), 7.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.matvec_pitched(fmt, wd, rows, n, pitch, xd, y)
    ctx.sync()
    assert ctx.status() == 0
    y = y.cpu().numpy()
    assert np.all(y[rows:] == 7.0)
    assert rel_err(y[:rows], want) <= MATVEC_RTOL
    # the slices of all ranks add up to the whole product (linearity across the split)
    if c0 == 0 or rows > 1000:
        return
    xf = rng.standard_normal(cols).astype(np.float32)
    full = checker.matvec(fmt, w, rows, cols, xf)
    acc = np.zeros(rows, dtype=np.float64)
    for r in range(cols // n):
        wr = dev(tp.slice_cols(w, fmt, r * n, n)); xr = dev(xf[r * n:(r + 1) * n]); yr = torch.zeros(rows, device="cuda")
        torch.cuda.synchronize()
        ctx.matvec_pitched(fmt, wr, rows, n, pitch, xr, yr)
        ctx.sync()
        acc += yr.cpu().numpy()
    assert rel_err(acc.astype(np.float32), full) <= MATVEC_RTOL


def test_matvec_config0_vs_f64_and_golden(ctx, checker):
    c0 = synth.config0(0)
    got = gpu_matvec(ctx, capi.Q4_K, c0["w"], 4096, 4096, c0["x"])
    deq = checker.dequant(capi.Q4_K, c0["w"], 4096, 4096).astype(np.float64)
    y64 = deq @ c0["x"].astype(np.float64)
    S = np.sqrt((deq ** 2) @ (c0["x"].astype(np.float64) ** 2))
    # error normalised by S = ||w o x||_2 (tests/test_runtime.cpp:489-512): the canonical CPU dot itself is ~8e-6
    assert np.max(np.abs(got - y64) / S) < 2e-5
    g = np.load(GOLDEN)
    for name, fmt in (("q4_k", capi.Q4_K), ("q6_k", capi.Q6_K), ("q8_0", capi.Q8_0), ("q5_0", capi.Q5_0)):
        w, x = g[name + "_w"], g[name + "_x"]
        assert rel_err(gpu_matvec(ctx, fmt, w, w.shape[0], x.size, x), g[name + "_y"]) <= MATVEC_RTOL
        assert np.array_equal(bits(gpu_dequant(ctx, fmt, w, w.shape[0], x.size)), bits(g[name + "_deq"]))


def test_matvec_linearity_full_size(ctx):
    """Size-independent property at the head's full size: W(a x1 + x2) = a W x1 + W x2."""
    rows, cols = 128256, 4096
    rng = np.random.default_rng(5)
    w = synth.q6k_tensor(rng, rows, cols)
    x1 = rng.standard_normal(cols).astype(np.float32)
    x2 = rng.standard_normal(cols).astype(np.float32)
    y1, y2 = gpu_matvec(ctx, capi.Q6_K, w, rows, cols, x1), gpu_matvec(ctx, capi.Q6_K, w, rows, cols, x2)
    y3 = gpu_matvec(ctx, capi.Q6_K, w, rows, cols, (2.0 * x1 + x2).astype(np.float32))
    assert rel_err(y3, 2.0 * y1.astype(np.float64) + y2) <= 1e-4


def test_stream_dot_semantics(ctx, checker):
    """fl_b200_matvec accumulates into y and handles nx columns like the reference's STREAM_DOT."""
    rng = np.random.default_rng(8)
    rows, cols, nx = 300, 2048, 3
    w = synth.q4k_tensor(rng, rows, cols)
    x = rng.standard_normal((nx, cols)).astype(np.float32)
    y0 = rng.standard_normal((nx, rows)).astype(np.float32)
    want = y0.copy()
    checker.stream_dot(capi.Q4_K, w, rows, cols, x, want, nx=nx, xstride=cols, ystride=rows)
    wd, xd, yd = dev(w), dev(x), dev(y0)
    torch.cuda.synchronize()
    ctx.matvec(capi.Q4_K, wd, rows, cols, xd, yd, nx=nx, xstride=cols, ystride=rows)
    ctx.sync()
    assert rel_err(yd.cpu().numpy().ravel(), want.ravel()) <= MATVEC_RTOL


@pytest.mark.parametrize("rows,cols,nx", [(320, 4096, 2), (64, 4096, 3), (1024, 4096, 8), (48, 8192, 4), (160, 4096, 9), (32, 4096, 17)])
def test_stream_dot_multi_column_tensor_core(ctx, checker, rows, cols, nx):
    """Task::nx > 1 (draft verification): the columns go through the tensor-core kernel in one pass
    over the weights (up to 8 at a time); results equal the reference's STREAM_DOT column by column."""
    rng = np.random.default_rng(rows + cols + nx)
    w = synth.q4k_tensor(rng, rows, cols)
    xstride, ystride = cols + 64, rows + 16
    x = rng.standard_normal((nx, xstride)).astype(np.float32)
    x[:, cols:] = np.nan                                   # the gap between columns is never read
    x[1] *= 1000.0                                         # columns with very different scales
    y0 = rng.standard_normal((nx, ystride)).astype(np.float32)
    want = y0.copy()
    for p in range(nx):
        want[p, :rows] += checker.matvec(capi.Q4_K, w, rows, cols, x[p, :cols].copy())
    wd, xd, yd = dev(w), dev(x), dev(y0)
    torch.cuda.synchronize()
    ctx.matvec(capi.Q4_K, wd, rows, cols, xd, yd, nx=nx, xstride=xstride, ystride=ystride)
    ctx.sync()
    assert ctx.status() == 0
    got = yd.cpu().numpy()
    assert np.array_equal(got[:, rows:], y0[:, rows:])     # nothing outside the rows is touched
    for p in range(nx):
        assert rel_err(got[p, :rows], want[p, :rows]) <= MATVEC_RTOL, p


def test_matvec_host_entry(ctx, checker):
    rng = np.random.default_rng(4)
    rows, cols = 2048, 4096
    w = synth.q4k_tensor(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    y = np.zeros(rows, dtype=np.float32)
    wd = dev(w)
    torch.cuda.synchronize()
    ctx.matvec_host(capi.Q4_K, wd, rows, cols, x, y)
    assert rel_err(y, checker.matvec(capi.Q4_K, w, rows, cols, x)) <= MATVEC_RTOL


def test_boundary_rejects_bad_arguments(ctx):
    w = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    x = torch.zeros(4096, dtype=torch.float32, device="cuda")
    with pytest.raises(capi.Fl200Error):
        ctx.matvec_assign(capi.Q4_K, w, 1, 100, x, x)            # cols not a multiple of the block
    with pytest.raises(capi.Fl200Error):
        ctx.matvec_assign(9, w, 1, 256, x, x)                    # unknown format
    with pytest.raises(capi.Fl200Error):
        ctx.matvec_assign(capi.Q4_K, None, 1, 256, x, x)         # null weights
    with pytest.raises(capi.Fl200Error):
        ctx.attn_decode(x, w, w, 32, 8, 64, 10, 16, 1, 1.0, x)   # head_dim 64 is not built
    with pytest.raises(capi.Fl200Error):
        ctx.attn_decode(x, w, w, 32, 8, 128, 0, 16, 1, 1.0, x)   # empty KV
    t = capi.Task()
    t.kind = 9                                                   # ATTN_HEAD (f32 MHA): not implemented on the device
    with pytest.raises(capi.Fl200Error):
        ctx.exec_task(t)


def gpu_attn(ctx, q, k, v, kv_len, scale, batch=1):
    n_q, d = q.shape[-2], q.shape[-1]
    n_kv, stride = k.shape[-3], k.shape[-2]
    qd, kd, vd = dev(q), dev(k.view(np.uint16)), dev(v.view(np.uint16))
    out = torch.zeros(q.shape, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.attn_decode(qd, kd, vd, n_q, n_kv, d, kv_len, stride, batch, scale, out)
    ctx.sync()
    assert ctx.status() == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("kv_len", [1, 7, 63, 64, 65, 191, 400, 1024, 3000])
def test_attn_vs_oracle(ctx, checker, kv_len):
    rng = np.random.default_rng(23 + kv_len)
    n_q, n_kv, d = 32, 8, 128
    stride = kv_len + 3
    q = rng.standard_normal((n_q, d)).astype(np.float32)
    k = (rng.standard_normal((n_kv, stride, d)) / np.sqrt(d)).astype(np.float16)
    v = (rng.standard_normal((n_kv, stride, d)) / np.sqrt(d)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(d)))
    got = gpu_attn(ctx, q, k, v, kv_len, scale)
    want = checker.attn_gqa_f16(q, k, v, kv_len, scale)
    assert np.max(np.abs(got - want)) <= ATTN_ATOL
    assert np.array_equal(bits(got), bits(gpu_attn(ctx, q, k, v, kv_len, scale)))   # reproducible


def test_attn_config0_and_golden(ctx, checker):
    c0 = synth.config0(0)
    got = gpu_attn(ctx, c0["q"], c0["k"], c0["v"], 1024, c0["scale"])
    want = checker.attn_gqa_f16(c0["q"], c0["k"], c0["v"], 1024, c0["scale"])
    assert np.max(np.abs(got - want)) <= ATTN_ATOL
    g = np.load(GOLDEN)
    got = gpu_attn(ctx, g["attn_q"], g["attn_k"], g["attn_v"], int(g["attn_kv_len"]), float(g["attn_scale"]))
    assert np.max(np.abs(got - g["attn_out"])) <= ATTN_ATOL


def test_attn_peaked_and_batched(ctx, checker):
    """Large score range (softmax close to one-hot) and batch > 1 with separate caches."""
    rng = np.random.default_rng(77)
    n_q, n_kv, d, kv, batch = 32, 8, 128, 333, 3
    q = (rng.standard_normal((batch, n_q, d)) * 8).astype(np.float32)
    k = rng.standard_normal((batch, n_kv, kv, d)).astype(np.float16)
    v = rng.standard_normal((batch, n_kv, kv, d)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(d)))
    got = gpu_attn(ctx, q, k, v, kv, scale, batch=batch)
    for b in range(batch):
        want = checker.attn_gqa_f16(q[b], k[b], v[b], kv, scale)
        assert np.max(np.abs(got[b] - want)) <= ATTN_ATOL


def test_attn_long_context_property(ctx):
    """At 32K keys (too slow for the scalar oracle): attention over identical
    value rows returns that row, and splitting invariance holds for a cache whose
    second half is masked out by a very negative score."""
    rng = np.random.default_rng(3)
    n_q, n_kv, d, kv = 32, 8, 128, 32768
    q = rng.standard_normal((n_q, d)).astype(np.float32)
    k = (rng.standard_normal((n_kv, kv, d)) / np.sqrt(d)).astype(np.float16)
    row = rng.standard_normal((n_kv, 1, d)).astype(np.float16)
    v = np.broadcast_to(row, (n_kv, kv, d)).copy()
    got = gpu_attn(ctx, q, k, v, kv, 0.088)
    for h in range(n_q):
        assert np.max(np.abs(got[h] - row[h // 4, 0].astype(np.float32))) <= ATTN_ATOL


def test_glue_ops_vs_oracle(ctx, checker):
    rng = np.random.default_rng(12)
    n = 4096
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    u = rng.standard_normal(n).astype(np.float32)
    wn = rng.uniform(0.9, 1.1, n).astype(np.float32)
    xd, ud, wd = dev(x), dev(u), dev(wn)
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.rmsnorm(xd, wd, y, 1e-5, n); ctx.sync()
    want = checker.rmsnorm(wn, x, 1e-5)
    assert np.max(np.abs(y.cpu().numpy() - want) / (np.abs(want) + 1e-6)) < 1e-5   # tests/test_decode_ops.cpp:20-35
    ctx.add2(xd, ud, y, n); ctx.sync()
    assert np.array_equal(bits(y.cpu().numpy()), bits(checker.add2(x, u)))
    ctx.silu_mul(xd, ud, y, n); ctx.sync()
    want = checker.silu_mul(x, u)
    assert np.max(np.abs(y.cpu().numpy() - want)) <= 1e-5 * (1 + np.max(np.abs(want)))


@pytest.mark.parametrize("pos", [0, 1, 100, 8191])
def test_rope_kv_append_vs_oracle(ctx, checker, pos):
    rng = np.random.default_rng(pos + 1)
    n_q, n_kv, d, stride = 32, 8, 128, 8200
    q = rng.standard_normal(n_q * d).astype(np.float32)
    k = rng.standard_normal(n_kv * d).astype(np.float32)
    v = rng.standard_normal(n_kv * d).astype(np.float32)
    qd, kd, vd = dev(q), dev(k), dev(v)
    kc = torch.zeros((n_kv, stride, d), dtype=torch.float16, device="cuda")
    vc = torch.zeros((n_kv, stride, d), dtype=torch.float16, device="cuda")
    pd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ctx.rope_kv_append(qd, kd, vd, kc, vc, pd, n_q, n_kv, d, stride, 500000.0); ctx.sync()
    want_q = checker.rope(q, pos, n_q, d, 0, d, 500000.0)
    want_k = checker.rope(k, pos, n_kv, d, 0, d, 500000.0)
    # angles are bit-identical; cosf/sinf may differ from the host libm by a few ulp
    assert np.max(np.abs(qd.cpu().numpy() - want_q)) <= 2e-6 * np.max(np.abs(q)) + 1e-6
    got_k = kc[:, pos, :].cpu().numpy().astype(np.float32).ravel()
    assert np.max(np.abs(got_k - want_k.astype(np.float16).astype(np.float32))) <= 2e-3   # one f16 ulp at |k| < 4
    assert np.array_equal(vc[:, pos, :].cpu().numpy().ravel().view(np.uint16), v.astype(np.float16).view(np.uint16))
    # nothing else was touched
    assert int(torch.count_nonzero(kc).item()) <= n_kv * d and int(torch.count_nonzero(vc).item()) <= n_kv * d


def test_argmax_tie_rule_and_margin(ctx):
    rng = np.random.default_rng(6)
    n = 128256
    lg = rng.standard_normal(n).astype(np.float32)
    lg[777] = 9.0
    lg[90000] = 9.0            # tie: the lower index wins, margin 0
    ld = dev(lg)
    idx = torch.zeros(1, dtype=torch.int32, device="cuda")
    mg = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.argmax(ld, n, idx, mg); ctx.sync()
    assert int(idx.item()) == 777 and float(mg.item()) == 0.0
    lg[90000] = 8.5
    ld = dev(lg)
    torch.cuda.synchronize()
    ctx.argmax(ld, n, idx, mg); ctx.sync()
    assert int(idx.item()) == 777 and abs(float(mg.item()) - 0.5) < 1e-6


def test_exec_task_stream_dot(ctx, checker):
    """The task-level entry with a reference-layout Task record."""
    rng = np.random.default_rng(10)
    rows, cols = 192, 4096            # one tile as the reference's builder emits (decoder.cpp:713-716)
    w = synth.q4k_tensor(rng, rows, cols)
    x = rng.standard_normal(cols).astype(np.float32)
    wd, xd = dev(w), dev(x)
    yd = torch.zeros(rows, dtype=torch.float32, device="cuda")
    t = capi.Task()
    t.kind, t.fmt = 0, capi.Q4_K
    t.w, t.w_bytes, t.x, t.y = wd.data_ptr(), rows * capi.row_bytes(capi.Q4_K, cols), xd.data_ptr(), yd.data_ptr()
    t.rows, t.cols, t.nx = rows, cols, 1
    torch.cuda.synchronize()
    ctx.exec_task(t); ctx.sync()
    assert rel_err(yd.cpu().numpy(), checker.matvec(capi.Q4_K, w, rows, cols, x)) <= MATVEC_RTOL
    t.w_bytes += 1                    # freeze() rule: w_bytes must equal rows * row_bytes
    with pytest.raises(capi.Fl200Error):
        ctx.exec_task(t)


@pytest.mark.parametrize("fmt,rows,cols,nx", [
    (capi.Q6_K, 1024, 4096, 2), (capi.Q6_K, 1024, 4096, 4), (capi.Q6_K, 4096, 4096, 8), (capi.Q6_K, 320, 4096, 9),
    (capi.Q6_K, 512, 14336, 8),      # rows of ffn_down: the columns span several resident chunks of the activation
    (capi.Q6_K, 100, 14336, 5), (capi.Q6_K, 37, 6144, 3),
    (capi.Q4_K, 256, 14336, 8), (capi.Q4_K, 37, 2048, 3), (capi.Q4_K, 1029, 4096, 6), (capi.Q4_K, 64, 768, 2),
])
def test_stream_dot_multi_column_both_formats(ctx, checker, fmt, rows, cols, nx):
    multi_column_case(ctx, checker, fmt, rows, cols, nx)


@pytest.mark.parametrize("rows,cols,nx", [
    (256, 14336, 8),      # two row tiles, the k range split over several work items (partial results through the ticket)
    (4096, 4096, 8), (1029, 4096, 6), (37, 2048, 3), (64, 768, 2), (300, 14336, 9), (128, 512, 8),
])
def test_stream_dot_multi_column_tcgen05(ctx, checker, monkeypatch, rows, cols, nx):
    """The same contract on the tcgen05 kernel (accumulator in tensor memory, split-K with ordered partial sums), which
    is off by default: FLB_UMMA=1 is read at every call."""
    monkeypatch.setenv("FLB_UMMA", "1")
    multi_column_case(ctx, checker, capi.Q4_K, rows, cols, nx)


def multi_column_case(ctx, checker, fmt, rows, cols, nx):
    """Task::nx > 1 on Q6_K as well as Q4_K tensors (draft verification, prompt chunks): all columns in one pass over
    the weights (up to 8 at a time); every column equals the reference's STREAM_DOT of that column, accumulate and
    assign-after-zero alike; ragged row counts, column counts that are not a multiple of 2048, strides with gaps."""
    rng = np.random.default_rng(7 * rows + cols + nx + fmt)
    w = synth.quant_tensor(fmt, rng, rows, cols)
    xstride, ystride = cols + 64, rows + 16
    x = rng.standard_normal((nx, xstride)).astype(np.float32)
    x[:, cols:] = np.nan                                   # the gap between columns is never read
    x[1] *= 1000.0                                         # columns with very different scales
    x[0, 300] *= 1e3                                       # and one outlier inside a block
    y0 = rng.standard_normal((nx, ystride)).astype(np.float32)
    want = y0.copy()
    deq = checker.dequant(fmt, w, rows, cols).astype(np.float64)
    for p in range(nx):
        want[p, :rows] += checker.matvec(fmt, w, rows, cols, x[p, :cols].copy())
    wd, xd, yd = dev(w), dev(x), dev(y0)
    torch.cuda.synchronize()
    ctx.matvec(fmt, wd, rows, cols, xd, yd, nx=nx, xstride=xstride, ystride=ystride)
    ctx.sync()
    assert ctx.status() == 0
    got = yd.cpu().numpy()
    assert np.array_equal(got[:, rows:], y0[:, rows:])     # nothing outside the rows is touched
    for p in range(nx):
        if p == 0:   # the outlier column: against the exact product (the f32 oracle rounds at the outlier's magnitude)
            ref = y0[p, :rows] + deq @ x[p, :cols].astype(np.float64)
            x0 = x[p, :cols].astype(np.float64); x0[300] = 0.0
            base = deq @ x0
            floor = 0.1 * np.sqrt(np.mean(base ** 2))
            err = float(np.max(np.abs(got[p, :rows] - ref) / np.maximum(np.abs(base), floor)))
            slack = float(np.max(np.abs(ref)) * 2.0 ** -22 / floor)
            assert err <= MATVEC_RTOL + slack, (p, err, slack)
        else:
            assert rel_err(got[p, :rows] - y0[p, :rows], want[p, :rows] - y0[p, :rows]) <= MATVEC_RTOL, p
    # run-to-run reproducible
    yd2 = dev(y0)
    torch.cuda.synchronize()
    ctx.matvec(fmt, wd, rows, cols, xd, yd2, nx=nx, xstride=xstride, ystride=ystride)
    ctx.sync()
    assert np.array_equal(bits(yd2.cpu().numpy()), bits(got))
