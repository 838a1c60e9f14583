"""GPU test of fl_b200_attn_decode_static: decode attention whose split-KV
scratch is a fixed array inside the library instead of context-owned heap
memory. Called through the C ABI and compared with fl_b200_attn_decode on the
same inputs. The file sorts last so that it also runs after every other GPU
test has used the library (and the shared scratch) in the same process; it does
not depend on them and passes alone."""
import numpy as np
import pytest

from fast_llm_b200 import capi

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _inputs(seed, n_kv, kv_len, kv_stride, batch):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((batch, 4 * n_kv, 128), generator=g, device="cuda", dtype=torch.float32)
    k = (0.5 * torch.randn((batch, n_kv, kv_stride, 128), generator=g, device="cuda")).to(torch.float16)
    v = torch.randn((batch, n_kv, kv_stride, 128), generator=g, device="cuda").to(torch.float16)
    # rows past kv_len must never be read: poison them
    k[:, :, kv_len:] = float("nan")
    v[:, :, kv_len:] = float("nan")
    return q, k.view(torch.int16), v.view(torch.int16)


@pytest.mark.parametrize("n_kv,kv_len,kv_stride,batch", [(8, 8192, 8192, 1), (8, 300, 1024, 1), (2, 1, 64, 1),
                                                         (4, 777, 1024, 3)])
def test_static_scratch_matches_heap_scratch_twice(ctx, n_kv, kv_len, kv_stride, batch):
    q, k, v = _inputs(11 + kv_len, n_kv, kv_len, kv_stride, batch)
    scale = 1.0 / np.sqrt(128.0)
    want = torch.zeros_like(q)
    torch.cuda.synchronize()
    ctx.attn_decode(q, k, v, 4 * n_kv, n_kv, 128, kv_len, kv_stride, batch, scale, want)
    ctx.sync()
    want = want.cpu().numpy()
    assert np.all(np.isfinite(want))
    # two calls in a row share the array: the second must not see anything the first left behind
    for call in range(2):
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        ctx.attn_decode_static(q, k, v, 4 * n_kv, n_kv, 128, kv_len, kv_stride, batch, scale, got)
        ctx.sync()
        assert ctx.status() == 0
        # same kernel, same split plan, partials combined in split order: identical bits
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), call
    # and back to back without a host synchronisation in between (stream order protects the array)
    a, b = torch.zeros_like(q), torch.zeros_like(q)
    q2 = q * 0.5
    want2 = torch.zeros_like(q)
    torch.cuda.synchronize()
    ctx.attn_decode_static(q, k, v, 4 * n_kv, n_kv, 128, kv_len, kv_stride, batch, scale, a)
    ctx.attn_decode_static(q2, k, v, 4 * n_kv, n_kv, 128, kv_len, kv_stride, batch, scale, b)
    ctx.attn_decode(q2, k, v, 4 * n_kv, n_kv, 128, kv_len, kv_stride, batch, scale, want2)
    ctx.sync()
    assert np.array_equal(a.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(b.cpu().numpy().view(np.uint32), want2.cpu().numpy().view(np.uint32))


def test_static_scratch_against_oracle(ctx, checker):
    from fast_llm_b200 import synth
    c0 = synth.config0(0)
    q = torch.from_numpy(c0["q"]).cuda()
    k = torch.from_numpy(c0["k"].view(np.uint16).astype(np.int16)).cuda()
    v = torch.from_numpy(c0["v"].view(np.uint16).astype(np.int16)).cuda()
    out = torch.zeros((32, 128), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx.attn_decode_static(q, k, v, 32, 8, 128, 300, 1024, 1, c0["scale"], out)
    ctx.sync()
    want = checker.attn_gqa_f16(c0["q"], c0["k"], c0["v"], 300, c0["scale"])
    assert float(np.max(np.abs(out.cpu().numpy() - want))) <= 2e-3   # the attention gate: max abs 2e-3


def test_static_scratch_rejects_oversize(ctx):
    # 64 sequences x 8 KV heads = 512 (KV head, sequence) pairs; the array has 256 counters
    n_kv, batch, kv_len = 8, 64, 4096
    q = torch.zeros((batch, 32, 128), device="cuda")
    k = torch.zeros((batch, n_kv, kv_len, 128), device="cuda", dtype=torch.float16).view(torch.int16)
    out = torch.full_like(q, 7.0)
    torch.cuda.synchronize()
    with pytest.raises(capi.Fl200Error) as e:
        ctx.attn_decode_static(q, k, k, 32, n_kv, 128, kv_len, kv_len, batch, 0.1, out)
    assert "fixed scratch" in str(e.value)
    ctx.sync()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0       # nothing was launched
    # the limit does not depend on kv_len
    with pytest.raises(capi.Fl200Error):
        ctx.attn_decode_static(q, k, k, 32, n_kv, 128, 1, kv_len, 64, 0.1, out)
    # the heap-scratch entry point takes the same call
    ctx.attn_decode(q, k, k, 32, n_kv, 128, kv_len, kv_len, batch, 0.1, out)
    ctx.sync()
    assert float(out.abs().max()) == 0.0
