"""GPU parity tests of decode attention at the shapes of the other benchmark
configurations: the long-context sweep (KV 32K / 64K / 128K, batch 1 / 4 / 16,
32 query heads over 8 KV heads, K/V ~ N(0,1)/sqrt(128)) and draft verification
(causal within a draft of k tokens on top of a 4096-token cache).

The scalar CPU oracle is used where it finishes in seconds; the larger cases are
checked against a plain PyTorch fp32 attention on the same device (the gate is
the attention gate, 2e-3 max-abs) and through splitting invariance."""
import numpy as np
import pytest

from fast_llm_b200 import capi

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ATTN_ATOL = 2e-3
SCALE = float(1.0 / np.sqrt(128.0))


def torch_ref(q, k16, v16, kv_len):
    """q [B][32][128] f32, k16 / v16 [B][8][stride][128] f16 -> [B][32][128] f32, plain softmax attention."""
    B = q.shape[0]
    k = k16[:, :, :kv_len].float().repeat_interleave(4, dim=1)     # [B][32][kv][128]
    v = v16[:, :, :kv_len].float().repeat_interleave(4, dim=1)
    s = torch.einsum("bhd,bhkd->bhk", q, k) * SCALE
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhk,bhkd->bhd", p, v)


def make_kv(seed, batch, kv, stride):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((batch, 32, 128), generator=g, device="cuda")
    k = (torch.randn((batch, 8, stride, 128), generator=g, device="cuda") * SCALE).half()
    v = (torch.randn((batch, 8, stride, 128), generator=g, device="cuda") * SCALE).half()
    return q, k, v


@pytest.mark.parametrize("kv,batch", [(32768, 1), (32768, 16), (65536, 4), (131072, 1), (131072, 4)])
def test_long_context_vs_torch_fp32(ctx, kv, batch):
    q, k, v = make_kv(kv + batch, batch, kv, kv)
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    ctx.attn_decode(q, k.view(torch.int16), v.view(torch.int16), 32, 8, 128, kv, kv, batch, SCALE, out)
    ctx.sync()
    assert ctx.status() == 0
    want = torch_ref(q, k, v, kv)
    assert float((out - want).abs().max()) <= ATTN_ATOL
    # ragged length inside the same cache: the rows past kv_len must not matter
    kv2 = kv - 777
    k[:, :, kv2:] = float("nan")
    out2 = torch.zeros_like(q)
    torch.cuda.synchronize()
    ctx.attn_decode(q, k.view(torch.int16), v.view(torch.int16), 32, 8, 128, kv2, kv, batch, SCALE, out2)
    ctx.sync()
    k[:, :, kv2:] = 0
    want2 = torch_ref(q, k, v, kv2)
    assert float((out2 - want2).abs().max()) <= ATTN_ATOL


def test_long_context_32k_vs_oracle(ctx, checker):
    """One sequence at 32K keys against the reference's one-head operator (a few seconds of CPU)."""
    rng = np.random.default_rng(32)
    kv = 32768
    q = rng.standard_normal((32, 128)).astype(np.float32)
    k = (rng.standard_normal((8, kv, 128)) * SCALE).astype(np.float16)
    v = (rng.standard_normal((8, kv, 128)) * SCALE).astype(np.float16)
    out = torch.zeros((32, 128), device="cuda")
    qd = torch.from_numpy(q).cuda()
    kd = torch.from_numpy(k.view(np.int16)).cuda(); vd = torch.from_numpy(v.view(np.int16)).cuda()
    torch.cuda.synchronize()
    ctx.attn_decode(qd, kd, vd, 32, 8, 128, kv, kv, 1, SCALE, out)
    ctx.sync()
    want = checker.attn_gqa_f16(q, k, v, kv, SCALE)
    assert float(np.max(np.abs(out.cpu().numpy() - want))) <= ATTN_ATOL


@pytest.mark.parametrize("n_draft,base", [(8, 4096), (4, 4096), (2, 100), (1, 63), (8, 57)])
def test_verify_attention_causal_within_draft(ctx, checker, n_draft, base):
    """Query b of the draft sees keys 0 .. base + b of one shared cache: equal to one decode call per
    draft position (the reference's fl_op_attn_head with pos = base + b)."""
    rng = np.random.default_rng(n_draft * 1000 + base)
    stride = base + n_draft + 5
    q = rng.standard_normal((n_draft, 32, 128)).astype(np.float32)
    k = (rng.standard_normal((8, stride, 128)) * SCALE).astype(np.float16)
    v = (rng.standard_normal((8, stride, 128)) * SCALE).astype(np.float16)
    k[:, base + n_draft:] = np.nan                       # never attended
    qd = torch.from_numpy(q).cuda()
    kd = torch.from_numpy(k.view(np.int16)).cuda(); vd = torch.from_numpy(v.view(np.int16)).cuda()
    out = torch.zeros((n_draft, 32, 128), device="cuda")
    torch.cuda.synchronize()
    ctx.attn_verify(qd, kd, vd, 32, 8, 128, base + 1, stride, n_draft, SCALE, out)
    ctx.sync()
    assert ctx.status() == 0
    got = out.cpu().numpy()
    for b in range(n_draft):
        want = checker.attn_gqa_f16(q[b], k, v, base + 1 + b, SCALE)
        assert float(np.max(np.abs(got[b] - want))) <= ATTN_ATOL, b
        # and bit-identical to the single-sequence entry point with the same length
        one = torch.zeros((32, 128), device="cuda")
        torch.cuda.synchronize()
        ctx.attn_decode(qd[b].contiguous(), kd, vd, 32, 8, 128, base + 1 + b, stride, 1, SCALE, one)
        ctx.sync()
        if n_draft == 1:
            assert np.array_equal(one.cpu().numpy().view(np.uint32), got[b].view(np.uint32))
        else:
            assert float(np.max(np.abs(one.cpu().numpy() - got[b]))) <= 1e-5   # the split plan may differ
