"""GPU parity tests of a decoder with mixture-of-experts layers (Mixtral shape: attention as in the dense
model, the feed-forward block replaced by router -> top-k experts -> weighted merge; the chain the reference's graph
builder emits per MoE layer, src/model/decoder.cpp:925-1045) against the CPU oracle's step on identical weights."""
import numpy as np
import pytest

from fast_llm_b200 import capi, synth
from fast_llm_b200.moe import MoeBlock
from test_gpu_decoder import build_pair, force_kv, logits_close, LOGIT_TOL, HIDDEN_TOL

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# two MoE layers around a dense one; the query width equals n_embd (the block's output borrows the query buffer)
CFG = dict(n_layer=3, n_embd=2048, n_head=16, n_kv_head=4, head_dim=128, n_ff=4096, n_vocab=1000, max_kv=96,
           rope_base=500000.0, eps=1e-5)
MOE_LAYERS = (0, 2)
NE, K, F = 4, 2, 1024


def build_moe_pair(ctx, checker, seed, n_prefill, fmt_down=capi.Q4_K, max_tokens=8):
    """build_pair's dense model, then layers MOE_LAYERS get an expert block on both sides (their dense gate / up / down
    stay set on the oracle side and are simply not used there either)."""
    dec, orc = build_pair(ctx, checker, CFG, seed, n_prefill, finalize=False)
    blocks = []
    for l in MOE_LAYERS:
        rng = synth.rng_for(seed, "L%d.moe" % l)
        E = CFG["n_embd"]
        wg = synth.q4k_tensor(rng, NE * F, E); wu = synth.q4k_tensor(rng, NE * F, E)
        wd = synth.quant_tensor(fmt_down, rng, NE * E, F)
        wr = rng.standard_normal((NE, E)).astype(np.float32)     # wide logits: no near-ties between experts
        blk = MoeBlock(ctx, E, F, NE, K, norm=1, scale=1.0, fmt_gate_up=capi.Q4_K, fmt_down=fmt_down, max_tokens=max_tokens)
        blk.set_weights(*(torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (wr, wg, wu, wd)))
        dec.set_layer_moe(l, blk)
        orc.set_layer_moe(l, NE, K, 1, 1.0, F, wr, capi.Q4_K, wg, wu, fmt_down, wd)
        blocks.append(blk)
    torch.cuda.synchronize()
    dec.finalize()
    dec.rewind_to(n_prefill)
    orc.set_n_past(n_prefill)
    return dec, orc, blocks


@pytest.mark.parametrize("fmt_down", [capi.Q4_K, capi.Q6_K])
def test_moe_model_teacher_forced(ctx, checker, fmt_down):
    dec, orc, blocks = build_moe_pair(ctx, checker, seed=11, n_prefill=30, fmt_down=fmt_down)
    tok = 7
    for step in range(8):
        want_tok = orc.step(tok)
        got_tok = dec.step(tok)
        got, want = dec.logits(), orc.logits()
        assert np.all(np.isfinite(got)) and ctx.status() == 0
        err = logits_close(got, want)
        assert err < LOGIT_TOL, (step, err)
        if got_tok != want_tok:
            assert orc.margin() <= 2 * np.max(np.abs(got - want)), (step, got_tok, want_tok, orc.margin())
        assert logits_close(dec.tap(0), orc.hidden()) < HIDDEN_TOL
        # the last MoE layer routed to the experts the oracle chose
        ids, gates = blocks[-1].routing(1)
        assert sorted(ids[0]) == sorted(int(i) for i in np.ctypeslib.as_array(orc.p.flo_llama_moe_ids(orc.h), shape=(K,)))
        force_kv(ctx, dec, orc, CFG, 30 + step)
        tok = want_tok
    # the step's bytes: attention tensors of every layer, dense FFN of layer 1, router + K experts of the MoE layers
    wb, _ = dec.bytes_per_step(30)
    E, QD, KD = CFG["n_embd"], CFG["n_head"] * 128, CFG["n_kv_head"] * 128
    rb = capi.row_bytes
    attn = QD * rb(capi.Q4_K, E) + KD * rb(capi.Q4_K, E) + KD * rb(capi.Q6_K, E) + E * rb(capi.Q4_K, QD) + 2 * E * 4
    dense = 2 * CFG["n_ff"] * rb(capi.Q4_K, E) + E * rb(capi.Q6_K, CFG["n_ff"])
    moe = NE * E * 4 + K * (2 * F * rb(capi.Q4_K, E) + E * rb(fmt_down, F))
    assert wb == 3 * attn + dense + 2 * moe + CFG["n_vocab"] * rb(capi.Q6_K, E) + E * 4
    dec.close(); orc.close()


def test_moe_model_run_and_batch_pass(ctx, checker):
    """Device feedback equals step-by-step calls; the batch pass (every expert once for the tokens that chose it)
    gives the tokens of single steps."""
    dec, orc, _ = build_moe_pair(ctx, checker, seed=13, n_prefill=12)
    toks = [int(t) for t in dec.run(3, 6)]
    dec.rewind_to(12)
    t, seq = 3, []
    for _ in range(6):
        t = dec.step(t)
        seq.append(t)
    assert toks == seq
    dec.rewind_to(12)
    outs, margins = dec.step_batch([3] + seq[:5])          # teacher-forced inputs: 3, a0 .. a4
    for i, (o, mg) in enumerate(zip(outs, margins)):
        assert o == seq[i] or mg < 1e-2, (i, o, seq[i], mg)
    dec.close(); orc.close()
