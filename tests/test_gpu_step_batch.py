"""GPU tests of the decoder's batch pass (Decoder::step_batch of the reference:
m tokens at consecutive positions in one pass) against the same tokens fed one
by one, and against the CPU oracle's steps."""
import numpy as np
import pytest

from fast_llm_b200 import capi, synth
from fast_llm_b200.decoder import Decoder

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

# SMALL: no tensor qualifies for the multi-column kernel (2048 columns); WIDE: wq, wk, wo, gate, up do.
SMALL = dict(n_layer=2, n_embd=2048, n_head=16, n_kv_head=4, head_dim=128, n_ff=4096, n_vocab=1000, max_kv=96,
             rope_base=500000.0, eps=1e-5)
WIDE = dict(n_layer=2, n_embd=4096, n_head=32, n_kv_head=8, head_dim=128, n_ff=4096, n_vocab=1024, max_kv=96,
            rope_base=500000.0, eps=1e-5)
TOL = 3e-3


def build(ctx, checker, cfg, seed, n_prefill, with_oracle=True):
    from oracle import pyoracle
    dec = Decoder(ctx, cfg)
    orc = pyoracle.LlamaOracle(checker, cfg) if with_oracle else None
    for l in range(cfg["n_layer"]):
        for i, name in enumerate(synth.LAYER_TENSORS):
            w = synth.llama_tensor(cfg, seed, name, l)
            dec.set_layer_tensor(l, i, synth.Q4_K_M[name], torch.from_numpy(w).cuda())
            if orc:
                orc.set_layer_tensor(l, i, synth.Q4_K_M[name], w)
        an, fn = synth.llama_norm(cfg, seed, "attn_norm", l), synth.llama_norm(cfg, seed, "ffn_norm", l)
        dec.set_layer_norms(l, torch.from_numpy(an).cuda(), torch.from_numpy(fn).cuda())
        if orc:
            orc.set_layer_norms(l, an, fn)
        if n_prefill:
            k, v = synth.llama_kv(cfg, seed, l, n_prefill)
            if orc:
                orc.seed_kv(l, k, v)
            for src, dst in zip((k, v), dec.kv_ptrs(l)):
                full = np.zeros((cfg["n_kv_head"], cfg["max_kv"], cfg["head_dim"]), dtype=np.float16)
                full[:, :n_prefill] = src
                capi._ck(ctx.lib.fl_b200_upload(ctx._h, capi.C.c_void_p(dst), capi.C.c_void_p(full.ctypes.data),
                                                capi.C.c_size_t(full.nbytes)))
    for which, name in ((capi.G_TOK_EMBD, "tok_embd"), (capi.G_OUTPUT, "output")):
        w = synth.llama_tensor(cfg, seed, name)
        dec.set_global(which, synth.Q4_K_M[name], torch.from_numpy(w).cuda())
        if orc:
            orc.set_global(which, synth.Q4_K_M[name], w)
    on = synth.llama_norm(cfg, seed, "out_norm")
    dec.set_out_norm(torch.from_numpy(on).cuda())
    if orc:
        orc.set_out_norm(on)
        orc.set_n_past(n_prefill)
    torch.cuda.synchronize()
    dec.finalize()
    dec.rewind_to(n_prefill)
    return dec, orc


def rel_err(got, want):
    return float(np.max(np.abs(got - want)) / (np.sqrt(np.mean(want.astype(np.float64) ** 2)) + 1e-30))


@pytest.mark.parametrize("cfg,m", [(SMALL, 5), (WIDE, 8), (WIDE, 3), (WIDE, 1), (WIDE, 16), (SMALL, 11)])
def test_batch_pass_equals_single_steps_and_oracle(ctx, checker, cfg, m):
    n_prefill = 37
    dec, orc = build(ctx, checker, cfg, seed=31, n_prefill=n_prefill)
    rng = np.random.default_rng(5)
    toks = [int(t) for t in rng.integers(0, cfg["n_vocab"], m)]
    outs, margins = dec.step_batch(toks)
    assert dec.n_past() == n_prefill + m
    batch_logits = [dec.batch_logits(i) for i in range(m)]
    # the same tokens one by one from the same start (the pass's cache rows are overwritten before they are read)
    dec.rewind_to(n_prefill)
    for i, t in enumerate(toks):
        nxt = dec.step(t)
        single = dec.logits()
        err = rel_err(batch_logits[i], single)
        assert err < TOL, (i, err)
        if nxt != outs[i]:
            assert dec.last_margin() <= 2 * np.max(np.abs(batch_logits[i] - single)), (i, nxt, outs[i])
        assert abs(margins[i] - dec.last_margin()) <= 4 * np.max(np.abs(batch_logits[i] - single)) + 1e-6
        want_tok = orc.step(t)
        want = orc.logits()
        assert np.all(np.isfinite(batch_logits[i]))
        # position 0 sees only prefilled keys; later positions read rows whose f16 rounding may differ from the oracle's
        assert rel_err(batch_logits[i], want) < (TOL if i == 0 else 3 * TOL), (i, rel_err(batch_logits[i], want))
        if i == 0 and want_tok != outs[0]:
            assert orc.margin() <= 2 * np.max(np.abs(batch_logits[0] - want))
    assert ctx.status() == 0
    dec.close(); orc.close()


def test_batch_pass_rules(ctx, checker):
    dec, _ = build(ctx, checker, SMALL, seed=32, n_prefill=0, with_oracle=False)
    with pytest.raises(capi.Fl200Error) as e:
        dec.step_batch([])
    assert e.value.code == 1
    with pytest.raises(capi.Fl200Error) as e:
        dec.step_batch([1] * 17)
    assert e.value.code == 1
    with pytest.raises(capi.Fl200Error) as e:
        dec.step_batch([1, SMALL["n_vocab"]])
    assert e.value.code == 1
    dec.rewind_to(SMALL["max_kv"] - 3)
    with pytest.raises(capi.Fl200Error) as e:
        dec.step_batch([1, 2, 3, 4])
    assert e.value.code == 4
    assert dec.n_past() == SMALL["max_kv"] - 3
    # prompt ingestion in chunks, then greedy decoding: same tokens as feeding the prompt one by one
    prompt = [3, 14, 15, 92, 65, 35, 89, 79, 32, 38, 46]
    dec.rewind_to(0)
    for i in range(0, len(prompt), 8):
        outs, _ = dec.step_batch(prompt[i:i + 8])
    a = [outs[-1]] + [int(t) for t in dec.run(outs[-1], 4)]
    dec.rewind_to(0)
    for t in prompt:
        nxt = dec.step(t)
    b = [nxt] + [int(t) for t in dec.run(nxt, 4)]
    assert a == b
    dec.close()


def test_speculative_generation_equals_greedy(ctx, checker):
    """The speculative loop emits the greedy sequence whatever the drafts are worth;
    only the number of passes changes."""
    from fast_llm_b200 import spec
    n_prefill, n_gen, first = 20, 40, 5
    dec, _ = build(ctx, checker, SMALL, seed=33, n_prefill=n_prefill, with_oracle=False)
    greedy = [first] + [int(t) for t in dec.run(first, n_gen - 1)]

    def gen(index, **kw):
        dec.rewind_to(n_prefill)
        toks, st = spec.generate(dec, first, n_gen, index, **kw)
        assert st.emitted == n_gen and st.accepted <= st.drafted
        # every pass yields its own token plus the accepted drafts (the last pass may overshoot n_gen)
        assert sum(st.n_hist) == st.passes and n_gen - 1 <= st.passes + st.accepted <= n_gen - 1 + 7
        return toks, st

    # an empty history: drafts come only from repetitions of the generated text itself
    toks, st = gen(spec.SuffixIndex(), spec_fixed=4)
    assert toks == greedy
    toks, st = gen(spec.SuffixIndex(), spec_fixed=0)
    assert toks == greedy and st.drafted == 0 and st.passes == n_gen - 1
    # the text was seen before: drafts are right, a pass emits several tokens
    seen = spec.SuffixIndex()
    for t in greedy:
        seen.push(t)
    toks, st = gen(seen, spec_fixed=7)
    assert toks == greedy
    assert st.accepted >= 25 and st.passes <= 12, (st.accepted, st.passes)
    # a misleading history: the same opening, then something else; every draft is rejected at some point
    wrong = spec.SuffixIndex()
    for t in greedy[:6] + [(t + 1) % SMALL["n_vocab"] for t in greedy[6:]]:
        wrong.push(t)
    toks, st = gen(wrong, spec_fixed=7)
    assert toks == greedy and st.drafted > 0 and st.accepted < st.drafted
    # the controller decides the draft length
    seen2 = spec.SuffixIndex()
    for t in greedy:
        seen2.push(t)
    ctrl = spec.SpecController()
    toks, st = gen(seen2, ctrl=ctrl)
    assert toks == greedy and st.accepted > 0
    assert ctrl.alpha() > 0.75
    with pytest.raises(capi.Fl200Error):
        spec.generate(dec, first, 4, seen2, spec_max=16, spec_fixed=1)   # one more than the batch pass takes
    with pytest.raises(capi.Fl200Error):
        spec.generate(dec, first, 4, seen2)            # no controller and no fixed length
    assert ctx.status() == 0
    dec.close()


def _upload_kv(ctx, cfg, ptr, src, n_pos):
    full = np.zeros((cfg["n_kv_head"], cfg["max_kv"], cfg["head_dim"]), dtype=np.float16)
    full[:, :n_pos] = src
    capi._ck(ctx.lib.fl_b200_upload(ctx._h, capi.C.c_void_p(ptr), capi.C.c_void_p(full.ctypes.data), capi.C.c_size_t(full.nbytes)))


def _oracle_conditioning(orc, cfg, kv, n_hist, tokens, replay):
    """one_ulp_move of the oracle at the last of `tokens` after the history `kv` (replay: the oracle is first put
    through that history and the earlier tokens; otherwise it has just taken the step)."""
    if replay:
        for l in range(cfg["n_layer"]):
            orc.seed_kv(l, *kv[l])
        orc.set_n_past(n_hist)
        for t in tokens:
            orc.step(t)
    return orc.one_ulp_move(tokens[-1])


@pytest.mark.parametrize("cfg,n_seq", [(WIDE, 3), (SMALL, 2), (WIDE, 11)])
def test_independent_sequences_equal_single_steps_and_oracle(ctx, checker, cfg, n_seq):
    """n sequences with their own caches, histories of different lengths and their own tokens, one token each per pass:
    every sequence gets the tokens and logits it gets when it is decoded alone (single steps on the decoder's own
    cache), and sequence 0 those of the CPU oracle."""
    dec, orc = build(ctx, checker, cfg, seed=41, n_prefill=0)
    dec.seqs_init(n_seq)
    lens = [5 + 7 * s for s in range(n_seq)]
    kvs = []
    for s in range(n_seq):
        per_layer = []
        for l in range(cfg["n_layer"]):
            k, v = synth.llama_kv(cfg, 100 + s, l, lens[s])
            per_layer.append((k, v))
            for src, dst in zip((k, v), dec.seqs_kv_ptrs(l, s)):
                _upload_kv(ctx, cfg, dst, src, lens[s])
        kvs.append(per_layer)
        dec.seqs_set_pos(s, lens[s])
    rng = np.random.default_rng(9)
    n_steps = 4
    toks = rng.integers(0, cfg["n_vocab"], (n_steps, n_seq))
    got_tok, got_logits = [], []
    for st in range(n_steps):
        outs, margins = dec.seqs_step([int(t) for t in toks[st]])
        got_tok.append(outs)
        got_logits.append([dec.batch_logits(s) for s in range(n_seq)])
    assert [dec.seqs_pos(s) for s in range(n_seq)] == [n + n_steps for n in lens]
    assert ctx.status() == 0
    # every sequence alone, on the single-sequence cache, from the same history
    for s in range(n_seq):
        for l in range(cfg["n_layer"]):
            for src, dst in zip(kvs[s][l], dec.kv_ptrs(l)):
                _upload_kv(ctx, cfg, dst, src, lens[s])
        dec.rewind_to(lens[s])
        if s == 0:
            for l in range(cfg["n_layer"]):
                orc.seed_kv(l, *kvs[0][l])
            orc.set_n_past(lens[0])
        for st in range(n_steps):
            nxt = dec.step(int(toks[st][s]))
            single = dec.logits()
            if s == 0:
                want_tok = orc.step(int(toks[st][0]))
            err = rel_err(got_logits[st][s], single)
            if err >= TOL:
                # The two passes run different kernels (one column: integer form; several: f16 form), each within about
                # 1e-5 of the exact products. A step where the oracle's OWN logits move by `move` for a one-ulp change of
                # an input turns that into a difference of some hundred times `move`: the bound scales with it.
                move = _oracle_conditioning(orc, cfg, kvs[s], lens[s], [int(toks[i][s]) for i in range(st + 1)], replay=s != 0)
                assert err < TOL + 200 * move, (s, st, err, move)
            if nxt != got_tok[st][s]:
                assert dec.last_margin() <= 2 * np.max(np.abs(got_logits[st][s] - single)), (s, st)
            if s == 0:
                assert rel_err(got_logits[st][0], orc.logits()) < (TOL if st == 0 else 3 * TOL), (st,)
                if st == 0 and want_tok != got_tok[0][0]:
                    assert orc.margin() <= 2 * np.max(np.abs(got_logits[0][0] - orc.logits()))
    with pytest.raises(capi.Fl200Error):
        dec.seqs_init(4)                      # already set up
    dec.close(); orc.close()
