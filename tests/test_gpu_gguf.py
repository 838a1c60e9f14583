"""GPU tests of the GGUF loading path: a synthetic "llama" file written to disk,
loaded by the library into a decoder, against (a) a decoder handed the same
tensors directly (identical bits) and (b) the CPU oracle's decode step."""
import numpy as np
import pytest

from fast_llm_b200 import capi, gguf, synth
from fast_llm_b200.decoder import Decoder

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SMALL = dict(n_layer=2, n_embd=2048, n_head=16, n_kv_head=4, head_dim=128, n_ff=4096, n_vocab=1000, max_kv=64,
             rope_base=500000.0, eps=1e-5)
Q8_ALL = {k: capi.Q8_0 for k in synth.Q4_K_M}
MIXED = dict(synth.Q4_K_M, wk=capi.Q8_0, up=capi.Q6_K, tok_embd=capi.Q4_K)   # launches that mix formats
LOGIT_TOL = 3e-3


def host_model(cfg, seed, recipe):
    layers = []
    for l in range(cfg["n_layer"]):
        L = {n: (recipe[n], synth.llama_tensor(cfg, seed, n, l, recipe)) for n in synth.LAYER_TENSORS}
        L["attn_norm"] = synth.llama_norm(cfg, seed, "attn_norm", l)
        L["ffn_norm"] = synth.llama_norm(cfg, seed, "ffn_norm", l)
        layers.append(L)
    return dict(layers=layers, tok_embd=(recipe["tok_embd"], synth.llama_tensor(cfg, seed, "tok_embd", None, recipe)),
                output=(recipe["output"], synth.llama_tensor(cfg, seed, "output", None, recipe)),
                out_norm=synth.llama_norm(cfg, seed, "out_norm"))


def fill(target, model, tied, to_dev):
    """Hands the model to a Decoder or a LlamaOracle through their common set_* interface."""
    for l, L in enumerate(model["layers"]):
        for i, n in enumerate(synth.LAYER_TENSORS):
            target.set_layer_tensor(l, i, L[n][0], to_dev(L[n][1]))
        target.set_layer_norms(l, to_dev(L["attn_norm"]), to_dev(L["ffn_norm"]))
    target.set_global(capi.G_TOK_EMBD, model["tok_embd"][0], to_dev(model["tok_embd"][1]))
    head = model["tok_embd"] if tied else model["output"]
    target.set_global(capi.G_OUTPUT, head[0], to_dev(head[1]))
    target.set_out_norm(to_dev(model["out_norm"]))


def rel_err(got, want):
    return float(np.max(np.abs(got - want)) / (np.sqrt(np.mean(want.astype(np.float64) ** 2)) + 1e-30))


@pytest.mark.parametrize("recipe,tied,alignment,parts", [(synth.Q4_K_M, False, None, 1), (synth.Q4_K_M, True, 64, 1),
                                                          (Q8_ALL, False, None, 1), (MIXED, False, 32, 3)])
def test_decoder_from_file(ctx, checker, tmp_path, recipe, tied, alignment, parts):
    from oracle import pyoracle
    model = host_model(SMALL, 21, recipe)
    if parts == 1:
        path = tmp_path / "m.gguf"
        gguf.write_llama_gguf(path, SMALL, model, tie_output=tied, alignment=alignment)
    else:
        kv, recs = gguf.llama_records(SMALL, model, tied)
        path = gguf.write_split(str(tmp_path / "m"), kv, recs, parts, alignment=alignment)[0]
    with gguf.Gguf(path) as g:
        assert g.counts()[1] == parts
        dec = Decoder.from_gguf(ctx, g, SMALL["max_kv"])
    dec.finalize()                       # the file is closed: the decoder holds its own copies
    direct = Decoder(ctx, SMALL)
    fill(direct, model, tied, lambda a: torch.from_numpy(a).cuda())
    torch.cuda.synchronize()
    direct.finalize()
    orc = pyoracle.LlamaOracle(checker, SMALL)
    fill(orc, model, tied, lambda a: a)
    tok = 7
    for step in range(4):
        a, b, want_tok = dec.step(tok), direct.step(tok), orc.step(tok)
        la, lb, want = dec.logits(), direct.logits(), orc.logits()
        assert a == b and np.array_equal(la.view(np.uint32), lb.view(np.uint32)), step
        assert np.all(np.isfinite(la))
        # from the second step on each side reads its own f16 cache rows (last-bit differences before the
        # rounding become 5e-4 relative differences of single cache elements)
        assert rel_err(la, want) < (LOGIT_TOL if step == 0 else 3 * LOGIT_TOL), (step, rel_err(la, want))
        if a != want_tok:
            assert orc.margin() <= 2 * np.max(np.abs(la - want))
        tok = want_tok
    dec.close(); direct.close(); orc.close()


def test_file_the_decoder_cannot_run(ctx, tmp_path):
    model = host_model(SMALL, 22, synth.Q4_K_M)
    kv, recs = gguf.llama_records(SMALL, model)
    cases = {
        "missing": [r for r in recs if r[0] != "blk.1.ffn_up.weight"],
        "shape": [(n, t, ([d[0], d[1] - 1] if n == "blk.0.attn_k.weight" else d), p) for n, t, d, p in recs],
        "type": [(n, (gguf.GGML_F16 if n == "blk.0.attn_norm.weight" else t), d, p) for n, t, d, p in recs],
        "q5": [(n, (gguf.GGML_Q5_0 if n == "blk.0.attn_q.weight" else t), d,
                (bytes(d[1] * capi.row_bytes(capi.Q5_0, d[0])) if n == "blk.0.attn_q.weight" else p)) for n, t, d, p in recs],
    }
    for name, bad in cases.items():
        path = tmp_path / (name + ".gguf")
        gguf.write_gguf(path, kv, bad)
        with gguf.Gguf(path) as g, pytest.raises(capi.Fl200Error) as e:
            Decoder.from_gguf(ctx, g, 32)
        assert e.value.code == 6, name
    # a group size the attention kernel is not built for is refused by the decoder itself
    kv8 = [(k, t, (2 if k == "llama.attention.head_count_kv" else v)) for k, t, v in kv]
    path = tmp_path / "group8.gguf"
    gguf.write_gguf(path, kv8, recs)
    with gguf.Gguf(path) as g, pytest.raises(capi.Fl200Error) as e:
        Decoder.from_gguf(ctx, g, 32)
    assert e.value.code == 1
