"""Tensor-parallel decoder on 2, 4 and 8 GPUs (one process per GPU) against the
same model on one GPU: identical greedy tokens, logits within the whole-step
tolerance. Each case is skipped on boxes with fewer GPUs than it needs."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SMALL = dict(n_layer=2, n_embd=2048, n_head=16, n_kv_head=4, head_dim=128, n_ff=4096, n_vocab=1000, max_kv=96,
             rope_base=500000.0, eps=1e-5)
# 8 ranks need 8 KV heads and at least 512 columns of O per rank
WIDE = dict(n_layer=2, n_embd=4096, n_head=32, n_kv_head=8, head_dim=128, n_ff=4096, n_vocab=1000, max_kv=96,
            rope_base=500000.0, eps=1e-5)
N_PREFILL, STEPS, SEED = 40, 6, 3
BATCH_TOKS = [11, 500, 7, 999, 123]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fill(dec, ctx, cfg, rank, world, prefill=True):
    """The seeded synthetic model, sliced for (rank, world)."""
    from fast_llm_b200 import capi, synth, tp
    for l in range(cfg["n_layer"]):
        for i, name in enumerate(synth.LAYER_TENSORS):
            fmt = synth.Q4_K_M[name]
            w = synth.llama_tensor(cfg, SEED, name, l)
            if world > 1:
                w = np.ascontiguousarray(tp.shard_tensor(name, w, fmt, cfg, rank, world))
            dec.set_layer_tensor(l, i, fmt, torch.from_numpy(w).cuda())
        an, fn = synth.llama_norm(cfg, SEED, "attn_norm", l), synth.llama_norm(cfg, SEED, "ffn_norm", l)
        dec.set_layer_norms(l, torch.from_numpy(an).cuda(), torch.from_numpy(fn).cuda())
        if not prefill:
            continue
        k, v = synth.llama_kv(cfg, SEED, l, N_PREFILL)
        nkv = cfg["n_kv_head"] // world
        kp, vp = dec.kv_ptrs(l)
        for src, dst in ((k, kp), (v, vp)):
            full = np.zeros((nkv, cfg["max_kv"], cfg["head_dim"]), dtype=np.float16)
            full[:, :N_PREFILL] = src[rank * nkv:(rank + 1) * nkv]
            capi._ck(ctx.lib.fl_b200_upload(ctx._h, capi.C.c_void_p(dst), capi.C.c_void_p(full.ctypes.data),
                                            capi.C.c_size_t(full.nbytes)))
    emb = synth.llama_tensor(cfg, SEED, "tok_embd")
    dec.set_global(capi.G_TOK_EMBD, synth.Q4_K_M["tok_embd"], torch.from_numpy(emb).cuda())
    head = synth.llama_tensor(cfg, SEED, "output")
    if world > 1:
        head = np.ascontiguousarray(tp.shard_tensor("output", head, synth.Q4_K_M["output"], cfg, rank, world))
    dec.set_global(capi.G_OUTPUT, synth.Q4_K_M["output"], torch.from_numpy(head).cuda())
    dec.set_out_norm(torch.from_numpy(synth.llama_norm(cfg, SEED, "out_norm")).cuda())
    torch.cuda.synchronize()


def _write_model_file(path):
    """The same seeded model as _fill's, as a "llama" GGUF file."""
    from fast_llm_b200 import gguf, synth
    layers = []
    for l in range(SMALL["n_layer"]):
        L = {n: (synth.Q4_K_M[n], synth.llama_tensor(SMALL, SEED, n, l)) for n in synth.LAYER_TENSORS}
        L["attn_norm"], L["ffn_norm"] = synth.llama_norm(SMALL, SEED, "attn_norm", l), synth.llama_norm(SMALL, SEED, "ffn_norm", l)
        layers.append(L)
    model = dict(layers=layers, tok_embd=(synth.Q4_K_M["tok_embd"], synth.llama_tensor(SMALL, SEED, "tok_embd")),
                 output=(synth.Q4_K_M["output"], synth.llama_tensor(SMALL, SEED, "output")),
                 out_norm=synth.llama_norm(SMALL, SEED, "out_norm"))
    gguf.write_llama_gguf(path, SMALL, model)


def _from_file_equals_sliced(rank, world, ctx, dist, path):
    """The slices the library cuts while it uploads a model file are the slices
    fast_llm_b200.tp cuts on the host: gathered logits of both decoders, bit for bit."""
    from fast_llm_b200 import gguf, tp
    from fast_llm_b200.decoder import Decoder
    a = Decoder(ctx, SMALL, tp=(rank, world))
    _fill(a, ctx, SMALL, rank, world, prefill=False)
    with gguf.Gguf(path) as g:
        b = Decoder.from_gguf(ctx, g, SMALL["max_kv"], tp=(rank, world))
    out = []
    for dec in (a, b):
        tp.connect(dec, dist)
        dec.finalize()
        dist.barrier()
        toks, tok = [], 5
        for _ in range(3):
            tok = dec.step(tok)
            toks.append(tok)
        sl = torch.from_numpy(dec.logits())
        parts = [torch.zeros_like(sl) for _ in range(world)]
        dist.all_gather(parts, sl)
        out.append((toks, torch.cat(parts).numpy()))
        dist.barrier()
    a.close(); b.close()
    return out[0][0] == out[1][0] and np.array_equal(out[0][1].view(np.uint32), out[1][1].view(np.uint32))


def _worker(rank, world, port, q, model_path=None, cfg=None):
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from fast_llm_b200 import capi, tp
        from fast_llm_b200.decoder import Decoder
        cfg = cfg or SMALL
        ctx = capi.Context(rank)
        dec = Decoder(ctx, cfg, tp=(rank, world))
        _fill(dec, ctx, cfg, rank, world)
        tp.connect(dec, dist)
        dec.finalize()
        dec.rewind_to(N_PREFILL)
        dist.barrier()
        res = {"tokens": [], "logits": [], "margin": []}
        tok = 11
        for _ in range(STEPS):
            tok = dec.step(tok)
            res["tokens"].append(tok)
            sl = torch.from_numpy(dec.logits())
            parts = [torch.zeros_like(sl) for _ in range(world)]
            dist.all_gather(parts, sl)
            res["logits"].append(torch.cat(parts).numpy())
            res["margin"].append(dec.last_margin())
        # device feedback loop: same tokens again from the same start
        dec.rewind_to(N_PREFILL)
        dist.barrier()
        res["run"] = [int(t) for t in dec.run(11, STEPS)]
        # the batch pass (Decoder::step_batch) on the tensor-parallel decoder: 5 tokens in one pass
        dec.rewind_to(N_PREFILL)
        dist.barrier()
        outs, margins = dec.step_batch(BATCH_TOKS)
        sl = torch.from_numpy(dec.batch_logits(len(BATCH_TOKS) - 1))
        parts = [torch.zeros_like(sl) for _ in range(world)]
        dist.all_gather(parts, sl)
        res["batch"] = (outs, margins, torch.cat(parts).numpy())
        dec.rewind_to(N_PREFILL)                             # a short pass runs as teacher-forced single steps
        dist.barrier()
        res["batch2"] = dec.step_batch(BATCH_TOKS[:2])
        res["status"] = ctx.status()
        dist.barrier()
        if rank == 0:   # the same model on one GPU
            one = Decoder(ctx, cfg)
            _fill(one, ctx, cfg, 0, 1)
            one.finalize()
            one.rewind_to(N_PREFILL)
            ref = {"tokens": [], "logits": [], "margin": []}
            tok = 11
            for _ in range(STEPS):
                tok = one.step(tok)
                ref["tokens"].append(tok)
                ref["logits"].append(one.logits())
                ref["margin"].append(one.last_margin())
            one.rewind_to(N_PREFILL)
            o1, m1 = one.step_batch(BATCH_TOKS)
            ref["batch"] = (o1, m1, one.batch_logits(len(BATCH_TOKS) - 1))
            res["ref"] = ref
            one.close()
        dist.barrier()
        dec.close()
        if model_path:
            res["file_equals_sliced"] = _from_file_equals_sliced(rank, world, ctx, dist, model_path)
        ctx.close()
        dist.destroy_process_group()
        q.put((rank, res))
    except Exception:
        import traceback
        q.put((rank, "ERROR " + traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_decoder_matches_single_gpu(tmp_path, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = _free_port()
    cfg = SMALL if world <= 4 else WIDE
    model_path = None
    if world == 2:   # the slices cut from a model file are checked once
        model_path = str(tmp_path / "small.gguf")
        _write_model_file(model_path)
    procs = [mpc.Process(target=_worker, args=(r, world, port, q, model_path, cfg)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=900) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for r in range(world):
        assert not isinstance(res[r], str), res[r]
        assert res[r]["status"] == 0
        if model_path:
            assert res[r]["file_equals_sliced"]
    a, ref = res[0], res[0]["ref"]
    # every rank holds the same token, margin and (gathered) logits, bit for bit
    for r in range(1, world):
        b = res[r]
        assert a["tokens"] == b["tokens"] and a["run"] == b["run"] and a["margin"] == b["margin"]
        for la, lb in zip(a["logits"], b["logits"]):
            assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        (oa, ma, la), (ob, mb, lb) = a["batch"], b["batch"]
        assert oa == ob and ma == mb and np.array_equal(la.view(np.uint32), lb.view(np.uint32))
        assert a["batch2"] == b["batch2"]
    assert a["run"] == a["tokens"]
    # the batch pass equals the single-GPU pass up to the summation order
    (oa, ma, la), (o1, m1, l1) = a["batch"], ref["batch"]
    err = float(np.max(np.abs(la - l1)) / np.sqrt(np.mean(l1.astype(np.float64) ** 2)))
    assert err < 3e-3, err
    for i in range(len(BATCH_TOKS)):
        if oa[i] != o1[i]:
            assert m1[i] <= 4 * float(np.max(np.abs(la - l1))), (i, oa[i], o1[i], m1[i])
    for i in range(2):   # the same two positions through the other path: same token unless the margin is tiny
        if a["batch2"][0][i] != oa[i]:
            assert ma[i] <= 1e-3, (i, a["batch2"][0][i], oa[i], ma[i])
    # against one GPU: only the summation order of O and down changes
    for s in range(STEPS):
        want, got = ref["logits"][s], a["logits"][s]
        err = float(np.max(np.abs(got - want)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        assert err < 3e-3, (world, s, err)
        if a["tokens"][s] != ref["tokens"][s]:
            assert ref["margin"][s] <= 2 * float(np.max(np.abs(got - want))), (s, a["tokens"][s], ref["tokens"][s])
            break   # the sequences differ from here on


# ---- sequence-parallel long-context attention (2 GPUs) ------------------------------------------

def _seq_worker(rank, world, port, q_out):
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from fast_llm_b200 import capi, tp
        ctx = capi.Context(rank)
        scale = float(1.0 / np.sqrt(128.0))
        res = {}
        sp = tp.SeqParallel(ctx, dist, max_records=32 * 4)
        for kv, batch in ((32768, 1), (4096 + 333, 4)):
            g = torch.Generator(device="cuda").manual_seed(kv + batch)      # same stream on both ranks
            q = torch.randn((batch, 32, 128), generator=g, device="cuda")
            k = (torch.randn((batch, 8, kv, 128), generator=g, device="cuda") * scale).half()
            v = (torch.randn((batch, 8, kv, 128), generator=g, device="cuda") * scale).half()
            # this rank's contiguous slice of the keys (uneven when kv is odd)
            lo, hi = kv * rank // world, kv * (rank + 1) // world
            ks = k[:, :, lo:hi].contiguous().view(torch.int16)
            vs = v[:, :, lo:hi].contiguous().view(torch.int16)
            out_l = torch.zeros_like(q); lse = torch.zeros((batch, 32, 2), device="cuda"); out = torch.zeros_like(q)
            torch.cuda.synchronize()
            dist.barrier()
            ctx.attn_decode_lse(q, ks, vs, 32, 8, 128, hi - lo, hi - lo, batch, scale, out_l, lse)
            sp.combine(out_l, lse, batch * 32, out)
            ctx.sync()
            full = torch.zeros_like(q)
            ctx.attn_decode(q, k.view(torch.int16), v.view(torch.int16), 32, 8, 128, kv, kv, batch, scale, full)
            ctx.sync()
            res[(kv, batch)] = (out.cpu().numpy(), float((out - full).abs().max()))
        res["status"] = ctx.status()
        dist.barrier()
        sp.close()
        ctx.close()
        dist.destroy_process_group()
        q_out.put((rank, res))
    except Exception:
        import traceback
        q_out.put((rank, "ERROR " + traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sequence_parallel_attention(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = _free_port()
    procs = [mpc.Process(target=_seq_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for r in range(world):
        assert not isinstance(res[r], str), res[r]
        assert res[r]["status"] == 0
    for key in ((32768, 1), (4096 + 333, 4)):
        a, err_a = res[0][key]
        assert err_a <= 1e-5, (key, err_a)                               # = one GPU over all keys (f32 reassociation)
        for r in range(1, world):
            b, err_b = res[r][key]
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # all ranks: identical bits
            assert err_b <= 1e-5, (key, r, err_b)


def _moe_worker(rank, world, port, q_out):
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from fast_llm_b200 import capi, synth
        from fast_llm_b200.moe import MoeBlock, local_experts
        ctx = capi.Context(rank)
        E, F, NE, K, T = 4096, 1024, 8, 2, 16
        rng = np.random.default_rng(41)                     # the same model on every rank
        wg = synth.q4k_tensor(rng, NE * F, E); wu = synth.q4k_tensor(rng, NE * F, E); wd = synth.q4k_tensor(rng, NE * E, F)
        wr = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
        x = rng.standard_normal((T, E)).astype(np.float32)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        first, n = local_experts(NE, rank, world)
        blk = MoeBlock(ctx, E, F, NE, K, max_tokens=T, ep=(rank, world))
        blk.set_weights(dev(wr), dev(wg[first * F:(first + n) * F]), dev(wu[first * F:(first + n) * F]),
                        dev(wd[first * E:(first + n) * E]))
        blk.connect(dist)
        xd = dev(x)
        res = {"y": []}
        for n_tok in (T, 3, T):                             # the exchange buffers alternate between calls
            y = torch.zeros((n_tok, E), device="cuda")
            torch.cuda.synchronize()
            dist.barrier()
            blk.forward(xd, n_tok, y)
            ctx.sync()
            res["y"].append(y.cpu().numpy())
        for _ in range(3):                                   # recorded as a CUDA graph, then replayed
            torch.cuda.synchronize()
            dist.barrier()
            blk.forward(xd, T, y)
            ctx.sync()
            res["y"].append(y.cpu().numpy())
        res["ids"] = blk.routing(T)[0]
        res["status"] = ctx.status()
        dist.barrier()
        if rank == 0:                                       # all experts on one GPU
            one = MoeBlock(ctx, E, F, NE, K, max_tokens=T)
            one.set_weights(dev(wr), dev(wg), dev(wu), dev(wd))
            y = torch.zeros((T, E), device="cuda")
            torch.cuda.synchronize()
            one.forward(xd, T, y)
            ctx.sync()
            res["ref"] = y.cpu().numpy()
            res["ref_ids"] = one.routing(T)[0]
            one.close()
        dist.barrier()
        blk.close()
        ctx.close()
        dist.destroy_process_group()
        q_out.put((rank, res))
    except Exception:
        import traceback
        q_out.put((rank, "ERROR " + traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_moe_matches_single_gpu(world):
    """Expert parallelism of the MoE block (8 / world of the 8 experts per GPU): the ranks'
    outputs are identical bits and equal the single-GPU block up to the order of one sum."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    port = _free_port()
    procs = [mpc.Process(target=_moe_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for r in range(world):
        assert not isinstance(res[r], str), res[r]
        assert res[r]["status"] == 0
    a = res[0]
    assert np.array_equal(a["ids"], a["ref_ids"])
    assert len(set(a["ids"].ravel() // (8 // world))) >= 2   # more than one rank's experts are in use
    for r in range(1, world):
        b = res[r]
        assert np.array_equal(a["ids"], b["ids"])
        for ya, yb in zip(a["y"], b["y"]):
            assert np.array_equal(ya.view(np.uint32), yb.view(np.uint32))
    ref = a["ref"]
    scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.max(np.abs(a["y"][0] - ref)) <= 1e-5 * scale
    assert np.array_equal(a["y"][0].view(np.uint32), a["y"][2].view(np.uint32))
    assert np.array_equal(a["y"][1].view(np.uint32), a["y"][0][:3].view(np.uint32))
    for later in a["y"][3:]:
        assert np.array_equal(later.view(np.uint32), a["y"][0].view(np.uint32))
