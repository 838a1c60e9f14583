"""CPU tests of the tensor-parallel partition (host logic only): two gloo ranks
split the tensors of a small Llama-shape layer with fast_llm_b200.tp, run the
CPU oracle on their shares, and the exchanged results must equal the oracle on
the whole tensors. Also the cross-rank argmax merge rule."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

CFG = dict(n_layer=1, n_embd=2048, n_head=8, n_kv_head=2, head_dim=128, n_ff=1024, n_vocab=96, max_kv=16,
           rope_base=500000.0, eps=1e-5)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from fast_llm_b200 import capi, synth, tp
        from oracle import pyoracle
        orc = pyoracle.Oracle("port")
        cfg, seed = CFG, 9
        rng = np.random.default_rng(4)
        x = rng.standard_normal(cfg["n_embd"]).astype(np.float32)
        out = {}
        # row-split tensors: the ranks' outputs concatenate to the whole output, bit for bit
        for name in ("wq", "wk", "wv", "gate", "up", "output"):
            fmt = synth.Q4_K_M[name]
            w = synth.llama_tensor(cfg, seed, name, None if name == "output" else 0)
            rows = w.shape[0]
            axis, start, count = tp.slice_of(name, cfg, rank, world)
            assert axis == 0 and count * world == rows
            mine = orc.matvec(fmt, np.ascontiguousarray(tp.shard_tensor(name, w, fmt, cfg, rank, world)), count,
                              cfg["n_embd"], x)
            parts = [torch.zeros(count) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(mine))
            whole = orc.matvec(fmt, w, rows, cfg["n_embd"], x)
            out[name] = bool(np.array_equal(torch.cat(parts).numpy().view(np.uint32), whole.view(np.uint32)))
        # column-split tensors: partial products sum to the whole product (f32 reassociation only)
        for name, cols in (("wo", cfg["n_head"] * cfg["head_dim"]), ("down", cfg["n_ff"])):
            fmt = synth.Q4_K_M[name]
            w = synth.llama_tensor(cfg, seed, name, 0)
            xin = rng.standard_normal(cols).astype(np.float32)   # same stream on both ranks
            axis, start, count = tp.slice_of(name, cfg, rank, world)
            assert axis == 1 and count * world == cols
            ws = tp.shard_tensor(name, w, fmt, cfg, rank, world)
            assert ws.shape[1] == tp.pitch_of(fmt, count) and ws.shape[1] % 16 == 0
            rb = capi.row_bytes(fmt, count)
            assert not ws[:, rb:].any()                          # the padding is zero
            part = orc.matvec(fmt, np.ascontiguousarray(ws[:, :rb]), w.shape[0], count, xin[start:start + count])
            t = torch.from_numpy(part.astype(np.float64))
            dist.all_reduce(t)
            whole = orc.matvec(fmt, w, w.shape[0], cols, xin).astype(np.float64)
            scale = np.sqrt(np.mean(whole ** 2))
            out[name] = float(np.max(np.abs(t.numpy() - whole)) / scale)
        # KV heads and query heads of a rank line up (GQA groups are not cut)
        _, q0, qn = tp.slice_of("wq", cfg, rank, world)
        _, k0, kn = tp.slice_of("wk", cfg, rank, world)
        out["heads"] = (q0 // 128 // 4 == k0 // 128) and (qn == 4 * kn)
        dist.destroy_process_group()
        q.put((rank, out))
    except Exception as e:   # surface the failure in the parent
        import traceback
        q.put((rank, "ERROR " + traceback.format_exc()))


def test_partition_matches_whole_tensors_gloo_world2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for rank in (0, 1):
        out = res[rank]
        assert not isinstance(out, str), out
        for name in ("wq", "wk", "wv", "gate", "up", "output"):
            assert out[name] is True, (rank, name)
        assert out["wo"] < 1e-5 and out["down"] < 1e-5, out
        assert out["heads"]


def test_local_dims_and_rejections():
    from fast_llm_b200 import synth, tp
    cfg = synth.LLAMA3_8B
    for world in (1, 2, 4, 8):
        loc = tp.local_dims(cfg, world)
        assert loc["n_head"] == 4 * loc["n_kv_head"]
        assert loc["n_ff"] % 256 == 0 and loc["n_vocab"] * world == cfg["n_vocab"]
        assert tp.pitch_of(4, loc["n_ff"]) % 16 == 0
    with pytest.raises(ValueError):
        tp.local_dims(cfg, 3)
    with pytest.raises(ValueError):
        tp.slice_cols(np.zeros((2, 144 * 4), dtype=np.uint8), 3, 100, 256)


def test_merge_top_tie_rule():
    from fast_llm_b200 import tp
    rng = np.random.default_rng(1)
    for trial in range(50):
        world = int(rng.integers(1, 9))
        n = 16
        lg = rng.integers(-3, 4, world * n).astype(np.float32)   # many ties
        recs = []
        for r in range(world):
            sl = lg[r * n:(r + 1) * n]
            i = int(np.argmax(sl))                                # first maximum
            rest = np.delete(sl, i)
            recs.append((float(sl[i]), r * n + i, float(rest.max())))
        idx, margin = tp.merge_top(recs)
        assert idx == int(np.argmax(lg))
        assert margin == float(lg[idx] - np.delete(lg, idx).max())


def test_merge_lse_equals_softmax_over_all_keys():
    from fast_llm_b200 import tp
    rng = np.random.default_rng(3)
    for world in (1, 2, 3, 8):
        n = 97 * world + 5
        s = rng.standard_normal(n) * 4.0
        v = rng.standard_normal((n, 128))
        p = np.exp(s - s.max()); p /= p.sum()
        want = p @ v
        bounds = [n * r // world for r in range(world + 1)]
        recs = []
        for r in range(world):
            sl = slice(bounds[r], bounds[r + 1])
            m = s[sl].max(); e = np.exp(s[sl] - m)
            recs.append((e @ v[sl] / e.sum(), m, e.sum()))
        assert np.allclose(tp.merge_lse(recs), want, rtol=1e-12, atol=1e-12)


def test_expert_partition():
    from fast_llm_b200.moe import local_experts
    assert [local_experts(8, r, 4) for r in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert local_experts(8, 0, 1) == (0, 8) and local_experts(8, 7, 8) == (7, 1)
    with pytest.raises(ValueError):
        local_experts(8, 0, 3)
