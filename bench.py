"""Benchmark of the decode hot path: greedy decode tokens/s of the synthetic
Llama-3-8B-shape Q4_K_M model (32 layers, hidden 4096, 32/8 heads of 128, FFN
14336, vocab 128256) with an 8192-token prefilled f16 KV cache, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decoded token: every packed weight and every cached K/V row is
read once. Prints ONE JSON line (rank 0).

  value      tokens/s with the token fed back on the device (CUDA-graph replays,
             inputs resident in HBM), device-timed with CUDA events
  e2e        tokens/s through the public per-token call: token host->device,
             graph, next token device->host, every step
  roofline   the streaming matvec kernel (dominant): packed weight bytes of one
             step / time of that step's matvec launches replayed alone
  cpu_baseline  the reference's CPU operators on this box's host cores, on a
             bounded sample (2 of the 32 layers + the output head), N=1 only

With --gpus N > 1 (torchrun, one rank per GPU) the headline value is the
tensor-parallel decode of ONE sequence over the N GPUs (KV heads and matvec
rows / columns per GPU, the partial sums exchanged through peer memory):
"strong" scaling, total work fixed; the roofline object then gives the
per-GPU fraction. The same run also times N independent replicas (one sequence
per GPU, no data-path collective) and reports them under the key "replicas".
--impl reference times only the CPU arm (rank 0), same metric and config.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_PREFILL = 8192
METRIC = "decode tokens/s at 8B Q4_K_M shape, 1/2/4/8 B200; HBM GB/s % of roofline"


NCU_TRAFFIC_RATIO = 1.0057
TIMED_REGION_MS = 1000.0   # device time the repeated K-step loops add up to, at least


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        import tempfile
        self.path = os.path.join(tempfile.gettempdir(), "fl_b200_bench_clocks_%d_rank%d.csv" % (os.getpid(), device))

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark(self):
        """Start of the region whose samples count (nvidia-smi itself is started earlier: it takes a while
        to come up, longer with one instance per rank)."""
        self.t0 = time.time()

    def stop(self):
        t1 = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        t0 = getattr(self, "t0", 0.0)
        inside = [r for r in rows if t0 - 0.05 <= r[0] <= t1 + 0.05]
        window = "timed region"
        if not inside:   # a region shorter than the sampling period: the nearest samples on either side of it
            inside = sorted(rows, key=lambda r: min(abs(r[0] - t0), abs(r[0] - t1)))[:2]
            window = "nearest to the timed region"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(r[1] for r in inside)
        reasons = sorted({n for r in inside for n in r[3]})
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(r[2] for r in inside), "reasons": reasons,
                "samples": len(inside), "window": window}


def cpu_reference_arm(steps, warmup, threads=None):
    """Times the reference's CPU operators (oracle/_ref when it travelled, else
    the pinned port) on a bounded sample of the workload: one decode step of a
    2-layer slice of the model plus the output head, at position 8192, on all
    host cores. tokens/s = 1 / (t_head + 16 * (t_2layers+head - t_head))."""
    import numpy as np
    from fast_llm_b200 import synth
    from oracle import pyoracle
    kind = "reference" if pyoracle.Oracle.available("reference") else "port"
    orc = pyoracle.Oracle(kind)
    cores = threads or os.cpu_count() or 1
    # torchrun exports OMP_NUM_THREADS=1 to its ranks and the OpenMP runtime has read it by now: set the count directly
    os.environ["OMP_NUM_THREADS"] = str(cores)
    orc.port.flo_set_threads(cores)
    full = dict(synth.LLAMA3_8B)

    def build(n_layer):
        cfg = dict(full, n_layer=n_layer)
        m = pyoracle.LlamaOracle(orc, cfg)
        for l in range(n_layer):
            for i, name in enumerate(synth.LAYER_TENSORS):
                m.set_layer_tensor(l, i, synth.Q4_K_M[name], synth.llama_tensor(cfg, 0, name, l))
            m.set_layer_norms(l, synth.llama_norm(cfg, 0, "attn_norm", l), synth.llama_norm(cfg, 0, "ffn_norm", l))
            k, v = synth.llama_kv(cfg, 0, l, N_PREFILL)
            m.seed_kv(l, k, v)
        return m

    head_w = synth.llama_tensor(full, 0, "output")
    on = synth.llama_norm(full, 0, "out_norm")
    models = []
    for n_layer in (0, 2):
        m = build(n_layer)
        m.set_global(0, synth.Q4_K_M["tok_embd"], head_w)   # same bytes serve as embedding table
        m.set_global(1, synth.Q4_K_M["output"], head_w)
        m.set_out_norm(on)
        models.append(m)

    def one(m):
        m.set_n_past(N_PREFILL)
        t0 = time.perf_counter()
        m.step(1)
        return time.perf_counter() - t0

    times = []
    for it in range(warmup + steps):
        t_head, t_two = one(models[0]), one(models[1])
        if it >= warmup:
            times.append(t_head + 16.0 * max(t_two - t_head, 0.0))
    for m in models:
        m.close()
    t_tok = sum(times) / len(times)
    return {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": "one decode step of 2 of the 32 layers + output head at position 8192, scaled to 32 layers; "
                      "reference STREAM_DOT tiles of 192 rows and one attention head per task on %d threads" % cores,
            "ms_per_token": t_tok * 1e3}


def cpu_pool_fast_arms(cores):
    """The other CPU arms, as extra keys of cpu_baseline: the reference's run_serial on one core and its own worker
    pool (Runtime, gpu_enabled = false) with fast_kernels off (canonical) and on (include/fastllm/fastllm.h:198),
    timed on the STREAM_DOT tiles of one layer's seven tensors and of the output head; tokens/s = 1 / (32 t_layer +
    t_head). Attention, norms and the other operators are left out, so the figures are upper bounds of what these
    decode. The fast pool once more at -O3 -march=x86-64-v3 (its AVX2 kernels), when the host has AVX2."""
    import numpy as np
    from fast_llm_b200 import synth
    from oracle import pyoracle
    if not pyoracle.Oracle.available("reference"):
        return {}
    cfg = dict(synth.LLAMA3_8B)
    shapes = synth.layer_shapes(cfg)
    tensors = [(synth.Q4_K_M[n], synth.llama_tensor(cfg, 0, n, 0), shapes[n]) for n in synth.LAYER_TENSORS]
    head = (synth.Q4_K_M["output"], synth.llama_tensor(cfg, 0, "output"), (cfg["n_vocab"], cfg["n_embd"]))
    rng = np.random.default_rng(7)
    out = {}
    # (key, library, build flags, threads (0 = run_serial on one core), fast_kernels, repetitions)
    ref_flags = "-O2 -ffp-contract=off (the reference's flags)"
    libs = [("run_serial_1_core", None, ref_flags, 0, False, 1),
            ("pool_canonical", None, ref_flags, cores, False, 3),
            ("pool_fast_kernels", None, ref_flags, cores, True, 3)]
    if os.path.exists(pyoracle.REF_O3_LIB) and pyoracle.host_has_avx2_fma():
        libs.append(("pool_fast_kernels_o3_avx2", pyoracle.REF_O3_LIB, "-O3 -march=x86-64-v3 (AVX2 + FMA kernels)", cores, True, 3))
    for key, lib, flags, threads, fast, reps in libs:
        orc = pyoracle.Oracle("reference", ref_lib=lib)

        def t_of(fmt, w, shape):
            x = rng.standard_normal(shape[1]).astype(np.float32)
            best = None
            for _ in range(reps):
                _, ns = orc.ref_stream_dot_tasks(fmt, w, shape[0], shape[1], x, threads, fast=fast)
                best = ns if best is None else min(best, ns)
            return best * 1e-9

        t_layer = sum(t_of(*t) for t in tensors)
        t_head = t_of(*head)
        orc.ref_pool_shutdown()
        t_tok = 32.0 * t_layer + t_head
        out[key] = {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": threads if threads > 0 else 1, "kind": "reference", "build": flags,
                    "sample": "STREAM_DOT tiles (192 rows) of one layer's seven tensors and of the output head through the "
                              "reference's %s, best of %d each, scaled to 32 layers; attention and the small operators left out "
                              "(an upper bound)" % ("run_serial" if threads <= 0 else "Runtime pool with fast_kernels %s" % ("on" if fast else "off"), reps),
                    "ms_per_token": t_tok * 1e3}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="both", choices=["both", "tp", "replicas"],
                    help="N > 1: tp = one sequence, the step split over the GPUs (KV heads, matvec rows / columns, exchange "
                         "through peer memory; strong scaling; the headline value); replicas = one independent sequence "
                         "per GPU (weak scaling); both = tp as the headline and the replica measurement of the same run "
                         "under the key \"replicas\"")
    ap.add_argument("--region-ms", type=float, default=TIMED_REGION_MS,
                    help="device time the repeated K-step loops add up to, at least (0 = one repetition: profiler captures)")
    ap.add_argument("--layers", type=int, default=32,
                    help="number of layers (32 = the benchmark; fewer = a small case of the same kernels for profiler captures, not a benchmark number)")
    ap.add_argument("--case", default="decode", choices=["decode", "matmul-nx8", "attn-long", "moe", "moe-decode"],
                    help="decode = the benchmark (default). matmul-nx8 = the multi-column Q4_K matmul alone (gate|up shape, 8 "
                         "columns); attn-long = decode attention alone at 32K / 64K / 128K keys; moe = the MoE feed-forward "
                         "block at the Mixtral shape (8 experts, top-2, 16 tokens; expert parallel under torchrun); moe-decode = greedy "
                         "decode of a whole synthetic Mixtral-8x7B-shape model (32 layers, 8 experts, top-2) on one GPU: kernel "
                         "cases for profiler captures and sweeps, each prints its own JSON line and is not the benchmark number")
    args = ap.parse_args()
    if args.case != "decode":
        return kernel_case(args.case, max(1, args.steps), max(3, args.warmup))
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    config = {"workload": "synthetic Llama-3-8B-shape Q4_K_M greedy decode, batch 1, 8192-token prefilled f16 KV",
              "n_layer": args.layers, "hidden": 4096, "heads": "32/8 x 128", "ffn": 14336, "vocab": 128256,
              "kv_prefill": N_PREFILL,
              "parallelism": "single GPU" if world == 1 else
                             ("tp%d (KV heads + matvec rows/columns per GPU, 2 all-reduces per layer through peer memory)" % world
                              if args.parallelism != "replicas" else "replicas x%d (independent sequences, no data-path collective)" % world),
              "l2": "each step reads 6.0 GB of distinct weights and KV, far larger than L2; no flush needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        cpu_steps = min(steps, 3)
        r = cpu_reference_arm(cpu_steps, 1)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": cpu_steps, "warmup": 1, "ms_per_step": r["ms_per_token"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": dict({k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}, also=cpu_pool_fast_arms(r["cores"])),
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch
    from fast_llm_b200 import capi, synth
    from fast_llm_b200.decoder import Decoder
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = capi.Context(local_rank)
    cfg = dict(synth.LLAMA3_8B, n_layer=args.layers)
    if args.layers != 32:
        config["workload"] += " (REDUCED to %d layers: profiler case, not the benchmark)" % args.layers
    if steps + warmup + 8 > cfg["max_kv"] - N_PREFILL:
        cfg["max_kv"] = N_PREFILL + steps + warmup + 8
    gloo = dist.new_group(backend="gloo") if world > 1 else None   # IPC handles travel as Python objects
    modes = ["replicas"] if world == 1 else {"both": ["tp", "replicas"], "tp": ["tp"], "replicas": ["replicas"]}[args.parallelism]
    out = None
    for mode in modes:
        r = measure(mode == "tp", args, ctx, cfg, config, dist, gloo, rank, local_rank, world, steps, warmup)
        if out is None:
            out = r
        else:   # the replica measurement of the same run, beside the headline
            out["replicas"] = {"value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"], "scaling": "weak",
                               "parallelism": "replicas x%d: one independent sequence per GPU, no data-path collective" % world,
                               "e2e": r["e2e"], "roofline": r["roofline"], "gpu_launches": r["gpu_launches"]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_arm(1, 1)
        out["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        out["cpu_baseline"]["also"] = cpu_pool_fast_arms(r["cores"])
    ctx.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out))


def kernel_case(case, steps, warmup):
    """One kernel alone on cuda:0, through the C ABI, timed with device events; inputs rotate over
    more than L2 (126 MB) of distinct weights or keys."""
    import torch
    from fast_llm_b200 import capi, synth
    peak, _ = measured_peaks()
    if case == "moe":
        return moe_case(steps, warmup, peak)
    if case == "moe-decode":
        return moe_decode_case(steps, warmup, peak)
    if case == "attn-long" and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return attn_long_multi(steps, warmup, peak, int(os.environ.get("RANK", "0")), int(os.environ["WORLD_SIZE"]))
    ctx = capi.Context(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    if case == "matmul-nx8":
        rows, cols, nx, copies = 28672, 4096, 8, 3
        w = [synth.device_quant_tensor(capi.Q4_K, rows, cols, gen) for _ in range(copies)]
        x = torch.randn((nx, cols), device="cuda", generator=gen)
        y = torch.zeros((nx, rows), device="cuda")
        torch.cuda.synchronize()

        def run(n):
            for i in range(n):
                ctx.matvec(capi.Q4_K, w[i % copies], rows, cols, x, y, nx=nx, xstride=cols, ystride=rows)
        run(warmup)
        ctx.sync()
        ctx.timer_start()
        run(steps)
        us = ctx.timer_stop() * 1e3 / steps
        nbytes = rows * capi.row_bytes(capi.Q4_K, cols)
        print(json.dumps({"case": case, "kernel": "matmul_umma_kernel (tcgen05, FLB_UMMA=1)" if os.environ.get("FLB_UMMA", "")[:1] == "1" else "matmul_tc_nx_kernel",
                          "rows": rows, "cols": cols, "columns": nx,
                          "us_per_pass": us, "weight_bytes": nbytes, "achieved_gbs": nbytes / us / 1e3,
                          "frac_of_measured_hbm": nbytes / us / 1e3 / peak, "status": ctx.status()}))
        return
    # attn-long: the long-context configuration (f16 K/V ~ N(0, 1)/sqrt(128), 32 query / 8 KV heads of 128)
    out = []
    for kv_len, batch in ((32768, 1), (32768, 4), (65536, 1), (65536, 4), (131072, 1), (131072, 4), (32768, 16), (131072, 16)):
        nkv, nq, d = 8, 32, 128
        copies = max(1, int(300e6 // (2 * batch * nkv * kv_len * d * 2)) + 1)   # distinct caches worth more than L2
        k = [(torch.randn((batch, nkv, kv_len, d), device="cuda", generator=gen) / 128 ** 0.5).half() for _ in range(copies)]
        v = [(torch.randn((batch, nkv, kv_len, d), device="cuda", generator=gen) / 128 ** 0.5).half() for _ in range(copies)]
        q = torch.randn((batch, nq, d), device="cuda", generator=gen)
        o = torch.zeros((batch, nq, d), device="cuda")
        torch.cuda.synchronize()

        def run(n):
            for i in range(n):
                ctx.attn_decode(q, k[i % copies], v[i % copies], nq, nkv, d, kv_len, kv_len, batch, 1.0 / 128 ** 0.5, o)
        run(warmup)
        ctx.sync()
        ctx.timer_start()
        run(steps)
        us = ctx.timer_stop() * 1e3 / steps
        nbytes = 2 * batch * nkv * kv_len * d * 2
        out.append({"kv_len": kv_len, "batch": batch, "us": us, "kv_bytes": nbytes, "achieved_gbs": nbytes / us / 1e3,
                    "frac_of_measured_hbm": nbytes / us / 1e3 / peak})
        del k, v
        torch.cuda.empty_cache()
    print(json.dumps({"case": case, "kernel": "attn_decode_kernel", "peak_gbs": peak, "points": out, "status": ctx.status()}))


def attn_long_multi(steps, warmup, peak, rank, world):
    """The long-context configuration over the GPUs of one box (torchrun, one rank per GPU), both partitions:
    "heads": rank r owns 8 / world KV heads with their query heads over ALL keys: no exchange at all;
    "seq":   every rank owns all heads over a contiguous 1 / world of the keys and the ranks' (context, max, sum)
             records are merged through peer memory (fl_b200_seqpar_combine).
    Per point: time of the slowest rank (device events), this rank-set's per-GPU rate, and for "seq" the merge alone."""
    import torch
    import torch.distributed as dist
    from fast_llm_b200 import capi, tp
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = capi.Context(local_rank)
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5 + rank)
    nkv, nq, d = 8, 32, 128
    scale = 1.0 / 128 ** 0.5
    sp = tp.SeqParallel(ctx, dist, max_records=nq * 16)
    points = []

    def timed(fn):
        for _ in range(warmup):
            fn()
        ctx.sync()
        dist.barrier()
        ctx.timer_start()
        for _ in range(steps):
            fn()
        ms = ctx.timer_stop() / steps
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3   # us, slowest rank

    for kv_len, batch in ((32768, 1), (32768, 4), (32768, 16), (65536, 1), (65536, 4), (65536, 16), (131072, 1), (131072, 4), (131072, 16)):
        total = 2 * batch * nkv * kv_len * d * 2
        pt = {"kv_len": kv_len, "batch": batch, "kv_bytes_total": total}
        # ---- KV heads over the ranks (up to 8 ranks): nothing to exchange ----
        if nkv % world == 0:
            hk = nkv // world
            k = (torch.randn((batch, hk, kv_len, d), device=dev, generator=gen) * scale).half()
            v = (torch.randn((batch, hk, kv_len, d), device=dev, generator=gen) * scale).half()
            q = torch.randn((batch, 4 * hk, d), device=dev, generator=gen)
            o = torch.zeros((batch, 4 * hk, d), device=dev)
            torch.cuda.synchronize(dev)
            us = timed(lambda: ctx.attn_decode(q, k, v, 4 * hk, hk, d, kv_len, kv_len, batch, scale, o))
            pt["heads"] = {"us": us, "per_gpu_gbs": total / world / us / 1e3, "per_gpu_frac_of_measured_hbm": total / world / us / 1e3 / peak,
                           "exchange": "none"}
            del k, v
        # ---- the keys over the ranks: every rank all heads, 1 / world of the positions, then the merge ----
        lo, hi = kv_len * rank // world, kv_len * (rank + 1) // world
        k = (torch.randn((batch, nkv, hi - lo, d), device=dev, generator=gen) * scale).half()
        v = (torch.randn((batch, nkv, hi - lo, d), device=dev, generator=gen) * scale).half()
        q = torch.randn((batch, nq, d), device=dev, generator=gen)
        ol = torch.zeros((batch, nq, d), device=dev)
        lse = torch.zeros((batch, nq, 2), device=dev)
        o = torch.zeros((batch, nq, d), device=dev)
        torch.cuda.synchronize(dev)

        def both():
            ctx.attn_decode_lse(q, k, v, nq, nkv, d, hi - lo, hi - lo, batch, scale, ol, lse)
            sp.combine(ol, lse, batch * nq, o)
        us = timed(both)
        us_attn = timed(lambda: ctx.attn_decode_lse(q, k, v, nq, nkv, d, hi - lo, hi - lo, batch, scale, ol, lse))
        pt["seq"] = {"us": us, "us_attention_alone": us_attn, "us_merge": us - us_attn, "per_gpu_gbs": total / world / us / 1e3,
                     "per_gpu_frac_of_measured_hbm": total / world / us / 1e3 / peak,
                     "exchange": "%d records of 130 floats to every rank" % (batch * nq)}
        points.append(pt)
        del k, v
        torch.cuda.empty_cache()
    status = ctx.status()
    dist.barrier()
    sp.close()
    if rank == 0:
        print(json.dumps({"case": "attn-long", "n_gpus": world, "kernel": "attn_decode_kernel + lse_combine_kernel", "peak_gbs": peak,
                          "points": points, "status": status}))
    ctx.close()
    dist.destroy_process_group()


def moe_case(steps, warmup, peak):
    """The MoE configuration's feed-forward block: 8 experts of gate / up 14336 x 4096 and down 4096 x 14336
    (Q4_K), f32 router ~ N(0, 0.02), 16 tokens, top-2 with renormalised weights. One process per GPU under
    torchrun: expert parallel (8 / N experts per rank), time = max over ranks."""
    import torch
    from fast_llm_b200 import capi, synth
    from fast_llm_b200.moe import MoeBlock, local_experts
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = capi.Context(local_rank)
    E, F, NE, K, T = 4096, 14336, 8, 2, 16
    first, n = local_experts(NE, rank, world)
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator(device=dev); gen.manual_seed(3 + rank)
    rep = torch.Generator(device=dev); rep.manual_seed(99)     # what every rank holds whole
    wg = synth.device_quant_tensor(capi.Q4_K, n * F, E, gen)
    wu = synth.device_quant_tensor(capi.Q4_K, n * F, E, gen)
    wd = synth.device_quant_tensor(capi.Q4_K, n * E, F, gen)
    wr = torch.randn((NE, E), device=dev, generator=rep) * 0.02
    x = torch.randn((T, E), device=dev, generator=rep)
    y = torch.zeros((T, E), device=dev)
    blk = MoeBlock(ctx, E, F, NE, K, max_tokens=T, ep=(rank, world) if world > 1 else None)
    blk.set_weights(wr, wg, wu, wd)
    if world > 1:
        blk.connect(dist)
    torch.cuda.synchronize(dev)
    for _ in range(max(warmup, 3)):   # the third call replays the recorded graph
        if dist:
            dist.barrier()
        blk.forward(x, T, y)
        ctx.sync()
    if dist:
        dist.barrier()
    ctx.timer_start()
    for _ in range(steps):
        blk.forward(x, T, y)
    ms = ctx.timer_stop() / steps
    ids = blk.routing(T)[0]
    mine = int(((ids >= first) & (ids < first + n)).sum())
    distinct = len({int(e) for e in ids.ravel() if first <= int(e) < first + n})   # experts of this rank that were walked
    if dist:
        t = torch.tensor([ms, float(mine), float(distinct)], dtype=torch.float64)
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        ms = max(float(p[0]) for p in parts)
        slots = [int(p[1]) for p in parts]
        experts = [int(p[2]) for p in parts]
    else:
        slots, experts = [mine], [distinct]
    status = ctx.status()
    if rank == 0:
        expert_bytes = 2 * F * capi.row_bytes(capi.Q4_K, E) + E * capi.row_bytes(capi.Q4_K, F)
        # algorithmic bytes: every DISTINCT expert a rank holds and somebody chose is read once per block
        print(json.dumps({"case": "moe", "n_gpus": world, "tokens": T, "experts": NE, "top_k": K, "ms_per_block": ms,
                          "tokens_per_s": T / (ms * 1e-3), "slots_per_rank": slots, "distinct_experts_per_rank": experts,
                          "bytes_per_expert": expert_bytes,
                          "busiest_rank_gbs": max(experts) * expert_bytes / ms / 1e6,
                          "busiest_rank_frac_of_measured_hbm": max(experts) * expert_bytes / ms / 1e6 / peak, "status": status}))
    if dist:
        dist.barrier()
    blk.close()
    if dist:
        dist.destroy_process_group()


def time_sequences(ctx, dec, cfg, n_seq, n_prefill, passes=8):
    """n_seq independent sequences in lock step (fl_b200_decoder_seqs_step): one token per sequence and pass, through the
    public call (tokens in, greedy tokens out), device events around the calls. Returns ms per pass."""
    from fast_llm_b200 import synth
    synth.device_seqs(dec, cfg, n_seq, n_prefill)
    toks = list(range(1, n_seq + 1))
    for _ in range(2):
        toks, _ = dec.seqs_step(toks)
    ctx.sync()
    ctx.timer_start()
    for _ in range(passes):
        toks, _ = dec.seqs_step(toks)
    ms = ctx.timer_stop() / passes
    for s in range(n_seq):
        dec.seqs_set_pos(s, n_prefill)
    return ms


def moe_decode_case(steps, warmup, peak):
    """Greedy decode of a synthetic Mixtral-8x7B-shape model on one GPU: 32 layers of the 8B shape's attention (hidden
    4096, 32 / 8 heads) with the feed-forward block of every layer replaced by 8 experts (gate / up 14336 x 4096, down
    4096 x 14336, Q4_K), top-2 routing with renormalised weights, f32 router ~ N(0, 0.02); vocabulary 32000; 4096
    prefilled positions. Per token the step reads the attention tensors, the routers and 2 experts per layer."""
    import torch
    from fast_llm_b200 import capi, synth
    from fast_llm_b200.decoder import Decoder
    from fast_llm_b200.moe import MoeBlock
    ctx = capi.Context(0)
    n_prefill = 4096
    cfg = dict(synth.LLAMA3_8B, n_vocab=32000, max_kv=n_prefill + steps + warmup + 64)
    E, F, NE, K = cfg["n_embd"], cfg["n_ff"], 8, 2
    dec = Decoder(ctx, cfg)
    layers = range(cfg["n_layer"])
    synth.device_llama(dec, cfg, seed=77, n_prefill=n_prefill, skip_ffn=set(layers))
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(5)
    blocks = []
    for l in layers:
        blk = MoeBlock(ctx, E, F, NE, K, max_tokens=16)
        blk.set_weights(torch.randn((NE, E), device=dev, generator=gen) * 0.02,
                        synth.device_quant_tensor(capi.Q4_K, NE * F, E, gen), synth.device_quant_tensor(capi.Q4_K, NE * F, E, gen),
                        synth.device_quant_tensor(capi.Q4_K, NE * E, F, gen))
        dec.set_layer_moe(l, blk)
        blocks.append(blk)
    torch.cuda.synchronize(dev)
    dec.finalize()
    dec.rewind_to(n_prefill)
    last = int(dec.run(1, warmup)[-1])
    times = []
    for _ in range(5):
        dec.rewind_to(n_prefill + warmup)
        ctx.sync()
        ctx.timer_start()
        toks = dec.run(last, steps)
        times.append(ctx.timer_stop())
    ms = sorted(times)[len(times) // 2] / steps
    w_bytes, kv_bytes = dec.bytes_per_step(n_prefill + warmup + steps // 2)
    # 8 and 16 positions in one batch pass (draft verification / a prompt chunk): every expert is walked once for the
    # positions that chose it (multi-column kernel), the attention tensors once
    passes = {}
    for m in (8, 16):
        for _ in range(2):
            dec.rewind_to(n_prefill)
            dec.step_batch(list(range(1, m + 1)))
        ctx.sync()
        ctx.timer_start()
        for _ in range(5):
            dec.rewind_to(n_prefill)
            dec.step_batch(list(range(1, m + 1)))
        bp_ms = ctx.timer_stop() / 5
        passes["m%d" % m] = {"m": m, "ms_per_pass": bp_ms, "positions_per_s": m / (bp_ms * 1e-3), "single_steps_ms": m * ms}
    # 16 independent sequences in flight (the MoE configuration's 16 tokens), 4096 prefilled positions each
    sq_ms = time_sequences(ctx, dec, cfg, 16, n_prefill)
    print(json.dumps({"case": "moe-decode", "model": "synthetic Mixtral-8x7B shape, Q4_K experts, top-2 of 8, 4096-token prefilled f16 KV",
                      "tokens_per_s": 1e3 / ms, "ms_per_token": ms, "steps": steps, "repeats": len(times),
                      "launches_per_step": dec.launches_per_step(), "bytes_per_token": w_bytes + kv_bytes,
                      "achieved_gbs": (w_bytes + kv_bytes) / ms / 1e6, "frac_of_measured_hbm": (w_bytes + kv_bytes) / ms / 1e6 / peak,
                      "experts_read_per_token": 32 * K, "batch_pass": passes,
                      "sequences_16": {"n": 16, "kv_prefill": n_prefill, "ms_per_pass": sq_ms, "tokens_per_s": 16 / (sq_ms * 1e-3)},
                      "device_weight_gb": round((32 * NE * 3 * F * capi.row_bytes(capi.Q4_K, E)) / 1e9, 1),
                      "last_token": int(toks[-1]), "status": ctx.status()}))
    dec.close()
    for b in blocks:
        b.close()
    ctx.close()


def measure(tp_mode, args, ctx, cfg, config, dist, gloo, rank, local_rank, world, steps, warmup):
    """One decoder (this rank's replica, or its share of the tensor-parallel group), timed."""
    import torch
    from fast_llm_b200 import synth
    from fast_llm_b200.decoder import Decoder
    config = dict(config)
    if world > 1:
        config["parallelism"] = ("tp%d (one sequence; KV heads + matvec rows/columns per GPU, 2 all-reduces per layer through "
                                 "peer memory)" % world) if tp_mode else "replicas x%d (independent sequences, no data-path collective)" % world
    sampler = ClockSampler(local_rank)
    sampler.start()   # before the model is built: running by the time the timed region starts
    dec = Decoder(ctx, cfg, tp=(rank, world) if tp_mode else None)
    synth.device_llama(dec, cfg, seed=1234 if tp_mode else 1234 + rank, n_prefill=N_PREFILL)
    if tp_mode:
        from fast_llm_b200 import tp
        tp.connect(dec, dist, group=gloo)
    dec.finalize()
    seqs = 1 if tp_mode else world   # sequences decoded at once

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run_steps(first, n):
        """n greedy steps on the device, in calls of at most 4096 (the decoder's token history)."""
        out, t = [], first
        while n > 0:
            k = min(n, 4096)
            out += [int(x) for x in dec.run(t, k)]
            t, n = out[-1], n - k
        return out

    # The K-step loop is repeated until about a second of device time has been timed (each repetition starts
    # from the same position and times exactly K steps between barriers); the median repetition is reported.
    def repeated(prepare, loop):
        times = []
        while True:
            prepare()
            barrier()
            ctx.timer_start()
            res = loop()
            ms = ctx.timer_stop()
            barrier()
            times.append(max_over_ranks(ms))
            if len(times) >= 15 or (sum(times) >= args.region_ms and len(times) % 2 == 1):
                break
        return sorted(times)[len(times) // 2], times, res

    # ---- value: device-resident feedback loop ----
    dec.rewind_to(N_PREFILL)
    last = run_steps(1, warmup)[-1]
    sampler.mark()
    ms_dev, reps_dev, toks = repeated(lambda: dec.rewind_to(N_PREFILL + warmup), lambda: run_steps(last, steps))
    # ---- e2e: public per-token call with host token in / out ----
    dec.rewind_to(N_PREFILL)
    t = 1
    for _ in range(warmup):
        t = dec.step(t)

    def e2e_loop():
        tok = t
        for _ in range(steps):
            tok = dec.step(tok)
        return tok
    ms_e2e, reps_e2e, _ = repeated(lambda: dec.rewind_to(N_PREFILL + warmup), e2e_loop)
    clocks = sampler.stop()
    assert ctx.status() == 0, "a kernel reported a status"

    # ---- roofline of the dominant kernel: the step's matvec launches alone ----
    pos_mid = N_PREFILL + warmup + steps // 2
    w_bytes, kv_bytes = dec.bytes_per_step(pos_mid)
    dec.rewind_to(pos_mid)
    mv_ms, mv_n = dec.time_class(1, 20)
    at_ms, at_n = dec.time_class(2, 20)
    ot_ms, ot_n = dec.time_class(4, 20)
    if tp_mode:
        barrier()
        cm_ms, cm_n = dec.time_class(8, 20)   # the exchange steps alone (all ranks together)
        barrier()
    peak, peak_kind = measured_peaks()
    achieved = w_bytes / (mv_ms * 1e-3) / 1e9
    launches = dec.launches_per_step()
    out = {
        "metric": METRIC, "value": seqs * steps / (ms_dev * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_dev / steps, "higher_is_better": True,
        "repeats": {"n": len(reps_dev), "ms_per_repeat": [round(x, 3) for x in reps_dev], "reported": "median",
                    "e2e_n": len(reps_e2e), "e2e_ms_per_repeat": [round(x, 3) for x in reps_e2e]},
        "scaling": "strong" if tp_mode else "weak", "vs_baseline": None, "dtype": "s32 sums of u8 x s8 products (Q4_K / Q6_K quants x 30-bit fixed-point activation digits), f32 scales and row sums; f16 KV with f32 attention",
        "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "kernel": "matvec_tc_kernel", "achieved": achieved, "peak": peak,
                     "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peak_kind == "measured" else "fallback 6.65 TB/s",
                     "unit": "GB/s", "frac": achieved / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of the four matvec launch shapes in one ncu
                     # capture (profiles/matvec_tc_kernel_8b_layer_shapes.md) were 1.0079 x their algorithmic
                     # bytes; traffic grows in proportion to the weights streamed, so it is scaled to this launch mix
                     "traffic": NCU_TRAFFIC_RATIO * w_bytes / mv_n,
                     "bytes_per_launch": w_bytes / mv_n, "launches_per_step": mv_n, "avg_launch_us": mv_ms * 1e3 / mv_n,
                     "step": {"bytes": w_bytes + kv_bytes, "achieved": (w_bytes + kv_bytes) / (ms_dev / steps * 1e-3) / 1e9,
                              "frac": (w_bytes + kv_bytes) / (ms_dev / steps * 1e-3) / 1e9 / peak,
                              "frac_of_8TBs": (w_bytes + kv_bytes) / (ms_dev / steps * 1e-3) / 1e9 / 8000.0},
                     "attention": {"achieved": kv_bytes / (at_ms * 1e-3) / 1e9, "frac": kv_bytes / (at_ms * 1e-3) / 1e9 / peak,
                                   "launches_per_step": at_n, "avg_launch_us": at_ms * 1e3 / at_n},
                     "other_ms_per_step": ot_ms, "other_launches_per_step": ot_n},
        "e2e": {"value": seqs * steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 16,
                "d2h_bytes_per_step": 4},
        "gpu_launches": launches * steps, "clocks": clocks, "last_token": int(toks[-1]),
    }
    if not tp_mode and world == 1:
        # Decoder::step_batch (draft verification / prompt chunks): 8 tokens at consecutive positions in one pass,
        # timed with device events around the public call (tokens in, greedy tokens and margins out)
        m, reps = 8, 5
        dec.rewind_to(N_PREFILL)
        dec.step_batch(list(range(1, m + 1)))
        dec.rewind_to(N_PREFILL)
        dec.step_batch(list(range(1, m + 1)))
        ctx.timer_start()
        for _ in range(reps):
            dec.rewind_to(N_PREFILL)
            dec.step_batch(list(range(1, m + 1)))
        bp_ms = ctx.timer_stop() / reps
        # 16 independent sequences decoded in lock step (fl_b200_decoder_seqs_step), each with its own 8192-position cache
        sq_ms = time_sequences(ctx, dec, cfg, 16, N_PREFILL)
        out["sequences_16"] = {"n": 16, "kv_prefill": N_PREFILL, "ms_per_pass": sq_ms, "tokens_per_s": 16 / (sq_ms * 1e-3),
                               "note": "aggregate over 16 sequences; the headline value is one sequence (batch 1)"}
        out["batch_pass"] = {"m": m, "ms_per_pass": bp_ms, "positions_per_s": m / (bp_ms * 1e-3),
                             "single_steps_ms": m * ms_dev / steps,
                             "note": "every tensor (Q4_K and Q6_K) is walked once per pass by the multi-column kernel"}
    if tp_mode:
        out["roofline"]["per_gpu"] = "bytes are this rank's share (1/%d of the weights and KV); fractions are per GPU" % world
        out["roofline"]["exchange"] = {"launches_per_step": cm_n, "ms_per_step": cm_ms, "avg_launch_us": cm_ms * 1e3 / max(cm_n, 1)}
    barrier()
    dec.close()
    return out


if __name__ == "__main__":
    main()
