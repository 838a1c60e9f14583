"""Generates tests/golden/decode_ops_golden.npz from the REFERENCE's own code
(oracle/_ref/libflref.so, built from the reference sources by oracle/Makefile).
Run where the reference checkout is present:  python tests/golden/make_golden.py
The fixture is small (seeded inputs + the reference's outputs) and is what pins
the plain-C port on machines that have no reference checkout."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from fast_llm_b200 import capi, synth   # noqa: E402
from oracle import pyoracle             # noqa: E402


def main():
    ref = pyoracle.Oracle("reference")
    rng = np.random.default_rng(20240)
    out = {}
    for name, fmt, rows, cols in (("q8_0", capi.Q8_0, 4, 1408), ("q5_0", capi.Q5_0, 4, 1408),
                                  ("q4_k", capi.Q4_K, 8, 2048), ("q6_k", capi.Q6_K, 8, 2048)):
        w = synth.quant_tensor(fmt, rng, rows, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        out[name + "_w"], out[name + "_x"] = w, x
        out[name + "_deq"] = ref.dequant(fmt, w, rows, cols)
        out[name + "_y"] = ref.matvec(fmt, w, rows, cols, x)
    n_head, n_kv, d, kv = 8, 2, 128, 150
    q = rng.standard_normal((n_head, d)).astype(np.float32)
    k = (rng.standard_normal((n_kv, kv, d)) / np.sqrt(d)).astype(np.float16)
    v = (rng.standard_normal((n_kv, kv, d)) / np.sqrt(d)).astype(np.float16)
    scale = float(1.0 / np.sqrt(np.float32(d)))
    out.update(attn_q=q, attn_k=k, attn_v=v, attn_kv_len=kv, attn_scale=scale,
               attn_out=ref.attn_gqa_f16(q, k, v, kv, scale))
    nx = rng.standard_normal(1024).astype(np.float32)
    nw = rng.uniform(0.9, 1.1, 1024).astype(np.float32)
    out.update(norm_x=nx, norm_w=nw, norm_y=ref.rmsnorm(nw, nx, 1e-5), silu_y=ref.silu_mul(nx, nw))
    rx = rng.standard_normal(8 * 128).astype(np.float32)
    out.update(rope_x=rx, rope_y=ref.rope(rx, 4097, 8, 128, 0, 128, 500000.0))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_ops_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
