"""Generates tests/golden/spec_gguf_golden.json from the REFERENCE's own code
(oracle/_ref/libflref.so: its SuffixIndex, SpecController and Gguf reader). Run where
the reference checkout is present:  python tests/golden/make_spec_gguf_golden.py
The records are what tests/test_golden_spec_gguf.py holds the library against on
machines that have no reference build: the streams and call sequences are regenerated
there from the same seeds, only the reference's answers are stored."""
import ctypes as C
import json
import os
import sys
import tempfile
import zlib

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from fast_llm_b200 import gguf              # noqa: E402
import test_gguf                            # noqa: E402
import test_spec                            # noqa: E402

SUFFIX_CASES = [(1 << 20, 3, 50, 400), (4, 3, 5, 300), (1, 3, 3, 200), (64, 5, 5, 300)]
CTRL_CASES = [{}, dict(n_max=4, alpha0=0.5, alpha_decay=0.7, lat_decay=0.5, probe_iv=3, probe_n=1, seed_slope=0.4)]


def controller_script(seed, n_max, steps=300):
    """The observe() arguments of a run, as a function of what choose() returned."""
    import random
    rng = random.Random(seed)
    script, accept = [], 0.9
    for step in range(steps):
        if step % 75 == 0:
            accept = rng.choice((0.0, 0.3, 0.9, 1.0))
        script.append((rng.random(), [rng.random() for _ in range(n_max)], rng.uniform(0.9, 1.1), accept))
    return script


def observe_args(n, rec):
    """(n_drafted, n_accepted, pass_ms) for a round in which choose() returned n."""
    u, accepts, jitter, accept = rec
    nd = int(u * (n + 1)) if n else 0
    na = sum(1 for a in accepts[:nd] if a < accept)
    return nd, na, 2.0 * (1.0 + 0.3 * nd) * jitter


def main():
    lib = C.CDLL(test_spec.REF_LIB)
    lib.flref_suffix_create.restype = C.c_void_p
    lib.flref_spec_create.restype = C.c_void_p
    for n in ("flref_spec_alpha", "flref_spec_lat_est", "flref_spec_expected_emitted"):
        getattr(lib, n).restype = C.c_double
    out = {"suffix": [], "controller": [], "gguf": []}
    buf, dg = (C.c_int32 * 16)(), (C.c_int32 * 4)()
    for cap, mm, vocab, n in SUFFIX_CASES:
        ref = C.c_void_p(lib.flref_suffix_create(C.c_uint32(cap), C.c_uint32(mm)))
        rec = []
        for t in test_spec.planted_stream(1000 + vocab + mm, n, vocab):
            lib.flref_suffix_push(ref, C.c_int32(t))
            k = lib.flref_suffix_draft(ref, C.c_int(8), buf, dg)
            rec.append([list(buf[:k]), list(dg)])
        lib.flref_suffix_destroy(ref)
        out["suffix"].append({"chain_cap": cap, "min_match": mm, "vocab": vocab, "n": n, "drafts": rec})
    for i, cfg in enumerate(CTRL_CASES):
        full = dict(n_max=7, alpha0=0.75, alpha_decay=0.90, lat_decay=0.80, probe_iv=16, probe_n=2, seed_slope=0.15)
        full.update(cfg)
        ref = C.c_void_p(lib.flref_spec_create(C.c_int(full["n_max"]), C.c_double(full["alpha0"]), C.c_double(full["alpha_decay"]),
                                               C.c_double(full["lat_decay"]), C.c_int(full["probe_iv"]), C.c_int(full["probe_n"]),
                                               C.c_double(full["seed_slope"])))
        trace = []
        for rec in controller_script(50 + i, full["n_max"]):
            n = lib.flref_spec_choose(ref)
            nd, na, ms = observe_args(n, rec)
            lib.flref_spec_observe(ref, C.c_int(nd), C.c_int(na), C.c_double(ms))
            trace.append([n, lib.flref_spec_alpha(ref).hex(), lib.flref_spec_lat_est(ref, C.c_int(full["n_max"])).hex()])
        lib.flref_spec_destroy(ref)
        out["controller"].append({"cfg": full, "seed": 50 + i, "trace": trace})
    with tempfile.TemporaryDirectory() as tmp:
        for version, alignment, parts in ((3, None, 1), (2, 64, 1), (3, 32, 3)):
            recs = test_gguf.fixture_records()
            if parts == 1:
                path = os.path.join(tmp, "g.gguf")
                gguf.write_gguf(path, test_gguf.RICH_KV, recs, alignment=alignment, version=version)
            else:
                path = gguf.write_split(os.path.join(tmp, "s"), test_gguf.RICH_KV, recs, parts, alignment=alignment)[0]
            r = test_gguf.RefGguf(path)
            view = {"counts": list(r.counts()), "tensors": [], "kv": {}}
            for j in range(r.counts()[0]):
                t = r.tensor(j)
                t["crc32"] = zlib.crc32(t.pop("bytes"))
                view["tensors"].append(t)
            for k in test_gguf.KEYS_I + ["a.f64"]:
                view["kv"][k] = [bool(r.lib.flref_gguf_has(r.h, k.encode())), r.lib.flref_gguf_kv_i(r.h, k.encode(), C.c_int64(-5)),
                                 r.lib.flref_gguf_kv_f(r.h, k.encode(), C.c_double(2.5)).hex()]
            view["strings"] = {k: r.kv_s(k, "dflt") for k in test_gguf.KEYS_S}
            view["string_arrays"] = {k: r.kv_sarr(k) for k in test_gguf.KEYS_SA}
            r.close()
            out["gguf"].append({"version": version, "alignment": alignment, "parts": parts, "view": view})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "spec_gguf_golden.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
