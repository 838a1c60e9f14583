"""The library's draft source, draft-length controller and GGUF reader against answers
recorded from the reference's own code (tests/golden/spec_gguf_golden.json, written by
tests/golden/make_spec_gguf_golden.py where the reference builds). Needs neither the
reference nor a GPU: streams, call sequences and files are regenerated from the seeds."""
import importlib.util
import json
import os
import zlib

import pytest

from fast_llm_b200 import gguf, spec

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(name, path):
    s = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(s)
    s.loader.exec_module(m)
    return m


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "spec_gguf_golden.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def maker():
    return _load("make_spec_gguf_golden", os.path.join(HERE, "golden", "make_spec_gguf_golden.py"))


def test_drafts_equal_recorded_reference(golden, maker):
    import test_spec
    assert [(c["chain_cap"], c["min_match"], c["vocab"], c["n"]) for c in golden["suffix"]] == maker.SUFFIX_CASES
    for case in golden["suffix"]:
        idx = spec.SuffixIndex(case["chain_cap"], case["min_match"])
        stream = test_spec.planted_stream(1000 + case["vocab"] + case["min_match"], case["n"], case["vocab"])
        for i, (t, (want, want_dg)) in enumerate(zip(stream, case["drafts"])):
            idx.push(t)
            got, dg = idx.draft(8, diag=True)
            assert got == want and list(dg) == want_dg, (case["chain_cap"], i)


def test_controller_equals_recorded_reference(golden, maker):
    for case in golden["controller"]:
        cfg = case["cfg"]
        c = spec.SpecController(**cfg)
        for step, (rec, (want_n, want_alpha, want_lat)) in enumerate(zip(maker.controller_script(case["seed"], cfg["n_max"]),
                                                                         case["trace"])):
            n = c.choose()
            assert n == want_n, step
            c.observe(*maker.observe_args(n, rec))
            assert c.alpha() == float.fromhex(want_alpha) and c.lat_est(cfg["n_max"]) == float.fromhex(want_lat), step


def test_reader_equals_recorded_reference(golden, tmp_path):
    import test_gguf
    for case in golden["gguf"]:
        recs = test_gguf.fixture_records()
        if case["parts"] == 1:
            path = tmp_path / ("g%d.gguf" % case["version"])
            gguf.write_gguf(path, test_gguf.RICH_KV, recs, alignment=case["alignment"], version=case["version"])
        else:
            path = gguf.write_split(str(tmp_path / "s"), test_gguf.RICH_KV, recs, case["parts"], alignment=case["alignment"])[0]
        view = case["view"]
        with gguf.Gguf(path) as g:
            assert list(g.counts()) == view["counts"]
            for i, want in enumerate(view["tensors"]):
                name, t = g.tensor_at(i)
                got = dict(name=name, type=t.ggml_type, n_dims=t.n_dims, ne=list(t.ne), offset=t.offset, nbytes=t.nbytes,
                           shard=t.shard, fmt=t.fmt, crc32=zlib.crc32(t.bytes()))
                assert got == want, (case, i)
            for k, (has, vi, vf) in view["kv"].items():
                assert g.has(k) == has and g.kv_i(k, -5) == vi and g.kv_f(k, 2.5) == float.fromhex(vf), k
            for k, v in view["strings"].items():
                assert g.kv_s(k, "dflt") == v, k
            for k, v in view["string_arrays"].items():
                assert g.kv_sarr(k) == v, k
