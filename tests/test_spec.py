"""CPU tests of the speculative-decoding host components, after the reference's
own (tests/test_spec.cpp): the draft source against a brute-force restatement
of its definition and against the reference's SuffixIndex on the same streams,
the controller's policy behaviours and its agreement with the reference's
SpecController call by call. No GPU is used."""
import ctypes as C
import os
import random

import pytest

from fast_llm_b200 import spec

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "..", "oracle", "_ref", "libflref.so")


def brute_draft(t, n_max, min_match):
    """Longest match of the stream's suffix ending at an earlier position (ties: the most
    recent), then the tokens that followed it (tests/test_spec.cpp:20-39)."""
    n = len(t)
    if n < 3 or n_max <= 0:
        return []
    best_len, best_end = 0, -1
    for e in range(n - 2, -1, -1):
        ln = 0
        while ln < e + 1 and ln < n - 1 and t[e - ln] == t[n - 1 - ln]:
            ln += 1
        if ln > best_len:
            best_len, best_end = ln, e
    if best_end < 0 or best_len < min_match:
        return []
    return t[best_end + 1:n][:n_max]


def planted_stream(seed, n_toks, vocab):
    """Random tokens with planted repeats of earlier spans (tests/test_spec.cpp:41-59)."""
    rng = random.Random(seed)
    s = []
    while len(s) < n_toks:
        if len(s) > 20 and rng.randrange(4) == 0:
            start = rng.randrange(len(s) - 10)
            for k in range(3 + rng.randrange(8)):
                if len(s) < n_toks:
                    s.append(s[start + k])
        else:
            s.append(rng.randrange(vocab))
    return s


def ref_lib():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref is not built")
    lib = C.CDLL(REF_LIB)
    if not hasattr(lib, "flref_suffix_create"):
        pytest.skip("oracle/_ref predates the speculative shim")
    lib.flref_suffix_create.restype = C.c_void_p
    lib.flref_spec_create.restype = C.c_void_p
    for n in ("flref_spec_alpha", "flref_spec_lat_est", "flref_spec_expected_emitted"):
        getattr(lib, n).restype = C.c_double
    return lib


@pytest.mark.parametrize("seed,n_toks,vocab", [(s, 600, 50) for s in range(1, 9)] + [(s, 400, 5) for s in range(9, 13)])
def test_draft_equals_brute_force(seed, n_toks, vocab):
    idx = spec.SuffixIndex(1 << 20, 3)
    stream = planted_stream(seed, n_toks, vocab)
    for i, t in enumerate(stream):
        idx.push(t)
        if i + 1 > 8 and (i + 1) % 7 == 0:
            assert idx.draft(16) == brute_draft(stream[:i + 1], 16, 3), i
    assert idx.size() == n_toks


def test_draft_basics():
    idx = spec.SuffixIndex(64, 3)
    for t in (1, 2, 3, 4, 5):
        idx.push(t)
    assert idx.draft(8) == []                      # nothing repeats
    i2 = spec.SuffixIndex(64, 3)
    for t in (10, 11, 12, 13, 14, 7, 8, 9, 10, 11, 12):
        i2.push(t)
    assert i2.draft(8) == [13, 14, 7, 8, 9, 10, 11, 12]   # the stream after the match, up to n_max
    assert i2.draft(2) == [13, 14] and i2.draft(0) == []
    i3 = spec.SuffixIndex(64, 3)
    for _ in range(50):
        i3.push(42)
    assert i3.draft(4) == [42]                     # the longest match ends one before the tail: one token left
    i3.reset()
    assert i3.size() == 0 and i3.draft(4) == []
    i4 = spec.SuffixIndex(64, 5)                   # a 3-token match is shorter than min_match 5
    for t in (1, 2, 3, 9, 8, 1, 2, 3):
        i4.push(t)
    toks, dg = i4.draft(4, diag=True)
    assert toks == [] and dg[0] == 1 and dg[1] == 1 and dg[2] == 3


@pytest.mark.parametrize("chain_cap,min_match,vocab", [(1 << 20, 3, 50), (4, 3, 5), (2, 3, 3), (1, 3, 3), (64, 5, 5), (8, 1, 2)])
def test_draft_equals_reference_index(chain_cap, min_match, vocab):
    lib = ref_lib()
    ref = C.c_void_p(lib.flref_suffix_create(C.c_uint32(chain_cap), C.c_uint32(min_match)))
    idx = spec.SuffixIndex(chain_cap, min_match)
    out, dg = (C.c_int32 * 16)(), (C.c_int32 * 4)()
    for i, t in enumerate(planted_stream(100 + chain_cap % 97 + vocab, 500, vocab)):
        lib.flref_suffix_push(ref, C.c_int32(t))
        idx.push(t)
        for n_max in (16, 3):
            n = lib.flref_suffix_draft(ref, C.c_int(n_max), out, dg)
            got, got_dg = idx.draft(n_max, diag=True)
            assert got == list(out[:n]), (i, n_max)
            assert got_dg == tuple(dg), (i, n_max)    # a bounded walk examines the same entries
    lib.flref_suffix_destroy(ref)


def test_controller_policy():
    """The behaviours the reference's test asserts (tests/test_spec.cpp:95-127)."""
    assert spec.SpecController().choose() == 7                  # cold start: a full draft
    c1 = spec.SpecController()
    for _ in range(30):
        c1.observe(4, 4, 10.0 + 0.3 * 4)
    assert c1.alpha() > 0.9 and c1.choose() >= 4                 # high acceptance: long drafts
    c2 = spec.SpecController()
    for _ in range(40):
        c2.observe(4, 0, 12.0)
    c2.observe(0, 0, 10.0)
    assert c2.alpha() < 0.1
    zeros = probes = 0
    for _ in range(40):
        n = c2.choose()
        if n == 0:
            zeros += 1
            c2.observe(0, 0, 10.0)
        else:
            probes += 1
            c2.observe(n, 0, 11.0)
    assert zeros > 30 and probes >= 1                            # sustained rejection: no drafts, but probes
    c3, c4 = spec.SpecController(), spec.SpecController()
    for _ in range(20):
        for n in range(8):
            c3.observe(n, int(0.8 * n + 0.5), 10.0 * (1.0 + 0.05 * n))
            c4.observe(n, int(0.8 * n + 0.5), 10.0 * (1.0 + 1.50 * n))
    assert c3.choose() >= c4.choose()                            # steep latency growth: shorter drafts


@pytest.mark.parametrize("cfg", [{}, dict(n_max=4, alpha0=0.5, alpha_decay=0.7, lat_decay=0.5, probe_iv=3, probe_n=1,
                                          seed_slope=0.4)])
def test_controller_equals_reference_call_by_call(cfg):
    lib = ref_lib()
    mine = spec.SpecController(**cfg)
    c = mine.cfg
    ref = C.c_void_p(lib.flref_spec_create(C.c_int(c.n_max), C.c_double(c.alpha0), C.c_double(c.alpha_decay),
                                           C.c_double(c.lat_decay), C.c_int(c.probe_iv), C.c_int(c.probe_n),
                                           C.c_double(c.seed_slope)))
    rng = random.Random(7)
    phase_accept = 0.9
    for step in range(600):
        if step % 150 == 0:
            phase_accept = rng.choice((0.0, 0.3, 0.9, 1.0))
        n = mine.choose()
        assert n == lib.flref_spec_choose(ref), step
        nd = rng.randrange(n + 1) if n else 0                    # the draft source may return fewer
        na = sum(1 for _ in range(nd) if rng.random() < phase_accept)
        ms = 2.0 * (1.0 + 0.3 * nd) * rng.uniform(0.9, 1.1)
        mine.observe(nd, na, ms)
        lib.flref_spec_observe(ref, C.c_int(nd), C.c_int(na), C.c_double(ms))
        assert mine.alpha() == lib.flref_spec_alpha(ref)
        for k in (0, 1, c.n_max, 15, 40, -3):
            assert mine.lat_est(k) == lib.flref_spec_lat_est(ref, C.c_int(k))
            assert mine.expected_emitted(k) == lib.flref_spec_expected_emitted(ref, C.c_int(k))
    lib.flref_spec_destroy(ref)
