"""CPU restatement of the arithmetic the tensor-core matvec's integer forms rely on (csrc/matvec_tc.cu:
q4k_block_i8, q6k_block_i8 and the activation prologue), checked with numpy against exact integer / f64 sums:
the balanced-digit split of the fixed-point activation, the nibble masks of Q4_K with the factor 16 of the
high nibbles, the - 32 of Q6_K through the group sums, and the bound on what an outlier costs its sub-block."""
import numpy as np


def digits_of(n):
    """The kernel's split: n + 0x808080 holds the balanced digits, each plus 128, in its low three bytes; the top
    byte is the signed leading digit. Returns (D0, D1, D2, D3) with n = D0 2^24 + D1 2^16 + D2 2^8 + D3."""
    u = (n.astype(np.int64) + 0x00808080) & 0xFFFFFFFF
    v = u ^ 0x00808080
    by = [((v >> (8 * k)) & 0xFF).astype(np.int64) for k in range(4)]
    s8 = [np.where(b >= 128, b - 256, b) for b in by]
    return s8[3], s8[2], s8[1], s8[0]


def fixed_point(x):
    """Per 32-element sub-block: exponent e with amax / 2^e in [2^29, 2^30), n = round-to-nearest-even(x / 2^e)."""
    amax = np.max(np.abs(x))
    if amax == 0:
        return 0, np.zeros(x.shape, np.int64)
    e = int(np.floor(np.log2(amax))) - 29
    e = max(-122, min(e, 98))
    return e, np.rint(x.astype(np.float64) * 2.0 ** -e).astype(np.int64)


def test_balanced_digits_recompose_and_fit_a_signed_byte():
    rng = np.random.default_rng(1)
    n = np.concatenate([rng.integers(-(2 ** 30) + 1, 2 ** 30, 20000), [0, 1, -1, 127, 128, -128, -129, 2 ** 30 - 1, -(2 ** 30) + 1,
                                                                        0x7F7F7F, 0x808080, -0x808080, 0x7FFFFF, 0x800000]])
    d0, d1, d2, d3 = digits_of(n)
    assert np.array_equal(d0 * 2 ** 24 + d1 * 2 ** 16 + d2 * 2 ** 8 + d3, n)
    for d in (d1, d2, d3):
        assert d.min() >= -128 and d.max() <= 127
    assert d0.min() >= -65 and d0.max() <= 64


def test_q4k_sub_block_dot_from_digit_planes_is_exact():
    """Low nibbles as they are, high nibbles as (byte & 0xF0) = 16 q with 1/16 in the scale; four plane sums put
    together as ((P0 256 + P1) 65536 + (P2 256 + P3)): equal to the integer dot product, and inside int32."""
    rng = np.random.default_rng(2)
    for _ in range(200):
        packed = rng.integers(0, 256, 32).astype(np.int64)          # one chunk: low nibbles sub-block 2t, high 2t+1
        x = rng.standard_normal(64).astype(np.float32) * np.float32(10.0 ** rng.integers(-20, 20))
        for kind, q, xs in ((0, packed & 0x0F, x[:32]), (1, packed & 0xF0, x[32:])):
            e, n = fixed_point(xs)
            planes = digits_of(n)
            p = [int(np.sum(q * d)) for d in planes]
            assert all(abs(v) < 2 ** 31 for v in p)
            hi, lo = p[0] * 256 + p[1], p[2] * 256 + p[3]
            assert abs(hi) < 2 ** 31 and abs(lo) < 2 ** 31
            total = hi * 65536 + lo
            assert total == int(np.sum(q * n))
            scale = 2.0 ** e / (16.0 if kind else 1.0)
            want = float(np.sum((packed >> 4 if kind else packed & 0x0F) * n)) * 2.0 ** e
            assert total * scale == want


def test_q6k_offset_through_group_sums():
    rng = np.random.default_rng(3)
    for _ in range(200):
        q = rng.integers(0, 64, 16).astype(np.int64)
        x = rng.standard_normal(32).astype(np.float32)
        e, n = fixed_point(x)                                       # the scale of the 32-column sub-block
        n16, x16 = n[:16], x[:16].astype(np.float64)
        planes = digits_of(n16)
        p = [int(np.sum(q * d)) for d in planes]
        f = ((p[0] * 256 + p[1]) * 65536 + (p[2] * 256 + p[3])) * 2.0 ** e
        got = f - 32.0 * float(np.sum(x16))
        want = float(np.sum((q - 32) * x16))
        # the digits carry x to 2^-30 of the sub-block's maximum: the difference is that quantisation, not the offset
        assert abs(got - want) <= 64 * 16 * 2.0 ** (e - 1) + 1e-12 * abs(want)


def test_an_outlier_costs_only_its_own_sub_block():
    rng = np.random.default_rng(4)
    x = rng.standard_normal(256).astype(np.float32)
    x[77] *= 1e4
    err = np.zeros(256)
    for sb in range(8):
        e, n = fixed_point(x[32 * sb:32 * sb + 32])
        err[32 * sb:32 * sb + 32] = np.abs(n * 2.0 ** e - x[32 * sb:32 * sb + 32].astype(np.float64))
    own = slice(64, 96)
    assert err[own].max() <= 2.0 ** -30 * abs(x[77])                # 30 bits under the outlier: 1e-5 of a unit element
    other = np.ones(256, bool); other[own] = False
    assert err[other].max() <= 2.0 ** -29 * np.abs(x[other]).max()
