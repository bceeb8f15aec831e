"""Why the write kernel may skip the reference's division (horizon_kernels_b200/csrc/hkv_write.cu, block_codes_fast and
resolve_code), restated in numpy and checked against the reference's own arithmetic RN(|x| / s) -> threshold chain
(kv_fp4_ref.py:122-130, :142-145 in the reference).

The kernel brackets the quotient by |x| * RN(r (1 - 2^-20)) and |x| * RN(r (1 + 2^-20)), r = RN(1 / s), converts both
ends to E2M1 codes and, where they differ (codes k and k + 1), decides with one exact fp64 product: RN(q) <= t holds
iff q <= t + ulp(t)/2 for the "<=" thresholds (their mantissas are even, so a tie rounds down onto t), and RN(q) < t
iff q < t - ulp(pred t)/2 for the "<" thresholds. The cases below are the ones where that argument could break:
scales with few mantissa bits (every E4M3 scale times a global scale of the form amax / 2688, which puts many bf16
quotients EXACTLY on a rounding boundary), quotients within +-3 ulp of every threshold and of every boundary, and the
ends of the scale range the fast path accepts."""
import numpy as np
import pytest

import synth

THRESH = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
# rounding boundaries of the quotient between codes k and k + 1 (hkv_write.cu: kBoundary)
BOUNDARY = np.array([0.25 + 2.0 ** -26, 0.75 - 2.0 ** -25, 1.25 + 2.0 ** -24, 1.75 - 2.0 ** -24, 2.5 + 2.0 ** -23,
                     3.5 - 2.0 ** -23, 5.0 + 2.0 ** -22, 0.0])
K_UP, K_DOWN = np.float32(1 + 2.0 ** -20), np.float32(1 - 2.0 ** -20)
S_MIN, S_MAX = np.float32(1.2621774e-29), np.float32(7.9228163e28)       # fast_scale_ok: [2^-96, 2^96]


def mag(y):
    """the reference's threshold chain: ties to the even code, saturating at code 7"""
    return np.select([y <= 0.25, y < 0.75, y <= 1.25, y < 1.75, y <= 2.5, y < 3.5, y <= 5.0], [0, 1, 2, 3, 4, 5, 6], 7)


def reference_codes(ax, s):
    with np.errstate(over="ignore"):
        return mag((ax / s).astype(np.float32))                          # one IEEE fp32 division, then the chain


def kernel_codes(ax, s):
    """bracket + exact resolve, every step a single fp32 (or, in the resolve, fp64) operation as in the kernel"""
    with np.errstate(over="ignore"):
        r = (np.float32(1) / s).astype(np.float32)
        lo = mag((ax * (r * K_DOWN).astype(np.float32)).astype(np.float32))
        hi = mag((ax * (r * K_UP).astype(np.float32)).astype(np.float32))
    near = hi != lo
    assert np.all((hi - lo)[near] == 1)                                   # the bracket never spans two boundaries
    lhs, rhs = ax.astype(np.float64), BOUNDARY[np.minimum(lo, 7)] * s.astype(np.float64)
    keep = np.where(lo % 2 == 1, lhs < rhs, lhs <= rhs)
    return np.where(near & ~keep, lo + 1, lo), int(near.sum())


def e4m3_values():
    c = np.arange(1, 127)
    e, m = (c >> 3) & 15, c & 7
    return np.where(e > 0, (1 + m / 8.0) * 2.0 ** (e - 7), m * 2.0 ** -9).astype(np.float32)


def bf16_abs(seed, n, scale=1.0):
    return np.abs(synth.bf16_bits_to_f32(synth.to_bf16_bits(synth.normal(seed, (n,)) * scale)))


@pytest.mark.parametrize("seed", range(6))
def test_bracket_equals_division_on_tie_rich_scales(seed):
    """bf16 data against every E4M3 scale times a per-tensor global scale amax / (6 * 448): the benchmark's setting"""
    ax = bf16_abs(100 + seed, 1 << 16, 20.0 if seed % 2 else 1.0)
    g = [np.float32(ax.max()) / np.float32(6 * 448), np.float32(0.01), np.float32(1.0), np.float32(2.0 ** -7),
         np.float32(0.3217), np.float32(5.5 * 20 / 2688)][seed]
    sv = e4m3_values()
    s = (sv[synth.permutation(seed, ax.size) % sv.size] * g).astype(np.float32)
    got, near = kernel_codes(ax, s)
    assert np.array_equal(got, reference_codes(ax, s))
    if seed in (0, 2, 3):
        assert near > 0                                                   # the exact path was exercised


@pytest.mark.parametrize("t", list(THRESH))
def test_bracket_equals_division_around_every_threshold(t):
    """quotients on the threshold, on its rounding boundary, and up to 3 ulp to either side"""
    n = 100000
    u = synth.uniform(int(t * 100), n)
    s = np.exp(np.log(1e-3) + u * (np.log(1e4) - np.log(1e-3))).astype(np.float32)
    k = int(np.searchsorted(THRESH, t))
    for centre in (np.float64(t), BOUNDARY[k]):
        base = (centre * s.astype(np.float64)).astype(np.float32)         # |x| with |x| / s as close to the centre as fp32 allows
        for d in range(-3, 4):
            ax = base.copy()
            for _ in range(abs(d)):
                ax = np.nextafter(ax, np.float32(np.inf if d > 0 else 0)).astype(np.float32)
            got, _ = kernel_codes(ax, s)
            assert np.array_equal(got, reference_codes(ax, s)), (t, centre, d)


def test_bracket_equals_division_at_the_ends_of_the_fast_range_and_for_special_values():
    ax = np.concatenate([bf16_abs(7, 4096), bf16_abs(8, 4096, 1e30), bf16_abs(9, 4096, 1e-30),
                         np.array([0.0, np.inf, 3.3895314e38, 1e-40, 2688.0, 6.0, 5.0, 0.25], np.float32)])
    for s0 in (S_MIN, S_MAX, np.float32(1.0), np.nextafter(S_MIN, np.float32(1)), np.nextafter(S_MAX, np.float32(0))):
        s = np.full(ax.shape, s0, np.float32)
        got, _ = kernel_codes(ax, s)
        assert np.array_equal(got, reference_codes(ax, s)), float(s0)


def test_boundaries_are_exact_fp64_products():
    """the resolve compares |x| (24 bits) with boundary (at most 26 bits) * s (24 bits): at most 50 bits, exact in fp64"""
    for b in BOUNDARY[:7]:
        m, _ = np.frexp(b)
        assert (m * 2.0 ** 26) % 1 == 0                                   # a boundary has at most 26 significant bits
    s = np.float32(0.123456789)
    for b in BOUNDARY[:7]:
        exact = int(np.float64(b) * 2 ** 30) * int(np.float64(s) * 2 ** 40)          # integers: exact
        assert np.float64(b) * np.float64(s) == exact / 2.0 ** 70
