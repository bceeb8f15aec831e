"""Why the write kernel may skip the reference's division (horizon_kernels_b200/csrc/hkv_write.cu: div_ok, div2,
block_codes_fast), restated in numpy and checked against the reference's own arithmetic RN(|x| / s) -> threshold chain
(kv_fp4_ref.py:122-130, :142-145 in the reference).

The kernel computes r = RN(1 / s) once per scale and then, per value, y0 = RN(|x| r), rem = fma(-s, y0, |x|) and
q = fma(rem, r, y0). y0 is within one ulp of the quotient, so rem is exactly representable, and rounding y0 + rem r once
gives the correctly rounded quotient (Markstein's theorem), the same bits as the division, as long as nothing over- or
underflows; div_ok (2^-90 <= s <= 2^96, |x| <= 2^20 s) keeps every quotient of 0.125 or more inside that range (rem
is a multiple of ulp(s) ulp(y0)), smaller quotients may lose bits of rem to underflow and still get code 0, the first
rounding boundary being 0.25. The fused multiply-add is emulated with
fp64 and round-to-odd, and that emulation is itself checked against exact rational arithmetic. The cases are the ones
where the argument could break: scales with few mantissa bits (every E4M3 scale times a global scale of the form
amax / 2688, which puts many bf16 quotients EXACTLY on a rounding boundary), quotients within +-3 ulp of every
threshold, scales whose mantissa is all ones (the worst case for the reciprocal), and the ends of the accepted range."""
from fractions import Fraction

import numpy as np
import pytest

import synth

THRESH = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
S_MIN, S_MAX = np.float32(2.0 ** -90), np.float32(2.0 ** 96)             # div_ok: [2^-90, 2^96]


def mag(y):
    """the reference's threshold chain: ties to the even code, saturating at code 7"""
    return np.select([y <= 0.25, y < 0.75, y <= 1.25, y < 1.75, y <= 2.5, y < 3.5, y <= 5.0], [0, 1, 2, 3, 4, 5, 6], 7)


def fma32(a, b, c):
    """RN32(a * b + c) for float32 arrays: the product is exact in fp64, the sum is rounded to odd in fp64 (53 bits are
    more than 24 + 2), and the final rounding to fp32 is then the single rounding of the exact value"""
    a64, b64, c64 = a.astype(np.float64), b.astype(np.float64), c.astype(np.float64)
    p = a64 * b64
    s = p + c64
    bb = s - p
    e = (p - (s - bb)) + (c64 - bb)                                       # the sum's rounding error, exact (two-sum)
    even = (s.view(np.int64) & 1) == 0
    s = np.where((e != 0) & even, np.nextafter(s, np.where(e > 0, np.inf, -np.inf)), s)
    return s.astype(np.float32)


def div_ok(s, ax):
    with np.errstate(over="ignore"):
        return (s >= S_MIN) & (s <= S_MAX) & (ax <= (s * np.float32(1048576.0)).astype(np.float32))


def kernel_quotient(ax, s):
    r = (np.float32(1) / s).astype(np.float32)
    y0 = (ax * r).astype(np.float32)
    rem = fma32(-s, y0, ax)
    return fma32(rem, r, y0)


def check(ax, s):
    """bits of the quotient where it is at least 0.125, codes everywhere, for the pairs div_ok accepts"""
    ok = div_ok(s, ax)
    ax, s = ax[ok], s[ok]
    q, ref = kernel_quotient(ax, s), (ax / s).astype(np.float32)
    big = ref >= np.float32(0.125)
    assert np.array_equal(q[big].view(np.uint32), ref[big].view(np.uint32))
    assert np.array_equal(mag(q), mag(ref))
    return int(ok.sum())


def e4m3_values():
    c = np.arange(1, 127)
    e, m = (c >> 3) & 15, c & 7
    return np.where(e > 0, (1 + m / 8.0) * 2.0 ** (e - 7), m * 2.0 ** -9).astype(np.float32)


def bf16_abs(seed, n, scale=1.0):
    return np.abs(synth.bf16_bits_to_f32(synth.to_bf16_bits(synth.normal(seed, (n,)) * scale)))


def test_fused_multiply_add_emulation_is_exact():
    n = 4000
    a = (synth.normal(1, (n,)) * 3).astype(np.float32)
    b = (synth.normal(2, (n,)) * 3).astype(np.float32)
    c = (-(a.astype(np.float64) * b.astype(np.float64)) * (1 + synth.normal(3, (n,)) * 2.0 ** -22)).astype(np.float32)
    got = fma32(a, b, c)                                                  # heavy cancellation: the hard case
    for i in range(n):
        exact = Fraction(float(a[i])) * Fraction(float(b[i])) + Fraction(float(c[i]))
        lo = np.float32(float(exact))                                     # float(Fraction) rounds once to fp64 ...
        # ... so decide between the two fp32 neighbours of the exact value with rational arithmetic
        cands = sorted({float(lo), float(np.nextafter(lo, np.float32(np.inf))), float(np.nextafter(lo, np.float32(-np.inf)))})
        best = min(cands, key=lambda v: (abs(Fraction(v) - exact), int(np.float32(v).view(np.uint32)) & 1))
        assert float(got[i]) == best, (a[i], b[i], c[i])


@pytest.mark.parametrize("seed", range(6))
def test_quotient_equals_division_on_tie_rich_scales(seed):
    """bf16 data against every E4M3 scale times a per-tensor global scale amax / (6 * 448): the benchmark's setting"""
    ax = bf16_abs(100 + seed, 1 << 16, 20.0 if seed % 2 else 1.0)
    g = [np.float32(ax.max()) / np.float32(6 * 448), np.float32(0.01), np.float32(1.0), np.float32(2.0 ** -7),
         np.float32(0.3217), np.float32(5.5 * 20 / 2688)][seed]
    sv = e4m3_values()
    s = (sv[synth.permutation(seed, ax.size) % sv.size] * g).astype(np.float32)
    assert check(ax, s) > ax.size // 2
    if seed in (0, 2, 3):                                                 # quotients exactly on a rounding boundary occur
        q = (ax / s).astype(np.float32)
        assert np.isin(q, THRESH.astype(np.float32)).sum() > 0


@pytest.mark.parametrize("t", list(THRESH))
def test_quotient_equals_division_around_every_threshold(t):
    """quotients on the threshold and up to 3 ulp to either side"""
    n = 100000
    u = synth.uniform(int(t * 100), n)
    s = np.exp(np.log(1e-3) + u * (np.log(1e4) - np.log(1e-3))).astype(np.float32)
    base = (np.float64(t) * s.astype(np.float64)).astype(np.float32)      # |x| with |x| / s as close to t as fp32 allows
    for d in range(-3, 4):
        ax = base.copy()
        for _ in range(abs(d)):
            ax = np.nextafter(ax, np.float32(np.inf if d > 0 else 0)).astype(np.float32)
        assert check(ax, s) == n


def test_quotient_equals_division_for_scales_with_a_mantissa_of_all_ones():
    for bits in (0x3FFFFFFF, 0x3F7FFFFF, 0x407FFFFF, 0x3EFFFFFF, 0x3FFFFFFE, 0x3F800001):
        s0 = np.array([bits], np.uint32).view(np.float32)[0]
        ax = (synth.uniform(bits & 0xFFFF, 400000) * 8).astype(np.float32) * s0
        assert check(ax.astype(np.float32), np.full(ax.shape, s0, np.float32)) == ax.size


def test_quotient_equals_division_at_the_ends_of_the_accepted_range_and_for_special_values():
    ax = np.concatenate([bf16_abs(7, 4096), bf16_abs(8, 4096, 1e30), bf16_abs(9, 4096, 1e-30),
                         np.array([0.0, np.inf, 3.3895314e38, 1e-40, 2688.0, 6.0, 5.0, 0.25], np.float32)])
    seen = 0
    for s0 in (S_MIN, S_MAX, np.float32(1.0), np.nextafter(S_MIN, np.float32(1)), np.nextafter(S_MAX, np.float32(0)),
               np.nextafter(np.float32(2.0 ** -89), np.float32(0))):      # the smallest scales, one with all mantissa bits set
        # values scaled into the scale's neighbourhood too, so that the accepted range is populated at both ends
        both = np.concatenate([ax, (bf16_abs(10, 4096) * s0).astype(np.float32),
                               (bf16_abs(11, 4096, 1e5) * s0).astype(np.float32)])
        with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
            seen += check(both, np.full(both.shape, s0, np.float32))
    assert seen > 6 * 8192
    # outside the accepted range the kernel divides: div_ok must refuse what would overflow on the way
    assert not div_ok(np.float32(1e-28), np.float32(1e-28)) and not div_ok(np.float32(1.0), np.float32(2e6))
    assert not div_ok(np.float32(0.0), np.float32(0.0)) and not div_ok(np.float32(np.nan), np.float32(1.0))


def test_lane_index_division_by_multiplication_is_exact():
    """the write kernel splits a lane index n < 2^31 into (token, block of the token) with the host's round-up magic
    number instead of a 64-bit division (hkv_write.cu: div_magic / div_shift): (umulhi(m, n) + n) >> l == n // d for
    every blocks-per-token count d = 2 * kv heads * head_dim / 16 the library accepts"""
    ds = sorted({2 * kvh * nb for kvh in range(1, 1025) for nb in (8, 16)})
    top = (1 << 31) - 1
    for d in ds:
        l = 0
        while (1 << l) < d:
            l += 1
        m = (((1 << l) - d) << 32) // d + 1
        assert 0 < m < (1 << 32)
        k = np.array([0, 1, 2, 3, 1000, top // d - 1, top // d], np.int64)
        n = np.unique(np.clip(np.concatenate([k * d - 1, k * d, k * d + 1, k * d + d - 1, [top, top - 1, 12345678]]), 0, top))
        q = (((m * n.astype(object)) >> 32) + n.astype(object))
        assert all(int(v) < (1 << 32) for v in q)                         # the 32-bit sum cannot overflow
        assert [int(v) >> l for v in q] == [int(v) // d for v in n], d
