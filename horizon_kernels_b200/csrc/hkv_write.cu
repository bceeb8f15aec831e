// Quantize-on-write for the NVFP4 paged KV cache (sm_100a).
//
// A block of 16 consecutive channels of one (token, kv head, side) is 32 bytes of bf16 in and 8 code bytes + 1 scale
// byte out, stored at slot = page * PS + position. The E4M3 block scale is picked (optionally) by the reference's
// 4-candidate squared-error search. Large launches give every block to one lane, which scores the candidates in turn;
// small launches (decode appends) give it to a quad, one candidate per lane. The 16 magnitude codes of a candidate
// live in two registers (a nibble each), produced eight at a time by the hardware E2M1 conversion.
//
// Bit-exactness: the result must equal the reference's PyTorch quantiser (kv_fp4_ref.py:159-186 `quantize_rows`,
// rules at kv_fp4_ref.py:15-25) byte for byte. Every arithmetic step therefore produces the result of a single IEEE
// fp32 operation, issued through an explicit intrinsic or an explicit .rn instruction: no fast-math, and no
// contraction where the reference rounds twice (the one place the assembler would contract is written so that it
// cannot, see sub_from). The squared error is summed sequentially over i = 0..15 and a later candidate wins only on a
// strict "<".
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "hkv_common.cuh"

namespace hkv {

int record_cuda(cudaError_t e);

struct WriteParams {
  const __nv_bfloat16* key;
  const __nv_bfloat16* val;
  long long ks0, ks1, vs0, vs1;
  uint8_t* kd;
  uint8_t* ksf;
  uint8_t* vd;
  uint8_t* vsf;
  long long dsp, dst, dsh, ssp, sst, ssh;
  const long long* slots;
  long long n_slots;
  const float* gk;
  const float* gv;
  const float* signs;                              // +-1 per channel of the optional key rotation, or null
  float rot_scale;                                 // head_dim^-0.5 rounded to fp32
  int PS, KVH;
  // lane index / blocks per token as (umulhi(div_magic, n) + n) >> div_shift, exact for n < 2^31; div_shift < 0: the
  // launch has 2^31 lanes or more and the kernel divides
  unsigned div_magic;
  int div_shift;
};

// e4m3fn of x >= 0, round to nearest even, saturating at 448 (kv_fp4_ref.py:94-97)
__device__ __forceinline__ unsigned e4m3_enc(float x) {
  return (unsigned)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
// value of a non-negative finite e4m3 code 0..126 (exact)
__device__ __forceinline__ float e4m3_dec(unsigned c) {
  const unsigned e = (c >> 3) & 15u, m = c & 7u;
  return e ? __uint_as_float(((e + 120u) << 23) | (m << 20)) : __fmul_rn((float)m, 0.001953125f);
}
// E2M1 magnitude code of y >= 0, ties to the even code, saturating (kv_fp4_ref.py:122-130)
__device__ __forceinline__ unsigned e2m1_mag(float y) {
  return y <= 0.25f ? 0u : y < 0.75f ? 1u : y <= 1.25f ? 2u : y < 1.75f ? 3u : y <= 2.5f ? 4u : y < 3.5f ? 5u
       : y <= 5.0f ? 6u : 7u;
}
__device__ __forceinline__ unsigned mag_of(float ax, float s) { return s > 0.0f ? e2m1_mag(__fdiv_rn(ax, s)) : 0u; }

// ---- packed fp32 pairs --------------------------------------------------------------------------------------------
// sm_100 has fp32 instructions on register pairs (mul / fma .f32x2): each half is an ordinary IEEE operation with
// round to nearest even, so two of the reference's operations cost one issue slot. Two neighbouring channels of a block
// travel as one pair.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float lo(f32x2 v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi(f32x2 v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// RN(a - p) for a product p = mul2(..): written as fma(p, -1, a), one rounding of the exact difference like a
// subtraction. A sub.rn.f32x2 (or add) fed by a mul.rn.f32x2 is contracted by ptxas 12.9 into ONE fused multiply-add,
// rounding once where the reference rounds twice (seen as a different winner of the scale search in about one block in
// 10^5); an fma cannot absorb the multiply that feeds its first operand. Only the square of the result is used, so the
// sign (a - p instead of the reference's p - a) does not matter: rounding to nearest is symmetric.
__device__ __forceinline__ f32x2 sub_from(f32x2 a, f32x2 p) { return fma2(p, 0xbf800000bf800000ull, a); }

// ---- the quotients without a division instruction -------------------------------------------------------------------
// The reference rounds y = RN(ax / s) onto the E2M1 grid, with one s for the 16 values of a block. With r = RN(1 / s)
// (one IEEE reciprocal per scale) the quotient of every value takes three multiply-adds: y0 = RN(ax * r) is within one
// ulp of ax / s, rem = ax - s * y0 is then exactly representable (a single fma computes it without error), and
// RN(y0 + rem * r) is the correctly rounded quotient (Markstein's theorem: it needs r to be the correctly rounded
// reciprocal, which __frcp_rn is, and no over- or underflow on the way). div_ok states the range in which nothing over-
// or underflows for every quotient of 0.125 or more (rem is a multiple of ulp(s) ulp(y0) >= 2^-113 2^-26; smaller
// quotients may lose bits of rem to underflow, move by an ulp, and still get code 0, the first rounding boundary being
// 0.25): 2^-90 <= s <= 2^96 and amax <= 2^20 s. Outside it the IEEE-division path runs. The
// hardware conversion cvt.rn.satfinite.e2m1x2.f32 is identical to the reference's threshold chain for every
// non-negative fp32 input. hkv_selftest_codec compares both statements with the division instruction and the chain.
__device__ __forceinline__ bool div_ok(float s, float amax) {
  return s >= 0x1p-90f && s <= 0x1p+96f && amax <= s * 1048576.0f;
}
__device__ __forceinline__ f32x2 div2(f32x2 a, f32x2 r2, f32x2 neg_s2) {
  const f32x2 y0 = mul2(a, r2);
  const f32x2 rem = fma2(neg_s2, y0, a);
  return fma2(rem, r2, y0);
}
// E2M1 magnitude codes of y0 .. y7 (all >= 0), value i in nibble i
__device__ __forceinline__ uint32_t e2m1_codes8(float y0, float y1, float y2, float y3, float y4, float y5, float y6,
                                                float y7) {
  uint32_t w;
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
      "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
      : "=r"(w)
      : "f"(y0), "f"(y1), "f"(y2), "f"(y3), "f"(y4), "f"(y5), "f"(y6), "f"(y7));
  return w;
}

// the same, and the E2M1 values of the eight codes as four f16x2 (value 2j in the low half of v[j]): the conversion
// back reads the code bytes where the conversion forth left them
__device__ __forceinline__ uint32_t e2m1_codes8_values(float y0, float y1, float y2, float y3, float y4, float y5,
                                                       float y6, float y7, uint32_t (&v)[4]) {
  uint32_t w;
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %8, %7;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %10, %9;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %12, %11;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, t0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, t1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, t2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %4, t3;\n\t"
      "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
      : "=r"(w), "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
      : "f"(y0), "f"(y1), "f"(y2), "f"(y3), "f"(y4), "f"(y5), "f"(y6), "f"(y7));
  return w;
}

// the 16 magnitude codes of a block under scale s: value i in nibble i % 8 of word i / 8
struct BlockCodes {
  uint32_t w[2];
};
// AX[j] = (|x[2j]|, |x[2j + 1]|). ERR: also the sequential squared error of the block under these codes
// (kv_fp4_ref.py:148-156: single IEEE operations, i = 0..15), from the E2M1 values the conversion's own asm block
// returns. (With the conversion forth and the conversion back in separate asm statements, joined only by the packed
// word, nvcc 12.9 lost bytes 2 and 3 of the first word inside the unrolled four-candidate loop.)
template <bool ERR>
__device__ __forceinline__ BlockCodes block_codes_fast(const f32x2 (&AX)[8], float s, float r, float& err) {
  const f32x2 r2 = pk(r, r), ns2 = pk(-s, -s), s2 = pk(s, s);
  BlockCodes c;
  float acc = 0.0f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const f32x2 q0 = div2(AX[4 * h], r2, ns2), q1 = div2(AX[4 * h + 1], r2, ns2), q2 = div2(AX[4 * h + 2], r2, ns2),
                q3 = div2(AX[4 * h + 3], r2, ns2);
    if (!ERR) {
      c.w[h] = e2m1_codes8(lo(q0), hi(q0), lo(q1), hi(q1), lo(q2), hi(q2), lo(q3), hi(q3));
    } else {
      uint32_t v[4];
      c.w[h] = e2m1_codes8_values(lo(q0), hi(q0), lo(q1), hi(q1), lo(q2), hi(q2), lo(q3), hi(q3), v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 hv = u32_as_h2(v[j]);
        const f32x2 d = sub_from(AX[4 * h + j], mul2(pk(__low2float(hv), __high2float(hv)), s2));
        const f32x2 q = mul2(d, d);
        acc = (h == 0 && j == 0) ? lo(q) : __fadd_rn(acc, lo(q));
        acc = __fadd_rn(acc, hi(q));
      }
    }
  }
  err = acc;
  return c;
}
__device__ __forceinline__ BlockCodes block_codes_exact(const f32x2 (&AX)[8], float s) {   // IEEE divisions
  BlockCodes c;
  c.w[0] = c.w[1] = 0u;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c.w[j >> 2] |= mag_of(lo(AX[j]), s) << (8 * (j & 3));
    c.w[j >> 2] |= mag_of(hi(AX[j]), s) << (8 * (j & 3) + 4);
  }
  return c;
}
// sequential squared error of the block for given codes (kv_fp4_ref.py:148-156): single IEEE operations, i = 0..15
__device__ __forceinline__ float codes_sse(const f32x2 (&AX)[8], const BlockCodes& c, float s) {
  const f32x2 s2 = pk(s, s);
  float acc = 0.0f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t v[4];                                // f16x2 values of the word's code pairs
    e2m1x8_to_f16x2(c.w[h], v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 hv = u32_as_h2(v[j]);
      const f32x2 d = sub_from(AX[4 * h + j], mul2(pk(__low2float(hv), __high2float(hv)), s2));
      const f32x2 q = mul2(d, d);
      acc = (h == 0 && j == 0) ? lo(q) : __fadd_rn(acc, lo(q));
      acc = __fadd_rn(acc, hi(q));
    }
  }
  return acc;
}
__device__ __forceinline__ void score(const f32x2 (&AX)[8], float amax, float sc, BlockCodes& c, float& err,
                                      bool want_err) {
  if (div_ok(sc, amax)) {
    const float r = __frcp_rn(sc);
    c = want_err ? block_codes_fast<true>(AX, sc, r, err) : block_codes_fast<false>(AX, sc, r, err);
  } else {                                        // rare: a zero or extreme scale
    c = block_codes_exact(AX, sc);
    if (want_err) err = codes_sse(AX, c, sc);
  }
}

// LPB lanes own one block of 16 consecutive channels of one (token, kv head, side). LPB = 1 (prefill-sized launches):
// the lane reads the block's 32 bytes, scores the four scale candidates one after the other, keeps the codes of the
// best one and stores 8 code bytes and the scale byte: consecutive lanes cover consecutive blocks, so a warp reads 1 KB
// and stores 256 B contiguous. LPB = 4 (few tokens, latency matters): the four lanes of a quad read the same block,
// lane k scores candidate k, the quad agrees on the winner with shuffles in candidate order (strict "<", so the
// earliest candidate wins a tie, as in the reference) and every lane stores 4 of the 16 codes.
//
// HAD = 1 (with LPB = 1): the keys are rotated first, k' = FWHT(k * signs) * head_dim^-0.5 in fp32 with the
// reference's butterfly order (kv_fp4_ref.py:31-35, :55-87), and quantised from the fp32 result. The D / 16 lanes of
// a key row sit side by side in a warp: stages h = 1 .. 8 run inside a lane, the others exchange with the lane
// 1, 2, 4 (, 8) positions away. Values are never rotated.
//
// K8 = 1 (with LPB = 1): the K8V4 slot of the reference (kv_fp4_ref.py:283-311): keys are stored as D signed E4M3
// bytes, e4m3(k / gk) with an IEEE division, round to nearest even, saturating at +-448 (what vLLM's fp8 cache
// holds); values keep the FP4 format. A key lane stores 16 bytes instead of 8 code bytes + a scale byte.
template <int D, int SEARCH, int LPB, int HAD, int K8 = 0>
__global__ void __launch_bounds__(256) write_kernel(const WriteParams p) {
  constexpr int NB = D / 16;                      // blocks per row
  pdl_wait();                                     // inputs and the cache may come from the preceding launch
  pdl_launch_dependents();
  const int n_blocks = 2 * p.KVH * NB;            // per token (a multiple of 16)
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPB;
  const int cand = LPB == 4 ? (threadIdx.x & 3) : 0;
  long long t;
  if (p.div_shift >= 0) {
    // gid < 2^31 (the host checked): gid / n_blocks by multiplication with the host's magic number
    const unsigned n = (unsigned)gid;
    t = (__umulhi(p.div_magic, n) + n) >> p.div_shift;
  } else {
    t = gid / n_blocks;
  }
  const int bid = (int)(gid - t * n_blocks);
  // With LPB == 4 a warp holds one token's blocks, so this exit is warp-uniform. With the rotation the lanes of a warp
  // exchange values, so lanes past the end stay (on the last token's data) and only skip the stores.
  const bool in_range = t < p.n_slots;
  if (!in_range) {
    if (!HAD) return;
    t = p.n_slots - 1;
  }
  const long long slot = p.slots[t];
  // a quad shares its token, so `active` is uniform in a quad; inactive lanes still take part in the shuffles below
  const bool active = in_range && slot >= 0;
  long long page = 0, pos = 0;
  if (active) {
    if ((p.PS & (p.PS - 1)) == 0) {
      const int sh = 31 - __clz(p.PS);
      page = slot >> sh;
      pos = slot & (p.PS - 1);
    } else {
      page = slot / p.PS;
      pos = slot - page * p.PS;
    }
  }
  const int side = bid >= p.KVH * NB;
  const int hb = side ? bid - p.KVH * NB : bid;
  const int h = hb / NB, blk = hb - h * NB;

  const __nv_bfloat16* src = side ? p.val + t * p.vs0 + h * p.vs1 : p.key + t * p.ks0 + h * p.ks1;
  const uint4 w0 = *reinterpret_cast<const uint4*>(src + blk * 16);
  const uint4 w1 = *reinterpret_cast<const uint4*>(src + blk * 16 + 8);
  const uint32_t ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float x[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = __uint_as_float(ws[i] << 16);
    x[2 * i + 1] = __uint_as_float(ws[i] & 0xffff0000u);
  }
  // sign bit of every code from "x < 0" (false for -0.0 and NaN, as in the reference). Without the rotation the test
  // runs on the bf16 pairs as they were loaded: a packed compare gives 0xffff / 0 per value, byte permutes bring the
  // eight masks of a code word side by side, and two logic operations drop them onto bit 3 of every nibble.
  uint32_t sg[2] = {0u, 0u};
  if (!HAD) {
    uint32_t m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      m[i] = __hlt2_mask(*reinterpret_cast<const __nv_bfloat162*>(&ws[i]), __floats2bfloat162_rn(0.0f, 0.0f));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t a = __byte_perm(m[4 * h], m[4 * h + 1], 0x6420);
      const uint32_t b = __byte_perm(m[4 * h + 2], m[4 * h + 3], 0x6420);
      // a = masks of values 0, 1, 2, 3 of the word (one byte each), b = those of values 4 .. 7
      const uint32_t even = __byte_perm(a, b, 0x6420), odd = __byte_perm(a, b, 0x7531);
      sg[h] = ((even & 0x08080808u) | (odd & 0x80808080u));
    }
  }
  if (HAD) {
    // every lane of the warp runs the exchange (value rows too, whose results are dropped)
    float y[16];
    const float4* flips = reinterpret_cast<const float4*>(p.signs + blk * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 s4 = __ldg(flips + i);
      y[4 * i] = __fmul_rn(x[4 * i], s4.x);
      y[4 * i + 1] = __fmul_rn(x[4 * i + 1], s4.y);
      y[4 * i + 2] = __fmul_rn(x[4 * i + 2], s4.z);
      y[4 * i + 3] = __fmul_rn(x[4 * i + 3], s4.w);
    }
#pragma unroll
    for (int hh = 1; hh < 16; hh *= 2)
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if ((i & hh) == 0) {
          const float a = y[i], b = y[i + hh];
          y[i] = __fadd_rn(a, b);
          y[i + hh] = __fsub_rn(a, b);
        }
#pragma unroll
    for (int m = 1; m < NB; m *= 2) {                // stage h = 16 m: partner block = blk ^ m
      const bool upper = (blk & m) != 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float o = __shfl_xor_sync(0xffffffffu, y[i], m);
        y[i] = upper ? __fsub_rn(o, y[i]) : __fadd_rn(y[i], o);
      }
    }
    if (side == 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = __fmul_rn(y[i], p.rot_scale);
    }
  }
  f32x2 AX[8];                                    // (|x[2j]|, |x[2j + 1]|)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a0 = fabsf(x[2 * i]), a1 = fabsf(x[2 * i + 1]);
    AX[i] = pk(a0, a1);
    amax = fmaxf(amax, fmaxf(a0, a1));
  }
  const float g = side ? p.gv[h] : p.gk[h];
  if (K8 && side == 0) {
    if (!active) return;
    uint32_t wq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x[4 * i], g), __fdiv_rn(x[4 * i + 1], g)),
                                                   __NV_SATFINITE, __NV_E4M3);
      const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x[4 * i + 2], g), __fdiv_rn(x[4 * i + 3], g)),
                                                   __NV_SATFINITE, __NV_E4M3);
      wq[i] = lo | (hi << 16);
    }
    *reinterpret_cast<uint4*>(p.kd + page * p.dsp + pos * p.dst + h * p.dsh + blk * 16) =
        make_uint4(wq[0], wq[1], wq[2], wq[3]);
    return;
  }
  const int c0 = (int)e4m3_enc(__fdiv_rn(amax, __fmul_rn(g, 6.0f)));
  int cb = c0;
  BlockCodes best;
  if (!SEARCH) {
    float unused;
    score(AX, amax, __fmul_rn(e4m3_dec((unsigned)c0), g), best, unused, false);
  } else {
    const int c3 = (int)e4m3_enc(__fdiv_rn(amax, __fmul_rn(g, 4.0f)));
    if (LPB == 1) {
      // candidates in the reference's order: c0, c0 + 1, c0 - 1, c3; a later one wins only on a strict "<"
      const int cm = max(c0 - 1, 0), cp = min(c0 + 1, 126);
      // the four scales at once: the hardware decodes the four E4M3 codes (exactly: every E4M3 value is an f16 value),
      // two packed multiplies by the global scale round like the reference's single multiplies
      uint32_t d01, d23;
      e4m3x4_to_f16x2((uint32_t)c0 | ((uint32_t)cp << 8) | ((uint32_t)cm << 16) | ((uint32_t)c3 << 24), d01, d23);
      const f32x2 g2 = pk(g, g);
      const f32x2 s01 = mul2(pk(__low2float(u32_as_h2(d01)), __high2float(u32_as_h2(d01))), g2),
                  s23 = mul2(pk(__low2float(u32_as_h2(d23)), __high2float(u32_as_h2(d23))), g2);
      // one decision for the four: the smallest scale is that of c0 - 1, the largest that of c0 + 1 or c3
      float best_err = 0.0f;
      // (an encoder fed NaN, 0 / 0 with a zero global scale, returns code 127, which only the other path decodes)
      if (max(c0, c3) < 127 && div_ok(lo(s23), amax) && fmaxf(hi(s01), hi(s23)) <= 0x1p+96f) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int cc = k == 0 ? c0 : k == 1 ? cp : k == 2 ? cm : c3;
          const float sc = k == 0 ? lo(s01) : k == 1 ? hi(s01) : k == 2 ? lo(s23) : hi(s23);
          float err;
          const BlockCodes c = block_codes_fast<true>(AX, sc, __frcp_rn(sc), err);
          if (k == 0 || err < best_err) {
            best_err = err;
            best = c;
            cb = cc;
          }
        }
      } else {                                      // rare: a zero or extreme scale among the four
#pragma unroll 1
        for (int k = 0; k < 4; ++k) {
          const int cc = k == 0 ? c0 : k == 1 ? cp : k == 2 ? cm : c3;
          const float sc = __fmul_rn(e4m3_dec((unsigned)cc), g);
          const BlockCodes c = block_codes_exact(AX, sc);
          const float err = codes_sse(AX, c, sc);
          if (k == 0 || err < best_err) {
            best_err = err;
            best = c;
            cb = cc;
          }
        }
      }
    } else {
      const int cc = cand == 0 ? c0 : cand == 1 ? min(c0 + 1, 126) : cand == 2 ? max(c0 - 1, 0) : c3;
      BlockCodes c;
      float err;
      score(AX, amax, __fmul_rn(e4m3_dec((unsigned)cc), g), c, err, true);
      const int lane0 = (threadIdx.x & 31) & ~3;
      float best_err = __shfl_sync(0xffffffffu, err, lane0);
      int win = 0;
      cb = __shfl_sync(0xffffffffu, cc, lane0);
#pragma unroll
      for (int k = 1; k < 4; ++k) {
        const float ek = __shfl_sync(0xffffffffu, err, lane0 + k);
        const int ck = __shfl_sync(0xffffffffu, cc, lane0 + k);
        if (ek < best_err) {
          best_err = ek;
          cb = ck;
          win = k;
        }
      }
      best.w[0] = __shfl_sync(0xffffffffu, c.w[0], lane0 + win);
      best.w[1] = __shfl_sync(0xffffffffu, c.w[1], lane0 + win);
    }
  }
  if (!active) return;
  if (HAD) {
#pragma unroll
    for (int i = 0; i < 16; ++i) sg[i >> 3] |= x[i] < 0.0f ? (8u << (4 * (i & 7))) : 0u;
  }
  const uint32_t lo = best.w[0] | sg[0], hi = best.w[1] | sg[1];
  uint8_t* dd = (side ? p.vd : p.kd) + page * p.dsp + pos * p.dst + h * p.dsh + blk * 8;
  if (LPB == 1) {
    *reinterpret_cast<uint2*>(dd) = make_uint2(lo, hi);
  } else {
    const uint32_t wsel = cand < 2 ? lo : hi;
    *reinterpret_cast<uint16_t*>(dd + 2 * cand) = (uint16_t)(cand & 1 ? wsel >> 16 : wsel);
  }
  if (cand == 0) (side ? p.vsf : p.ksf)[page * p.ssp + pos * p.sst + h * p.ssh + blk] = (uint8_t)cb;
}

// ---- self-test of the conversions the write and decode kernels rely on (see hkv_selftest_codec in include/hkv.h)
// counts[0]: non-negative non-NaN fp32 bit patterns (0 .. +inf) whose hardware E2M1 code differs from the threshold
// chain e2m1_mag; counts[1]: the same among the NaN patterns above +inf.
__global__ void selftest_e2m1_encode_kernel(unsigned long long* counts) {
  unsigned long long bad = 0, bad_nan = 0;
  const unsigned long long step = 2ull * gridDim.x * blockDim.x;
  for (unsigned long long b = 2ull * (blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x); b < (1ull << 31);
       b += step) {
    const float y0 = __uint_as_float((unsigned)b), y1 = __uint_as_float((unsigned)b + 1u);
    const uint32_t w = e2m1_codes8(y0, y1, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f);
    const unsigned m0 = (w & 15u) != e2m1_mag(y0), m1 = ((w >> 4) & 15u) != e2m1_mag(y1);
    if (b <= 0x7f800000ull) bad += m0; else bad_nan += m0;
    if (b + 1 <= 0x7f800000ull) bad += m1; else bad_nan += m1;
  }
  if (bad) atomicAdd(counts, bad);
  if (bad_nan) atomicAdd(counts + 1, bad_nan);
}
// counts[2]: (value, scale) pairs inside div_ok's range whose quotient by three multiply-adds (div2) differs from the
// division instruction's: in any bit where the quotient is at least 0.125, in the E2M1 code everywhere. counts[3]: the
// pairs compared. Scales: RN(e4m3 value * g) for the codes 1..126 and 64 global scales g = blockIdx.y (few mantissa
// bits, hashed full mantissas, n / 2688, mantissas of all ones). Values per scale (index blockIdx.x * blockDim.x +
// threadIdx.x = 0 .. 8191): the bf16 patterns of the 17 binades around the scale, RN(u * s) for hashed u in [0, 8), and the seven
// rounding boundaries times s with their neighbours.
__global__ void selftest_quotient_kernel(unsigned long long* counts) {
  const unsigned gi = blockIdx.y, vi = blockIdx.x * blockDim.x + threadIdx.x;
  float g;
  if (gi < 16) g = __uint_as_float(((119u + gi) << 23) | ((gi & 7u) << 20));
  else if (gi < 32) g = __uint_as_float(((100u + 3u * (gi - 16u)) << 23) | ((gi * 2654435761u) >> 9));
  else if (gi < 48) g = __fdiv_rn((float)((gi - 32u) * 37u + 1u), 2688.0f);
  else g = __uint_as_float(((120u + (gi - 48u)) << 23) | (0x7fffffu - (gi & 3u)));
  unsigned long long bad = 0, n = 0;
  for (unsigned c = 1; c < 127; ++c) {
    const float s = __fmul_rn(e4m3_dec(c), g);
    float a;
    if (vi < 17u * 128u) {
      const int e = (int)((__float_as_uint(s) >> 23) & 255u) - 8 + (int)(vi >> 7);
      a = e < 1 || e > 254 ? 0.0f : __uint_as_float(((unsigned)e << 23) | ((vi & 127u) << 16));
    } else if (vi < 8192u - 32u) {
      const unsigned hsh = (vi * 2246822519u) ^ (c * 3266489917u) ^ (gi * 668265263u);
      a = __fmul_rn(__fmul_rn((float)(hsh >> 8), 4.76837158203125e-07f), s);     // u = hash / 2^21 in [0, 8)
    } else {
      const unsigned k = vi - (8192u - 32u);                                    // 7 boundaries x {-1, 0, +1, +2} ulp
      const float tb[8] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f, 6.0f};
      a = __uint_as_float(__float_as_uint(__fmul_rn(tb[k >> 2], s)) + (k & 3u) - 1u);
    }
    if (!div_ok(s, a)) continue;
    const float r = __frcp_rn(s);
    const f32x2 q2 = div2(pk(a, a), pk(r, r), pk(-s, -s));
    const float q = lo(q2), ref = __fdiv_rn(a, s);
    ++n;
    bad += (e2m1_mag(q) != e2m1_mag(ref)) || (ref >= 0.125f && __float_as_uint(q) != __float_as_uint(ref)) ||
           __float_as_uint(hi(q2)) != __float_as_uint(q);
  }
  if (bad) atomicAdd(counts + 2, bad);
  atomicAdd(counts + 3, n);
}
// counts[4]: blocks of 16 values whose codes or whose squared error from the packed-pair path (block_codes_fast<true>)
// differ in any bit from IEEE divisions, the threshold chain and the reference's chain of single fp32 operations
// (multiply, subtract, multiply, add in index order); counts[5]: the blocks compared. One block per thread: hashed
// bf16 magnitudes below 8, the scale an E4M3 code times a hashed global scale, so that all codes occur.
__global__ void selftest_block_error_kernel(unsigned long long* counts) {
  const unsigned id = blockIdx.x * blockDim.x + threadIdx.x;
  float ax[16], amax = 0.0f;
  f32x2 AX[8];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const unsigned hsh = (id * 16u + i) * 2654435761u + 0x9e3779b9u;
    ax[i] = __uint_as_float(((120u + (hsh >> 24) % 10u) << 23) | ((hsh >> 8) & 0x7f0000u));   // bf16, [2^-7, 8)
    if ((hsh & 31u) == 0u) ax[i] = 0.0f;
    amax = fmaxf(amax, ax[i]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) AX[j] = pk(ax[2 * j], ax[2 * j + 1]);
  const float g = __uint_as_float(0x3a000000u | ((id * 40503u) & 0x7fffffu) | (((id >> 9) & 3u) << 23));
  const float s = __fmul_rn(e4m3_dec(96u + (id % 31u)), g);               // E4M3 values 16 .. 448 times g around 10^-3
  unsigned long long bad = 0, n = 0;
  if (div_ok(s, amax)) {
    float err;
    const BlockCodes c = block_codes_fast<true>(AX, s, __frcp_rn(s), err);
    uint32_t w[2] = {0u, 0u};
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const unsigned k = e2m1_mag(__fdiv_rn(ax[i], s));
      w[i >> 3] |= k << (4 * (i & 7));
      const float val = k < 2u ? 0.5f * (float)k : __uint_as_float(0x3f000000u + (k << 22));
      const float d = __fsub_rn(__fmul_rn(val, s), ax[i]);
      const float q = __fmul_rn(d, d);
      acc = i == 0 ? q : __fadd_rn(acc, q);
    }
    n = 1;
    bad = c.w[0] != w[0] || c.w[1] != w[1] || __float_as_uint(err) != __float_as_uint(acc);
  }
  if (bad) atomicAdd(counts + 4, bad);
  if (n) atomicAdd(counts + 5, n);
}
// table[code * 256 + scale byte] = f16 bits of cvt.rn.f16x2.e2m1x2(code) * cvt.rn.f16x2.e4m3x2(scale byte), the product
// the decode and dequantisation kernels form (16 codes x 256 scale bytes)
__global__ void selftest_decode_table_kernel(uint16_t* table) {
  const unsigned code = blockIdx.x, sb = threadIdx.x;
  uint32_t v[4];
  e2m1x8_to_f16x2(code, v);                        // the code in the low nibble of byte 0: value in the low half of v[0]
  const uint32_t prod = hmul2(v[0], e4m3x2_to_f16x2(sb));
  table[code * 256 + sb] = (uint16_t)(prod & 0xffffu);
}

static std::atomic<int> g_last_cuda_error{0};

}  // namespace hkv

extern "C" int hkv_last_cuda_error(void) { return hkv::g_last_cuda_error.load(std::memory_order_relaxed); }

extern "C" int hkv_version(void) { return 100; }

extern "C" const char* hkv_error_string(int code) {
  switch (code) {
    case HKV_OK: return "ok";
    case HKV_ERR_NULL: return "a required pointer is null";
    case HKV_ERR_ALIGN: return "a pointer or stride misses the required alignment";
    case HKV_ERR_UNSUPPORTED: return "unsupported head_dim, group size, page size or layout";
    case HKV_ERR_SPLITS: return "more than 64 splits";
    case HKV_ERR_WORKSPACE: return "workspace too small";
    case HKV_ERR_RANGE: return "a size is negative or too large";
    case HKV_ERR_CUDA: return "a CUDA runtime call failed";
    case HKV_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel ran out";
    case HKV_ERR_NOALLOC_LIMIT:
      return "the call needs more scratch than the built-in 5 MiB of hkv_decode_noalloc: pass a smaller `splits` or use "
             "hkv_decode with a workspace";
    default: return "unknown error code";
  }
}

extern "C" int hkv_selftest_codec(void* out, size_t out_bytes, void* stream) {
  using namespace hkv;
  if (!out) return HKV_ERR_NULL;
  if ((uintptr_t)out & 7) return HKV_ERR_ALIGN;
  if (out_bytes < HKV_SELFTEST_CODEC_BYTES) return HKV_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(out, 0, 64, st);
  if (e != cudaSuccess) return record_cuda(e);
  selftest_e2m1_encode_kernel<<<148 * 8, 256, 0, st>>>((unsigned long long*)out);
  if ((e = cudaGetLastError()) != cudaSuccess) return record_cuda(e);
  selftest_quotient_kernel<<<dim3(32, 64), 256, 0, st>>>((unsigned long long*)out);
  if ((e = cudaGetLastError()) != cudaSuccess) return record_cuda(e);
  selftest_block_error_kernel<<<8192, 256, 0, st>>>((unsigned long long*)out);
  if ((e = cudaGetLastError()) != cudaSuccess) return record_cuda(e);
  selftest_decode_table_kernel<<<16, 256, 0, st>>>((uint16_t*)((uint8_t*)out + 64));
  return record_cuda(cudaGetLastError());
}

namespace hkv {
int record_cuda(cudaError_t e) {
  if (e == cudaSuccess) return HKV_OK;
  g_last_cuda_error.store((int)e, std::memory_order_relaxed);
  return HKV_ERR_CUDA;
}
}  // namespace hkv

static int write_impl(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1, void* kd,
                      void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS, const int64_t* slots,
                      int64_t n_slots, const float* gk, const float* gv, int KVH, int D, int search,
                      const float* signs, int k8, void* stream) {
  using namespace hkv;
  if (k8 && D != 256) return HKV_ERR_UNSUPPORTED;      // the K8V4 slot exists at head_dim 256 only, like the reference's
  if (k8 && strides && (((uintptr_t)kd | (uintptr_t)strides[0] | (uintptr_t)strides[1] | (uintptr_t)strides[2]) & 15))
    return HKV_ERR_ALIGN;                              // 16-byte key stores
  if (n_slots < 0) return HKV_ERR_RANGE;
  if (n_slots == 0) return HKV_OK;
  if (!key || !val || !kd || !ksf || !vd || !vsf || !strides || !slots || !gk || !gv) return HKV_ERR_NULL;
  if (D != 128 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (KVH < 1 || KVH > 1024 || PS < 1) return HKV_ERR_UNSUPPORTED;
  // 16-byte row loads of bf16 and 8-byte code stores
  if (((uintptr_t)key | (uintptr_t)val) & 15) return HKV_ERR_ALIGN;
  if ((ks0 | ks1 | vs0 | vs1) & 7) return HKV_ERR_ALIGN;
  if (((uintptr_t)kd | (uintptr_t)vd) & 7) return HKV_ERR_ALIGN;
  if ((strides[0] | strides[1] | strides[2]) & 7) return HKV_ERR_ALIGN;
  WriteParams p;
  p.key = (const __nv_bfloat16*)key;
  p.val = (const __nv_bfloat16*)val;
  p.ks0 = ks0; p.ks1 = ks1; p.vs0 = vs0; p.vs1 = vs1;
  p.kd = (uint8_t*)kd; p.ksf = (uint8_t*)ksf; p.vd = (uint8_t*)vd; p.vsf = (uint8_t*)vsf;
  p.dsp = strides[0]; p.dst = strides[1]; p.dsh = strides[2];
  p.ssp = strides[3]; p.sst = strides[4]; p.ssh = strides[5];
  p.slots = (const long long*)slots;
  p.n_slots = n_slots;
  p.gk = gk; p.gv = gv; p.PS = PS; p.KVH = KVH;
  p.signs = signs;
  p.rot_scale = (float)(1.0 / sqrt((double)D));
  if (signs && ((uintptr_t)signs & 15)) return HKV_ERR_ALIGN;
  // lanes: one per (token, block) for prefill-sized launches and whenever the keys are rotated, a quad per
  // (token, block) for few tokens (decode appends)
  const int lpb = (n_slots <= 4096 && !signs && !k8) ? 4 : 1;
  const int threads = 256;
  const long long lanes = n_slots * (2ll * KVH * (D / 16)) * lpb;
  {
    // round-up magic number of the division by d = blocks per token (Granlund and Montgomery): l = ceil(log2 d),
    // m = floor(2^32 (2^l - d) / d) + 1, n / d = (umulhi(m, n) + n) >> l for every n < 2^31 (the sum cannot overflow)
    const unsigned long long d = 2ull * KVH * (D / 16);
    int l = 0;
    while ((1ull << l) < d) ++l;
    p.div_magic = (unsigned)((((1ull << l) - d) << 32) / d + 1ull);
    p.div_shift = lanes + threads < (1ll << 31) ? l : -1;
  }
  const long long blocks = (lanes + threads - 1) / threads;
  if (blocks > 0x7fffffffll) return HKV_ERR_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  void (*k)(const WriteParams);
  if (k8) {
    k = search ? write_kernel<256, 1, 1, 0, 1> : write_kernel<256, 0, 1, 0, 1>;
  } else if (signs) {
    k = D == 128 ? (search ? write_kernel<128, 1, 1, 1> : write_kernel<128, 0, 1, 1>)
                 : (search ? write_kernel<256, 1, 1, 1> : write_kernel<256, 0, 1, 1>);
  } else if (D == 128) {
    k = lpb == 1 ? (search ? write_kernel<128, 1, 1, 0> : write_kernel<128, 0, 1, 0>)
                 : (search ? write_kernel<128, 1, 4, 0> : write_kernel<128, 0, 4, 0>);
  } else {
    k = lpb == 1 ? (search ? write_kernel<256, 1, 1, 0> : write_kernel<256, 0, 1, 0>)
                 : (search ? write_kernel<256, 1, 4, 0> : write_kernel<256, 0, 4, 0>);
  }
  return record_cuda(launch_pdl(k, dim3((unsigned)blocks), dim3(threads), 0, st, p));
}

extern "C" int hkv_write(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1,
                         void* kd, void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS,
                         const int64_t* slots, int64_t n_slots, const float* gk, const float* gv, int KVH, int D,
                         int search, void* stream) {
  return write_impl(key, val, ks0, ks1, vs0, vs1, kd, ksf, vd, vsf, strides, PS, slots, n_slots, gk, gv, KVH, D,
                    search, nullptr, 0, stream);
}

extern "C" int hkv_write_rot(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1,
                             void* kd, void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS,
                             const int64_t* slots, int64_t n_slots, const float* gk, const float* gv, int KVH, int D,
                             int search, const float* signs, void* stream) {
  if (!signs) return HKV_ERR_NULL;
  return write_impl(key, val, ks0, ks1, vs0, vs1, kd, ksf, vd, vsf, strides, PS, slots, n_slots, gk, gv, KVH, D,
                    search, signs, 0, stream);
}

extern "C" int hkv_write_k8(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1,
                            void* kd, void* vd, void* vsf, const int64_t strides[6], int PS, const int64_t* slots,
                            int64_t n_slots, const float* gk, const float* gv, int KVH, int D, int search,
                            void* stream) {
  return write_impl(key, val, ks0, ks1, vs0, vs1, kd, kd, vd, vsf, strides, PS, slots, n_slots, gk, gv, KVH, D, search,
                    nullptr, 1, stream);
}
