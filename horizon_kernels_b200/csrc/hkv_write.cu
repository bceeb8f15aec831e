// Quantize-on-write for the NVFP4 paged KV cache (sm_100a).
//
// A block of 16 consecutive channels of one (token, kv head, side) is 32 bytes of bf16 in and 8 code bytes + 1 scale
// byte out, stored at slot = page * PS + position. The E4M3 block scale is picked (optionally) by the reference's
// 4-candidate squared-error search. Large launches give every block to one lane, which scores the candidates in turn;
// small launches (decode appends) give it to a quad, one candidate per lane. The 16 magnitude codes of a candidate
// live in two registers (a nibble each), produced eight at a time by the hardware E2M1 conversion.
//
// Bit-exactness: the result must equal the reference's PyTorch quantiser (kv_fp4_ref.py:159-186 `quantize_rows`,
// rules at kv_fp4_ref.py:15-25) byte for byte. Every arithmetic step is therefore a single IEEE fp32 operation issued
// through an explicit intrinsic (__fdiv_rn, __fmul_rn, __fsub_rn, __fadd_rn): no contraction into FMA, no fast-math.
// The squared error is summed sequentially over i = 0..15 and a later candidate wins only on a strict "<".
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

// ---- division-free fast path -------------------------------------------------------------------------------------
// The reference rounds y = RN(ax / s) onto the E2M1 grid. Here the quotient is bracketed by ax * RN(r * (1 + 2^-20))
// and ax * RN(r * (1 - 2^-20)), r = RN(1 / s) (three roundings of relative error 2^-24 each, far inside the 2^-20
// band), and the hardware conversion cvt.rn.satfinite.e2m1x2.f32 (identical to the reference's threshold chain for
// every non-negative fp32 input) is applied to both at once. The conversion is monotone and RN(ax / s) lies between
// the two arguments, so equal codes prove the code of the exact quotient. Unequal codes k, k + 1 mean the quotient is
// within 2^-20 of the threshold t between them, often exactly on it when the global scale has few mantissa bits. That
// case is decided exactly without a division: every threshold has an even mantissa, so RN(q) <= t holds iff
// q <= t + ulp/2 and RN(q) < t iff q < t - ulp'/2 (ulp' of the binade below), and q <= m is ax <= m * s, a product
// of a 26-bit and a 24-bit significand that fp64 holds exactly. A scale outside [2^-96, 2^96] takes the IEEE-division
// path. The error terms (code * s - ax)^2 are still single IEEE operations in the reference's order.
constexpr float kUp = 1.0f + 9.5367431640625e-07f, kDown = 1.0f - 9.5367431640625e-07f;   // 1 +- 2^-20
__device__ __forceinline__ bool fast_scale_ok(float s) { return s >= 1.2621774e-29f && s <= 7.9228163e28f; }

// rounding boundary of the quotient between E2M1 magnitude codes k and k + 1: t + ulp(t) / 2 for the "<=" thresholds
// 0.25, 1.25, 2.5, 5 (k even), t - ulp(pred t) / 2 for the "<" thresholds 0.75, 1.75, 3.5 (k odd)
__constant__ double kBoundary[8] = {0.25 + 0x1p-26, 0.75 - 0x1p-25, 1.25 + 0x1p-24, 1.75 - 0x1p-24,
                                    2.5 + 0x1p-23,  3.5 - 0x1p-23,  5.0 + 0x1p-22,  0.0};
// exact magnitude code of RN(ax / s) when the bracket gave codes k and k + 1 (rare; never inlined into the hot loop)
static __device__ __noinline__ unsigned resolve_code(float ax, float s, unsigned k) {
  const double lhs = (double)ax, rhs = kBoundary[k & 7u] * (double)s;
  return ((k & 1u) ? lhs < rhs : lhs <= rhs) ? k : k + 1u;
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
__device__ __forceinline__ uint32_t bracket_codes8(const float (&ax)[16], int o, float r) {
  return e2m1_codes8(ax[o] * r, ax[o + 1] * r, ax[o + 2] * r, ax[o + 3] * r, ax[o + 4] * r, ax[o + 5] * r,
                     ax[o + 6] * r, ax[o + 7] * r);
}

// the 16 magnitude codes of a block under scale s: value i in nibble i % 8 of word i / 8
struct BlockCodes {
  uint32_t w[2];
};
__device__ __forceinline__ BlockCodes block_codes_fast(const float (&ax)[16], float s, float r) {
  const float r_up = r * kUp, r_down = r * kDown;
  BlockCodes c;
  uint32_t diff[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    c.w[h] = bracket_codes8(ax, 8 * h, r_down);
    diff[h] = c.w[h] ^ bracket_codes8(ax, 8 * h, r_up);
  }
  if (diff[0] | diff[1]) {                        // rare: some quotient lies within 2^-20 of a rounding boundary
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {                // four values at a time: most groups have no such quotient
      if (((diff[q4 >> 1] >> (16 * (q4 & 1))) & 0xffffu) == 0u) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * q4 + j, sh = 4 * (i & 7);
        if ((diff[i >> 3] >> sh) & 15u) {
          const unsigned k = resolve_code(ax[i], s, (c.w[i >> 3] >> sh) & 7u);
          c.w[i >> 3] = (c.w[i >> 3] & ~(15u << sh)) | (k << sh);
        }
      }
    }
  }
  return c;
}
__device__ __forceinline__ BlockCodes block_codes_exact(const float (&ax)[16], float s) {   // IEEE divisions
  BlockCodes c;
  c.w[0] = c.w[1] = 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i) c.w[i >> 3] |= mag_of(ax[i], s) << (4 * (i & 7));
  return c;
}
// sequential squared error of the block for given codes (kv_fp4_ref.py:148-156): single IEEE operations, i = 0..15
__device__ __forceinline__ float codes_sse(const float (&ax)[16], const BlockCodes& c, float s) {
  float acc = 0.0f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t v[4];                                // f16x2 values of the word's code pairs
    e2m1x8_to_f16x2(c.w[h], v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 hv = u32_as_h2(v[j]);
      const int i = 8 * h + 2 * j;
      const float d0 = __fsub_rn(__fmul_rn(__low2float(hv), s), ax[i]);
      const float q0 = __fmul_rn(d0, d0);
      acc = i == 0 ? q0 : __fadd_rn(acc, q0);
      const float d1 = __fsub_rn(__fmul_rn(__high2float(hv), s), ax[i + 1]);
      acc = __fadd_rn(acc, __fmul_rn(d1, d1));
    }
  }
  return acc;
}
__device__ __forceinline__ void score(const float (&ax)[16], float sc, BlockCodes& c, float& err, bool want_err) {
  if (fast_scale_ok(sc)) c = block_codes_fast(ax, sc, __frcp_rn(sc));
  else c = block_codes_exact(ax, sc);             // rare: a zero or extreme scale
  if (want_err) err = codes_sse(ax, c, sc);
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
  long long t = gid / n_blocks;
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
  float x[16], ax[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = __uint_as_float(ws[i] << 16);
    x[2 * i + 1] = __uint_as_float(ws[i] & 0xffff0000u);
  }
  if (HAD) {
    // every lane of the warp runs the exchange (value rows too, whose results are dropped)
    float y[16];
    const float4* sg = reinterpret_cast<const float4*>(p.signs + blk * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 s4 = __ldg(sg + i);
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
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ax[2 * i] = fabsf(x[2 * i]);
    ax[2 * i + 1] = fabsf(x[2 * i + 1]);
    amax = fmaxf(amax, fmaxf(ax[2 * i], ax[2 * i + 1]));
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
    score(ax, __fmul_rn(e4m3_dec((unsigned)c0), g), best, unused, false);
  } else {
    const int c3 = (int)e4m3_enc(__fdiv_rn(amax, __fmul_rn(g, 4.0f)));
    if (LPB == 1) {
      float best_err = 0.0f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int cc = k == 0 ? c0 : k == 1 ? min(c0 + 1, 126) : k == 2 ? max(c0 - 1, 0) : c3;
        BlockCodes c;
        float err;
        score(ax, __fmul_rn(e4m3_dec((unsigned)cc), g), c, err, true);
        if (k == 0 || err < best_err) {
          best_err = err;
          best = c;
          cb = cc;
        }
      }
    } else {
      const int cc = cand == 0 ? c0 : cand == 1 ? min(c0 + 1, 126) : cand == 2 ? max(c0 - 1, 0) : c3;
      BlockCodes c;
      float err;
      score(ax, __fmul_rn(e4m3_dec((unsigned)cc), g), c, err, true);
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
  // sign bit of every code from "x < 0" (false for -0.0 and NaN, as in the reference)
  uint32_t sg[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 16; ++i) sg[i >> 3] |= x[i] < 0.0f ? (8u << (4 * (i & 7))) : 0u;
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
  cudaError_t e = cudaMemsetAsync(out, 0, 16, st);
  if (e != cudaSuccess) return record_cuda(e);
  selftest_e2m1_encode_kernel<<<148 * 8, 256, 0, st>>>((unsigned long long*)out);
  if ((e = cudaGetLastError()) != cudaSuccess) return record_cuda(e);
  selftest_decode_table_kernel<<<16, 256, 0, st>>>((uint16_t*)((uint8_t*)out + 16));
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
