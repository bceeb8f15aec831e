// Quantize-on-write for the NVFP4 paged KV cache (sm_100a).
//
// Four threads own one block of 16 consecutive channels of one (token, kv head, side): they read its 32 bytes of
// bf16, pick the E4M3 block scale (optionally by the 4-candidate squared-error search, one candidate per thread),
// encode the 16 E2M1 codes and store 8 code bytes + 1 scale byte at slot = page * PS + position. Consecutive quads cover
// consecutive blocks, so a warp reads 256 contiguous bytes and stores 64 contiguous code bytes.
//
// Bit-exactness: the result must equal the reference's PyTorch quantiser (kv_fp4_ref.py:159-186 `quantize_rows`,
// rules at kv_fp4_ref.py:15-25) byte for byte. Every arithmetic step is therefore a single IEEE fp32 operation issued
// through an explicit intrinsic (__fdiv_rn, __fmul_rn, __fsub_rn, __fadd_rn): no contraction into FMA, no fast-math.
// The squared error is summed sequentially over i = 0..15 and a later candidate wins only on a strict "<".
#include <cuda_bf16.h>

#include <algorithm>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "hkv_common.cuh"

namespace hkv {

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
__device__ __forceinline__ float e2m1_val(unsigned m) {
  const unsigned e = (m >> 1) & 3u, l = m & 1u;
  return e ? __uint_as_float(((e + 126u) << 23) | (l << 22)) : (l ? 0.5f : 0.0f);
}
__device__ __forceinline__ unsigned mag_of(float ax, float s) { return s > 0.0f ? e2m1_mag(__fdiv_rn(ax, s)) : 0u; }

// sequential squared error of the block under effective scale s (kv_fp4_ref.py:148-156)
__device__ __forceinline__ float block_sse(const float (&ax)[16], float s) {
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float d = __fsub_rn(__fmul_rn(e2m1_val(mag_of(ax[i], s)), s), ax[i]);
    const float sq = __fmul_rn(d, d);
    acc = i == 0 ? sq : __fadd_rn(acc, sq);
  }
  return acc;
}

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
__device__ __forceinline__ unsigned e2m1_pair(float hi, float lo) {      // code(hi) in bits 7:4, code(lo) in bits 3:0
  unsigned short r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float e2m1_pair_value(unsigned b) {           // value of the code in bits 3:0
  unsigned h2;
  asm("{ .reg .b8 t, z; mov.b16 {t, z}, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "h"((unsigned short)b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
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
// magnitude code of RN(ax / s) from the bracket (ax * r_up, ax * r_down)
__device__ __forceinline__ unsigned fast_code(float ax, float s, float r_up, float r_down) {
  const unsigned b = e2m1_pair(ax * r_up, ax * r_down);
  unsigned k = b & 7u;
  if (((b >> 4) ^ b) & 7u) k = resolve_code(ax, s, k);
  return k;
}

// squared error of the block under scale s with bracketing reciprocals r_up, r_down
__device__ __forceinline__ float block_sse_fast(const float (&ax)[16], float s, float r_up, float r_down) {
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float d = __fsub_rn(__fmul_rn(e2m1_pair_value(fast_code(ax[i], s, r_up, r_down)), s), ax[i]);
    const float sq = __fmul_rn(d, d);
    acc = i == 0 ? sq : __fadd_rn(acc, sq);
  }
  return acc;
}

// Four lanes share one block of 16 values: every lane reads the whole block (the four identical 16-byte requests of
// a quad are served by one access), lane k of the quad scores scale candidate k, the quad agrees on the winner with
// shuffles in candidate order (strict "<", so the earliest candidate wins a tie, as in the reference), and every lane
// encodes 4 of the 16 values. One CTA handles one token: 2 * KVH * D / 16 blocks spread over its quads.
template <int D, int SEARCH>
__global__ void __launch_bounds__(1024) write_kernel(const WriteParams p) {
  constexpr int NB = D / 16;                      // blocks per row
  pdl_wait();                                     // inputs and the cache may come from the preceding launch
  pdl_launch_dependents();
  // one CTA per token; its 2 * KVH * NB blocks are spread over the CTA's quads (all index math in 32 bits)
  const long long t = blockIdx.x;
  const long long slot = p.slots[t];
  if (slot < 0) return;                           // uniform per CTA
  long long page, pos;
  if ((p.PS & (p.PS - 1)) == 0) {
    const int sh = 31 - __clz(p.PS);
    page = slot >> sh;
    pos = slot & (p.PS - 1);
  } else {
    page = slot / p.PS;
    pos = slot - page * p.PS;
  }
  const int cand = threadIdx.x & 3;
  const int n_blocks = 2 * p.KVH * NB;
  for (int bid = threadIdx.x >> 2; bid < n_blocks; bid += blockDim.x >> 2) {   // n_blocks is a multiple of 16
  const int side = bid >= p.KVH * NB;
  const int hb = side ? bid - p.KVH * NB : bid;
  const int h = hb / NB, blk = hb - h * NB;

  const __nv_bfloat16* src = side ? p.val + t * p.vs0 + h * p.vs1 : p.key + t * p.ks0 + h * p.ks1;
  const uint4 w0 = *reinterpret_cast<const uint4*>(src + blk * 16);
  const uint4 w1 = *reinterpret_cast<const uint4*>(src + blk * 16 + 8);
  const uint32_t ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float ax[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ax[2 * i] = fabsf(__uint_as_float(ws[i] << 16));
    ax[2 * i + 1] = fabsf(__uint_as_float(ws[i] & 0xffff0000u));
    amax = fmaxf(amax, fmaxf(ax[2 * i], ax[2 * i + 1]));
  }
  const float g = side ? p.gv[h] : p.gk[h];
  const int c0 = (int)e4m3_enc(__fdiv_rn(amax, __fmul_rn(g, 6.0f)));
  int cb = c0;
  if (SEARCH) {
    const int cc = cand == 0 ? c0 : cand == 1 ? min(c0 + 1, 126) : cand == 2 ? max(c0 - 1, 0)
                 : (int)e4m3_enc(__fdiv_rn(amax, __fmul_rn(g, 4.0f)));
    const float sc = __fmul_rn(e4m3_dec((unsigned)cc), g);
    float err;
    if (fast_scale_ok(sc)) {
      const float r = __frcp_rn(sc);
      err = block_sse_fast(ax, sc, r * kUp, r * kDown);
    } else {
      err = block_sse(ax, sc);                        // rare: a zero or extreme scale
    }
    const int lane0 = (threadIdx.x & 31) & ~3;
    float best = __shfl_sync(0xffffffffu, err, lane0);
    cb = __shfl_sync(0xffffffffu, cc, lane0);
#pragma unroll
    for (int k = 1; k < 4; ++k) {
      const float ek = __shfl_sync(0xffffffffu, err, lane0 + k);
      const int ck = __shfl_sync(0xffffffffu, cc, lane0 + k);
      if (ek < best) {
        best = ek;
        cb = ck;
      }
    }
  }
  const float s = __fmul_rn(e4m3_dec((unsigned)cb), g);
  // this lane's 4 values: elements 4 cand .. 4 cand + 3 (two bf16 pairs), sign from "x < 0" (false for -0.0)
  const uint32_t wa = cand == 0 ? ws[0] : cand == 1 ? ws[2] : cand == 2 ? ws[4] : ws[6];
  const uint32_t wb = cand == 0 ? ws[1] : cand == 1 ? ws[3] : cand == 2 ? ws[5] : ws[7];
  const float x0 = __uint_as_float(wa << 16), x1 = __uint_as_float(wa & 0xffff0000u);
  const float x2 = __uint_as_float(wb << 16), x3 = __uint_as_float(wb & 0xffff0000u);
  unsigned m0, m1, m2, m3;
  if (fast_scale_ok(s)) {
    const float r = __frcp_rn(s), r_up = r * kUp, r_down = r * kDown;
    m0 = fast_code(fabsf(x0), s, r_up, r_down);
    m1 = fast_code(fabsf(x1), s, r_up, r_down);
    m2 = fast_code(fabsf(x2), s, r_up, r_down);
    m3 = fast_code(fabsf(x3), s, r_up, r_down);
  } else {
    m0 = mag_of(fabsf(x0), s); m1 = mag_of(fabsf(x1), s); m2 = mag_of(fabsf(x2), s); m3 = mag_of(fabsf(x3), s);
  }
  const uint32_t code = (m0 | (x0 < 0.0f ? 8u : 0u)) | ((m1 | (x1 < 0.0f ? 8u : 0u)) << 4) |
                        ((m2 | (x2 < 0.0f ? 8u : 0u)) << 8) | ((m3 | (x3 < 0.0f ? 8u : 0u)) << 12);
  uint8_t* dd = (side ? p.vd : p.kd) + page * p.dsp + pos * p.dst + h * p.dsh + blk * 8 + 2 * cand;
  *reinterpret_cast<uint16_t*>(dd) = (uint16_t)code;
  if (cand == 0) (side ? p.vsf : p.ksf)[page * p.ssp + pos * p.sst + h * p.ssh + blk] = (uint8_t)cb;
  }
}

static int g_last_cuda_error = 0;

}  // namespace hkv

extern "C" int hkv_last_cuda_error(void) { return hkv::g_last_cuda_error; }

extern "C" int hkv_version(void) { return 100; }

extern "C" const char* hkv_error_string(int code) {
  switch (code) {
    case HKV_OK: return "ok";
    case HKV_ERR_NULL: return "a required pointer is null";
    case HKV_ERR_ALIGN: return "a pointer or stride misses the required alignment";
    case HKV_ERR_UNSUPPORTED: return "unsupported head_dim, group size, page size, query length or layout";
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

namespace hkv {
int record_cuda(cudaError_t e) {
  if (e == cudaSuccess) return HKV_OK;
  g_last_cuda_error = (int)e;
  return HKV_ERR_CUDA;
}
}  // namespace hkv

extern "C" int hkv_write(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1,
                         void* kd, void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS,
                         const int64_t* slots, int64_t n_slots, const float* gk, const float* gv, int KVH, int D,
                         int search, void* stream) {
  using namespace hkv;
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
  const long long blocks = n_slots;                 // one CTA per token
  if (blocks > 0x7fffffffll) return HKV_ERR_RANGE;
  cudaStream_t st = (cudaStream_t)stream;
  void (*k)(const WriteParams) = D == 128 ? (search ? write_kernel<128, 1> : write_kernel<128, 0>)
                                          : (search ? write_kernel<256, 1> : write_kernel<256, 0>);
  // few tokens (decode appends): one quad per block so that a token's blocks are quantised side by side; many tokens
  // (prefill): 256 threads per CTA loop over the token's blocks
  int threads = 256;
  if (n_slots <= 4096) threads = std::min(1024, std::max(128, 2 * KVH * (D / 16) * 4));
  return record_cuda(launch_pdl(k, dim3((unsigned)blocks), dim3(threads), 0, st, p));
}
