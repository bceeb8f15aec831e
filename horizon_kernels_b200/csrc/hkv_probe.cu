// Issue-rate probe (no counterpart in the reference): how many SM cycles a sub-partition needs per warp instruction for
// the instruction kinds the decode kernel is made of. The design notes of the decode kernel rest on these figures (on
// B200 the E2M1 conversion, logic ops and f16x2 multiplies issue every second cycle, fp32 fma every cycle; conversions
// and f16x2 multiplies sit on different pipes and overlap; a warp-level mma.m16n8k16 adds little more than a cycle to a
// dequantise group) and so do those of the write kernel (a packed mul.f32x2 takes one issue slot and holds the fp32
// pipe for two cycles; f16 -> f32 conversions, prmt and logic ops take two cycles each), so the probe ships with the
// library and anyone can re-measure them:
//     python -m horizon_kernels_b200.microbench pipes
#include "hkv_common.cuh"

namespace hkv {
int record_cuda(cudaError_t e);

constexpr int kProbeModes = 12;
constexpr int kProbeIter = 256, kProbeRep = 8;       // the body runs kProbeIter * kProbeRep times per warp

__device__ __forceinline__ uint32_t probe_cvt(uint32_t w) {
  uint32_t r;
  asm volatile("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(r) : "r"(w));
  return r;
}
__device__ __forceinline__ uint32_t probe_hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm volatile("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float probe_ffma(float a, float b, float c) {
  float r;
  asm volatile("fma.rn.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint32_t probe_lop(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm volatile("lop3.b32 %0, %1, %2, %3, 0x96;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ float probe_fmul(float a, float b) {
  float r;
  asm volatile("mul.rn.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ unsigned long long probe_fmul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm volatile("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint32_t probe_pack(float a, float b) {         // two fp32 -> one byte of two E2M1 codes
  uint32_t r;
  asm volatile("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tmov.b32 %0, {t, t, t, t};\n\t}" : "=r"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float probe_h2f(uint32_t h) {
  float r;
  asm volatile("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.f32.f16 %0, lo;\n\t}" : "=f"(r) : "r"(h));
  return r;
}
__device__ __forceinline__ uint32_t probe_prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm volatile("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ void probe_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: 8 E2M1 conversions   1: 8 f16x2 multiplies   2: 8 fp32 fma   3: 8 lop3   4: 4 conversions + 4 multiplies
//      5: the dequantise group of the decode kernel without its mma: 4 conversions, 4 multiplies, 1 integer add
//      6: the same group with its mma.m16n8k16 (8 independent accumulators)
//      7: 8 fp32 multiplies   8: 8 packed mul.f32x2   9: 8 E2M1 packs (cvt.rn.satfinite.e2m1x2.f32)
//     10: 8 f16 -> f32 conversions   11: 8 prmt
template <int MODE>
__global__ void probe_kernel(long long* cycles, uint32_t* sink, uint32_t seed) {
  uint32_t x[8];
  float f[8], d[8][4];
  unsigned long long u[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[i] = seed + threadIdx.x * 7u + i * 0x01010101u;
    f[i] = (float)(x[i] & 1023u);
    u[i] = ((unsigned long long)__float_as_uint(f[i] + 1.0f) << 32) | __float_as_uint(f[i] + 2.0f);
    d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.0f;
  }
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < kProbeIter; ++it) {
#pragma unroll
    for (int r = 0; r < kProbeRep; ++r) {
      if (MODE == 0) { for (int i = 0; i < 8; ++i) x[i] = probe_cvt(x[i]); }
      if (MODE == 1) { for (int i = 0; i < 8; ++i) x[i] = probe_hmul2(x[i], 0x3c003c00u); }
      if (MODE == 2) { for (int i = 0; i < 8; ++i) f[i] = probe_ffma(f[i], 1.0001f, 0.5f); }
      if (MODE == 3) { for (int i = 0; i < 8; ++i) x[i] = probe_lop(x[i], 0x55aa55aau, seed); }
      if (MODE == 4) { for (int i = 0; i < 4; ++i) { x[i] = probe_cvt(x[i]); x[i + 4] = probe_hmul2(x[i + 4], 0x3c003c00u); } }
      if (MODE == 7) { for (int i = 0; i < 8; ++i) f[i] = probe_fmul(f[i], 1.0001f); }
      if (MODE == 8) { for (int i = 0; i < 8; ++i) u[i] = probe_fmul2(u[i], 0x3f8003473f800347ull); }
      if (MODE == 9) { for (int i = 0; i < 8; ++i) x[i] = probe_pack(__uint_as_float(x[i]), f[i]); }
      if (MODE == 10) { for (int i = 0; i < 8; ++i) x[i] = __float_as_uint(probe_h2f(x[i])); }
      if (MODE == 11) { for (int i = 0; i < 8; ++i) x[i] = probe_prmt(x[i], seed, 0x2103u); }
      if (MODE == 5 || MODE == 6) {
        const uint32_t o0 = probe_cvt(x[0]), o1 = probe_cvt(x[0] >> 8), o2 = probe_cvt(x[0] >> 16), o3 = probe_cvt(x[0] >> 24);
        const uint32_t a0 = probe_hmul2(o0, x[1]), a1 = probe_hmul2(o1, x[1]), a2 = probe_hmul2(o2, x[1]), a3 = probe_hmul2(o3, x[1]);
        if (MODE == 6) probe_mma(d[r & 7], a0, a1, a2, a3, x[2], x[3]);
        else x[4 + (r & 3)] ^= a0 ^ a1 ^ a2 ^ a3;
        x[0] += 0x11u;
      }
    }
  }
  const long long t1 = clock64();
  uint32_t acc = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc ^= x[i] ^ (uint32_t)u[i] ^ (uint32_t)(u[i] >> 32) ^ __float_as_uint(f[i]) ^ __float_as_uint(d[i][0] + d[i][1] + d[i][2] + d[i][3]);
  sink[blockIdx.x * blockDim.x + threadIdx.x] = acc;
  if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
}

}  // namespace hkv

extern "C" int hkv_probe_issue_rates(void* scratch, size_t scratch_bytes, int warps_per_subpartition, void* stream) {
  using namespace hkv;
  if (!scratch) return HKV_ERR_NULL;
  if ((uintptr_t)scratch & 7) return HKV_ERR_ALIGN;
  if (warps_per_subpartition < 1 || warps_per_subpartition > 8) return HKV_ERR_RANGE;
  if (scratch_bytes < HKV_PROBE_SCRATCH_BYTES) return HKV_ERR_WORKSPACE;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda(e);
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return record_cuda(e);
  if (sms > 256) sms = 256;
  cudaStream_t st = (cudaStream_t)stream;
  long long* cyc = (long long*)scratch;                       // [kProbeModes][256] cycle counts, one per SM
  uint32_t* sink = (uint32_t*)((uint8_t*)scratch + kProbeModes * 256 * 8);
  if ((e = cudaMemsetAsync(scratch, 0, kProbeModes * 256 * 8, st)) != cudaSuccess) return record_cuda(e);
  const int threads = 128 * warps_per_subpartition;           // one block per SM, its warps spread over the 4 sub-partitions
  void (*ks[kProbeModes])(long long*, uint32_t*, uint32_t) = {probe_kernel<0>, probe_kernel<1>, probe_kernel<2>, probe_kernel<3>,
                                                               probe_kernel<4>, probe_kernel<5>, probe_kernel<6>, probe_kernel<7>,
                                                               probe_kernel<8>, probe_kernel<9>, probe_kernel<10>, probe_kernel<11>};
  for (int m = 0; m < kProbeModes; ++m)
    for (int rep = 0; rep < 2; ++rep) {                       // the second run overwrites the first (warm instruction cache)
      ks[m]<<<sms, threads, 0, st>>>(cyc + m * 256, sink, 12345u);
      if ((e = cudaGetLastError()) != cudaSuccess) return record_cuda(e);
    }
  return HKV_OK;
}
