// Shared device helpers for the hkv kernels (sm_100a): error codes, workspace header, mbarrier / bulk-copy / mma /
// narrow-float conversion wrappers. Everything here is inline PTX or plain CUDA; no library calls.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hkv.h"

namespace hkv {

// ---------------------------------------------------------------------------------------------------- workspace
// Layout of the decode workspace (all offsets from the 256-byte aligned base):
//   Header | tickets[kMaxParts] int | lse[n_parts][2][RPAD] fp32 | opart[n_parts][2][RPAD][D] fp32
// Each decode partition (one CTA) owns two partial slots: slot 0 for a sequence piece that begins the partition,
// slot 1 for a piece that ends it while the sequence continues in the next partition. tickets[p] counts the finished
// pieces of the split sequence that ENDS in partition p; the CTA that brings it to the number of pieces merges them
// and sets it back to zero, so the counters are zero between launches (the workspace starts zero-filled). The ticket
// table has a fixed size and place, so that launches with different partition counts on one workspace (another batch
// size or `splits` cap moves the partial slots) never write partials over a counter.
struct Header {
  int status;      // HKV_OK or HKV_ERR_DEVICE_WAIT, set by a kernel whose bounded wait ran out
  int pad[15];
};

constexpr int kMaxParts = 4096;          // partitions (CTAs) of one decode launch: SMs x resident CTAs per SM, capped here
constexpr int kMaxBatch = 8192;          // requests per decode call (coarse prefix table lives in shared memory)
constexpr long long kWaitCycles = 1ll << 32;   // bound of every device-side wait, in SM clock cycles (about 2 s)

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
  size_t ticket_off, lse_off, opart_off, total;
  __host__ __device__ WorkspaceLayout(int n_parts, int rpad, int D) {
    ticket_off = align_up(sizeof(Header), 256);
    lse_off = align_up(ticket_off + sizeof(int) * (size_t)kMaxParts, 256);
    opart_off = align_up(lse_off + sizeof(float) * (size_t)n_parts * 2 * rpad, 256);
    total = align_up(opart_off + sizeof(float) * (size_t)n_parts * 2 * rpad * D, 256);
  }
};

// ------------------------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the phase did not complete within kWaitCycles (the caller records the failure and
// leaves its loop; nothing spins for ever).
static __device__ __noinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}
// the same operations on 32-bit shared-memory addresses (what the main loop of the decode kernel keeps in registers)
__device__ __forceinline__ void mbar_arrive_u32(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_u32(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_u32(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
static __device__ __noinline__ bool mbar_wait_bounded_u32(uint32_t bar, uint32_t parity, long long limit = kWaitCycles) {
  if (mbar_try_wait_u32(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait_u32(bar, parity)) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}
__device__ __forceinline__ void bulk_g2s_u32(uint32_t dst, const void* src_gmem, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src_gmem), "r"(bytes), "r"(bar)
               : "memory");
}
// Ampere-style asynchronous copy of N bytes (8 or 16) global -> shared by this thread, and an arrival on an mbarrier that
// fires when all copies this thread has issued so far have completed (.noinc: the arrival is one of the count the
// barrier was initialised with)
template <int N>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src) {
  static_assert(N == 8 || N == 16, "cp.async moves 4, 8 or 16 bytes");
  if (N == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// shared-memory loads by 32-bit address. volatile keeps them behind the mbarrier wait that guards the stage.
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 r;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(a));
  return r;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(a));
  return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t r;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(a));
  return r;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
  uint32_t r;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(r) : "r"(a));
  return r;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
  uint32_t r;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(r) : "r"(a));
  return r;
}
// true in exactly one lane of a converged warp. The compiler knows that the guarded code runs in a single thread, so
// a bulk copy inside it takes its operands from that thread without a loop over the active lanes.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void sts64_zero(uint32_t a) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %1};" ::"r"(a), "r"(0u) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned), completion counted on
// the mbarrier. No multicast, this CTA's shared memory only.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------------- conversions
// four E2M1 pairs (the 4 bytes of w) -> four f16x2; low nibble of each byte in the low half
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&o)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3])
      : "r"(w));
}
// two E4M3 bytes (low 16 bits of x) -> f16x2, low byte in the low half. 0x7f / 0xff give NaN.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t x) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((unsigned short)x));
  return r;
}
// four E4M3 bytes -> two f16x2 (bytes 0, 1 and bytes 2, 3)
__device__ __forceinline__ void e4m3x4_to_f16x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t x) { return *reinterpret_cast<__half2*>(&x); }
__device__ __forceinline__ uint32_t h2_as_u32(__half2 x) { return *reinterpret_cast<uint32_t*>(&x); }
// f16x2 product with a scale pair that the compiler can take as a half-broadcast operand
__device__ __forceinline__ uint32_t hmul2h(uint32_t a, __half2 b) { return h2_as_u32(__hmul2(u32_as_h2(a), b)); }
// transpose of an 8x8 matrix of 16-bit elements held one row pair per lane (lane l holds row l / 4, columns 2 (l % 4),
// 2 (l % 4) + 1); used to turn the (token, query row) probabilities into the B operand of the second product
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t r;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// the same with out-of-range values (infinities included) clamped to +-65504; a NaN stays a NaN
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: every kernel of this library is launched with the "programmatic stream
// serialization" attribute, waits for the preceding launch to complete before it touches global memory, and lets the
// next launch be scheduled early. Only the launch latency overlaps; the memory order of a stream is unchanged.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace hkv
