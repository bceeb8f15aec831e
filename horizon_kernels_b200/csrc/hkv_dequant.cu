// Exact dequantisation of cached tokens to dense bf16 / fp16 rows, the step between the FP4 cache and a prefill
// attention that wants ordinary K / V tensors.
//
// value = e2m1(code) * e4m3(block scale), WITHOUT the per-tensor global scale: the product has at most five
// significant bits and lies in [2^-10, 2688], so it is exact in fp16 and in bf16 (the caller folds the global scales
// into its softmax scale and its output, as the reference does). Replaces `dequant_tokens` / `hz4::dequant_task`
// (kv_fp4_serving.py:918-925, :577-609) and `dequant_multi` / `hz4::dequant_multi_task` (kv_fp4_serving.py:1008-1016,
// :700-740) of the reference.
//
// One thread per 16-channel block: 8 code bytes + 1 scale byte in, 32 bytes out. Consecutive threads take consecutive
// blocks of a (token, kv head) row and consecutive rows, so a warp stores 1 KB contiguous; its loads are 8-byte pieces
// of 64-byte (head_dim 128) or 128-byte code rows. The kernel moves 2.56 bytes per element and is HBM-bound.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hkv_common.cuh"

namespace hkv {

int record_cuda(cudaError_t e);

struct DequantParams {
  const uint8_t* kd;
  const uint8_t* ksf;
  const uint8_t* vd;
  const uint8_t* vsf;
  long long dsp, dst, dsh, ssp, sst, ssh;
  const int* bt;
  const int* rows;
  const int* cu;
  uint32_t* out_k;
  uint32_t* out_v;
  int MP, n_rows, start, n_tokens, KVH, PS;
};

template <int F16>
__device__ __forceinline__ uint32_t out_pair(uint32_t h2) {        // f16x2 -> the output type's pair (exact)
  if (F16) return h2;
  const __half2 h = u32_as_h2(h2);
  const __nv_bfloat162 b = __floats2bfloat162_rn(__low2float(h), __high2float(h));
  return *reinterpret_cast<const uint32_t*>(&b);
}

// K8 = 1: the K8V4 slot (kv_fp4_ref.py:283-321): a key block is 16 signed E4M3 bytes, converted as they are (the
// key scale is global); value blocks as above.
template <int D, int F16, int K8>
__global__ void __launch_bounds__(256) dequant_kernel(const DequantParams p) {
  constexpr int NB = D / 16;
  pdl_wait();                                     // the cache may come from the preceding launch
  pdl_launch_dependents();
  const int side = blockIdx.y;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int blk = (int)(gid % NB);
  const long long rowid = gid / NB;               // (token, kv head)
  const int h = (int)(rowid % p.KVH);
  const long long tok = rowid / p.KVH;
  if (tok >= p.n_tokens) return;
  long long pos;                                  // position inside the request's context
  const int* btrow;
  if (p.cu == nullptr) {
    pos = p.start + tok;
    btrow = p.bt;
  } else {
    int lo = 0, hi = p.n_rows;                    // largest r with cu[r] <= tok
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(p.cu + mid) <= tok) lo = mid; else hi = mid;
    }
    pos = tok - __ldg(p.cu + lo);
    btrow = p.bt + (long long)__ldg(p.rows + lo) * p.MP;
  }
  uint4* dst = reinterpret_cast<uint4*>((side ? p.out_v : p.out_k) + ((tok * p.KVH + h) * (long long)D + blk * 16) / 2);
  if (pos / p.PS >= p.MP) {
    // a position beyond the block table's reach (bad packed offsets): never read past the table row; the output rows
    // of such positions are zero
    dst[0] = make_uint4(0, 0, 0, 0);
    dst[1] = make_uint4(0, 0, 0, 0);
    return;
  }
  const long long page = __ldg(btrow + pos / p.PS), off = pos % p.PS;
  if (K8 && side == 0) {
    const uint4 w8 = *reinterpret_cast<const uint4*>(p.kd + page * p.dsp + off * p.dst + h * p.dsh + blk * 16);
    const uint32_t ws[4] = {w8.x, w8.y, w8.z, w8.w};
    uint32_t o8[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo, hi;
      e4m3x4_to_f16x2(ws[i], lo, hi);
      o8[2 * i] = out_pair<F16>(lo);
      o8[2 * i + 1] = out_pair<F16>(hi);
    }
    dst[0] = make_uint4(o8[0], o8[1], o8[2], o8[3]);
    dst[1] = make_uint4(o8[4], o8[5], o8[6], o8[7]);
    return;
  }
  const uint8_t* data = (side ? p.vd : p.kd) + page * p.dsp + off * p.dst + h * p.dsh + blk * 8;
  const uint8_t* scl = (side ? p.vsf : p.ksf) + page * p.ssp + off * p.sst + h * p.ssh + blk;
  const uint2 w = *reinterpret_cast<const uint2*>(data);
  const uint32_t sf = e4m3x2_to_f16x2(*scl);      // the scale in the low half
  const __half2 s2 = __low2half2(u32_as_h2(sf));
  uint32_t e[8];
  {
    uint32_t a[4], b[4];
    e2m1x8_to_f16x2(w.x, a);
    e2m1x8_to_f16x2(w.y, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      e[i] = out_pair<F16>(hmul2h(a[i], s2));
      e[4 + i] = out_pair<F16>(hmul2h(b[i], s2));
    }
  }
  dst[0] = make_uint4(e[0], e[1], e[2], e[3]);
  dst[1] = make_uint4(e[4], e[5], e[6], e[7]);
}

}  // namespace hkv

static int dequant_impl(const void* kd, const void* ksf, const void* vd, const void* vsf, const int64_t strides[6],
                        int PS, const int32_t* block_tables, int MP, const int32_t* rows, const int32_t* cu, int n_rows,
                        int64_t start, int64_t n_tokens, void* out_k, void* out_v, int KVH, int D, int out_f16, int k8,
                        void* stream) {
  using namespace hkv;
  if (k8 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (k8 && kd && strides && (((uintptr_t)kd | (uintptr_t)strides[0] | (uintptr_t)strides[1] | (uintptr_t)strides[2]) & 15))
    return HKV_ERR_ALIGN;
  if (n_tokens < 0 || start < 0 || MP < 0 || n_rows < 0) return HKV_ERR_RANGE;
  if (n_tokens == 0) return HKV_OK;
  if (!kd || !ksf || !vd || !vsf || !strides || !block_tables || !out_k || !out_v) return HKV_ERR_NULL;
  if ((rows == nullptr) != (cu == nullptr)) return HKV_ERR_NULL;
  if (cu != nullptr && n_rows < 1) return HKV_ERR_RANGE;
  if (D != 128 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (KVH < 1 || KVH > 1024 || PS < 1) return HKV_ERR_UNSUPPORTED;
  if (((uintptr_t)kd | (uintptr_t)vd) & 7) return HKV_ERR_ALIGN;
  if ((strides[0] | strides[1] | strides[2]) & 7) return HKV_ERR_ALIGN;
  if (((uintptr_t)out_k | (uintptr_t)out_v) & 15) return HKV_ERR_ALIGN;
  if (n_tokens > 0x7fffffffll || start + n_tokens > 0x7fffffffll) return HKV_ERR_RANGE;
  if (cu == nullptr && start + n_tokens > (int64_t)MP * PS) return HKV_ERR_RANGE;   // positions beyond the table row
  DequantParams p;
  p.kd = (const uint8_t*)kd; p.ksf = (const uint8_t*)ksf; p.vd = (const uint8_t*)vd; p.vsf = (const uint8_t*)vsf;
  p.dsp = strides[0]; p.dst = strides[1]; p.dsh = strides[2];
  p.ssp = strides[3]; p.sst = strides[4]; p.ssh = strides[5];
  p.bt = block_tables; p.rows = rows; p.cu = cu;
  p.out_k = (uint32_t*)out_k; p.out_v = (uint32_t*)out_v;
  p.MP = MP; p.n_rows = n_rows; p.start = (int)start; p.n_tokens = (int)n_tokens; p.KVH = KVH; p.PS = PS;
  const long long threads = n_tokens * KVH * (D / 16);
  const long long blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffll) return HKV_ERR_RANGE;
  void (*k)(const DequantParams);
  if (k8) k = out_f16 ? dequant_kernel<256, 1, 1> : dequant_kernel<256, 0, 1>;
  else if (D == 128) k = out_f16 ? dequant_kernel<128, 1, 0> : dequant_kernel<128, 0, 0>;
  else k = out_f16 ? dequant_kernel<256, 1, 0> : dequant_kernel<256, 0, 0>;
  return record_cuda(launch_pdl(k, dim3((unsigned)blocks, 2), dim3(256), 0, (cudaStream_t)stream, p));
}

extern "C" int hkv_dequant(const void* kd, const void* ksf, const void* vd, const void* vsf, const int64_t strides[6],
                           int PS, const int32_t* block_tables, int MP, const int32_t* rows, const int32_t* cu,
                           int n_rows, int64_t start, int64_t n_tokens, void* out_k, void* out_v, int KVH, int D,
                           int out_f16, void* stream) {
  return dequant_impl(kd, ksf, vd, vsf, strides, PS, block_tables, MP, rows, cu, n_rows, start, n_tokens, out_k, out_v,
                      KVH, D, out_f16, 0, stream);
}

extern "C" int hkv_dequant_k8(const void* kd, const void* vd, const void* vsf, const int64_t strides[6], int PS,
                              const int32_t* block_tables, int MP, const int32_t* rows, const int32_t* cu, int n_rows,
                              int64_t start, int64_t n_tokens, void* out_k, void* out_v, int KVH, int D, int out_f16,
                              void* stream) {
  return dequant_impl(kd, kd, vd, vsf, strides, PS, block_tables, MP, rows, cu, n_rows, start, n_tokens, out_k, out_v,
                      KVH, D, out_f16, 1, stream);
}
