// Declarations shared by the two decode kernels (hkv_decode.cu: warp-level mma.sync path for every cache layout;
// hkv_decode_umma.cu: tcgen05 path for head-major slot pages): launch parameters, the per-request view of the unit
// stream, and the log-sum-exp merge of a split sequence.
#pragma once

#include <cuda_bf16.h>

#include "hkv_common.cuh"

namespace hkv {

constexpr int kMaxRows = 64;     // G * qlmax: more rows than one pass serves are handled by several passes over the cache
constexpr float NEG_BIG = -1.0e30f;
constexpr float TAU = 8.0f;      // lazy rescale threshold (log2 domain): P stays below 2^8, inside f16's range

struct DecodeParams {
  const __nv_bfloat16* q;
  const uint8_t* kd;
  const uint8_t* ksf;
  const uint8_t* vd;
  const uint8_t* vsf;
  long long dsh, ssh;                                // byte strides between kv heads (codes, scales)
  unsigned dst;                                      // byte stride between positions of a page (row-copy layout only)
  unsigned dsp, ssp;                                 // byte strides between pages (codes, scales), < 2^31
  const int* bt;
  const int* seq_lens;
  const int* qsl;
  const float* gk;
  const float* gv;
  uint8_t* ws;
  __nv_bfloat16* out;
  int MP, B, KVH, G, qlmax, PS;
  const float* signs;                                // +-1 per channel when the keys were written rotated, else null
  float rot_scale;                                   // head_dim^-0.5 rounded to fp32
  int row0;                                          // first query row (of the G * ql rows of a request and kv head) of this pass
  int max_len;                                       // MP * PS, capped at INT_MAX
  int early_meta;                                    // seq_lens / query_start_loc are read before the launch dependency
  float scale_log2, v_scale;
};

// one request as the unit stream sees it; all fields are warp-uniform
struct ReqInfo {
  int U, L, ql, q0;                                    // units per kv head, context length, query tokens, first query row
};
template <int LOG_UT>
__device__ __forceinline__ ReqInfo load_req(const DecodeParams& p, int b) {
  ReqInfo r;
  r.q0 = __ldg(p.qsl + b);
  int ql = __ldg(p.qsl + b + 1) - r.q0;
  ql = (ql < 0 || ql > p.qlmax || p.G * ql <= p.row0) ? 0 : ql;     // (no rows in this pass: the request is skipped)
  r.ql = ql;
  // (a length beyond the block table's reach is cut there, so that bad metadata can never read past a table row)
  r.L = ql > 0 ? min(max(__ldg(p.seq_lens + b), 0), p.max_len) : 0;
  r.U = ql > 0 ? max(1, (r.L + (1 << LOG_UT) - 1) >> LOG_UT) : 0;
  return r;
}

// a split sequence as the ticket round at the end of a partition needs it
struct SplitSeq {
  int h, U, q0, R;                                   // kv head, units of the whole sequence, first query token, rows of this pass
  long long seq0;                                    // stream position of the sequence (its cost slots come first)
};

// ------------------------------------------------------------------------------------------------------- combine
// Log-sum-exp merge of the pieces of one split sequence, run by the whole CTA that drew the sequence's last ticket.
// The pieces live in slot `first_slot` of partition `first`, and in slot 0 of every later partition up to `last`.
// w_i = 2^(lse_i - max) / sum, accumulated in partition order with a running maximum, so the result does not depend
// on which CTA merges. out_row points at row 0 of the (request, kv head) group's first query token; rows of the next
// token are tok_stride elements further. (Reference: hz4::combine_rg, kv_fp4_serving.py:518-558.)
// RP: rows of a partial slot in the workspace; NT: threads of the calling group; the call merges rows rbase .. rbase + RB - 1
template <int D, int RP, int NT, int RB = RP>
__device__ __forceinline__ void merge_split(const float* lse_ws, const float* opart_ws, int first, int last,
                                            int first_slot, int R, int row0, int G, __nv_bfloat16* out_row,
                                            long long tok_stride, float v_scale, int rbase = 0) {
  constexpr int IT = RB * (D / 2) / NT;      // (row, channel pair) items per thread
  constexpr int GRP = 4;                             // pieces per round: GRP * IT independent loads in flight
  const float ninf = -__int_as_float(0x7f800000);
  float mx[IT], tot[IT], n0[IT], n1[IT];
#pragma unroll
  for (int it = 0; it < IT; ++it) { mx[it] = ninf; tot[it] = n0[it] = n1[it] = 0.0f; }
  for (int pc0 = first; pc0 <= last; pc0 += GRP) {
    float ls[IT][GRP];
    float2 v[IT][GRP];
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int idx = threadIdx.x + it * NT, row = rbase + idx / (D / 2), ch = (idx - (row - rbase) * (D / 2)) * 2;
#pragma unroll
      for (int i = 0; i < GRP; ++i) {
        const int pc = pc0 + i;
        const int slot = pc * 2 + (pc == first ? first_slot : 0);
        const bool on = pc <= last && row < R;
        ls[it][i] = on ? __ldcg(lse_ws + slot * RP + row) : ninf;
        v[it][i] = on ? __ldcg(reinterpret_cast<const float2*>(opart_ws + ((size_t)slot * RP + row) * D + ch))
                      : make_float2(0.f, 0.f);
      }
    }
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      float gm = ls[it][0];
#pragma unroll
      for (int i = 1; i < GRP; ++i) gm = fmaxf(gm, ls[it][i]);
      if (gm == ninf) continue;                      // only empty pieces in this round
      const float nm = fmaxf(mx[it], gm);
      const float keep = mx[it] == ninf ? 0.0f : exp2f(mx[it] - nm);
      tot[it] *= keep; n0[it] *= keep; n1[it] *= keep;
      mx[it] = nm;
#pragma unroll
      for (int i = 0; i < GRP; ++i) {
        if (ls[it][i] == ninf) continue;             // an empty piece: its partial is garbage and must not be used
        const float wgt = exp2f(ls[it][i] - nm);
        tot[it] += wgt;
        n0[it] += v[it][i].x * wgt;
        n1[it] += v[it][i].y * wgt;
      }
    }
  }
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int idx = threadIdx.x + it * NT, row = rbase + idx / (D / 2), ch = (idx - (row - rbase) * (D / 2)) * 2;
    if (row >= R) continue;
    const float inv = tot[it] > 0.0f ? v_scale / tot[it] : 0.0f;
    const int t = (row0 + row) / G, gq = row0 + row - t * G;
    *reinterpret_cast<__nv_bfloat162*>(out_row + t * tok_stride + (long long)gq * D + ch) =
        __floats2bfloat162_rn(n0[it] * inv, n1[it] * inv);
  }
}

}  // namespace hkv
