// Paged split-K flash-decoding over the NVFP4 KV cache, and the log-sum-exp combine (sm_100a).
//
// Work decomposition ("balanced split-K"): the unit of work is UT consecutive tokens (32; 16 for the K8V4 slot)
// of one (request, kv head) sequence. All units of a batch, ordered (request, kv head, position), form one stream that
// is cut into equal partitions, one per CTA of a grid that fills the GPU exactly once. A CTA therefore streams the same
// number of cache bytes as every other CTA whatever the mix of context lengths. Inside a partition, a run of units of
// the same (request, kv head) is a *piece*. A piece that covers its whole sequence is finished by the CTA and written
// to the output; other pieces leave a normalised fp32 partial and a log2-sum-exp in the workspace. The log-sum-exp
// combine of a split sequence runs inside the same launch: every CTA that wrote a piece of it draws a ticket from a
// per-sequence counter when it is done, and the CTA that draws the last ticket merges all pieces in partition order
// (fixed order => deterministic results, whoever merges). No CTA ever waits for another one.
//
// Inside a CTA, TG warps take the partition's units round-robin. Every warp owns a private ring of NS shared-memory
// stages; it issues 1-D bulk copies (cp.async.bulk, completion on an mbarrier) for its own future units, driven by
// the block table, and consumes them in order, so the main loop needs no cross-warp synchronisation. Per 16 tokens a
// warp computes S^T = K Q^T with mma.m16n8k16 (A = 16 keys dequantised in registers from E2M1 codes with
// cvt.rn.f16x2.e2m1x2 and one f16x2 multiply by the E4M3 block scale, B = the query rows), an online softmax in the
// log2 domain whose running maximum moves lazily, a movmatrix transpose of P, and O^T += V^T P^T with A = dequantised
// values. code * scale is exact in f16 (at most 5 significant bits, magnitude in [2^-10, 2688]), so the only roundings
// are P to f16 and the fp32 accumulations. At the end of a piece the TG warps merge their (max, sum, accumulator)
// states through shared memory.
//
// Every wait on an mbarrier is bounded (hkv::kWaitCycles); when one runs out the kernel records
// HKV_ERR_DEVICE_WAIT in the workspace header, stops consuming and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <cmath>

#include "hkv_decode.cuh"

namespace hkv {

constexpr int TG = 4;            // consumer warps per CTA
constexpr bool kQueryPrefetch = true;   // ask for the next sequence's query rows (L2 prefetch) while a piece is computed
constexpr int NTHREADS = TG * 32;
constexpr int RPAD = 8;          // query rows per (request, kv head) of one pass, padded to the mma N tile

// Shared-memory geometry of one stage (K tile then V tile of one unit) for head_dim D and cache layout LAYOUT:
//   LAYOUT 0  token rows of [D/2 code bytes | D/16 scale bytes] back to back (the serving "slot" layout with heads
//             outermost inside a page): one bulk copy of 16 * slot bytes per 16 tokens and side
//   LAYOUT 1  code rows back to back, then the scale rows (the page-region layout of the reference's torch oracle):
//             two bulk copies per 16 tokens and side
//   LAYOUT 3  the same token rows as LAYOUT 0, but the rows of a head are NOT back to back in the cache (positions
//             outermost inside a page, vLLM's NHD order, or any other position / head strides): every lane copies one
//             row per 16 tokens and side with 8-byte (head_dim 128) or 16-byte (256) cp.async into the stage geometry
//             of LAYOUT 0, so the compute side is the same
//   LAYOUT 2  the K8V4 slot (head_dim 256; kv_fp4_ref.py:283-293): token rows of [D signed E4M3 key bytes | D/2 value
//             codes | D/16 value scales], heads outermost: keys and values of 16 tokens are ONE bulk copy of
//             16 * 400 bytes; the stage holds those rows as they are
template <int D, int LAYOUT>
struct Geo {
  static constexpr int SD = D / 2, SS = D / 16, SLOT = SD + SS;
  static constexpr int UB = (D == 128 || LAYOUT != 2) ? 2 : 1;   // 16-token blocks per unit (1 for the K8V4 slot)
  static constexpr int UT = 16 * UB, LOG_UT = UB == 2 ? 5 : 4;
  static constexpr int NS = D == 128 ? 3 : LAYOUT == 2 ? 3 : 2;   // stages per warp
  static constexpr int MINB = D == 128 ? 3 : 2;        // CTAs per SM the register budget is sized for
  static constexpr bool K8 = LAYOUT == 2;
  static constexpr int SLOT8 = D + SD + SS;            // K8V4 slot: 400 bytes at head_dim 256
  static constexpr int TILE = UT * SLOT;               // bytes of one (head, side) tile of a unit
  static constexpr int STAGE = K8 ? UT * SLOT8 : 2 * TILE;
  static constexpr bool SLOTROWS = LAYOUT == 0 || LAYOUT == 3;        // rows of [codes | scales] in shared memory
  static constexpr bool ROWCOPY = LAYOUT == 3;                         // fetched row by row with cp.async
  static constexpr int ROW = K8 ? SLOT8 : SLOTROWS ? SLOT : SD;      // byte stride between token rows in shared memory
  static constexpr int SD_ROW = ROW;                   // .. and between the rows of one head in the cache
  static constexpr int KB = K8 ? 16 : 8;               // bytes of one 16-channel key block
  static constexpr int V_BASE = K8 ? D : TILE;         // first value byte of the stage (of row 0)
  static constexpr int SF_BASE = LAYOUT == 1 ? UT * SD : SD;        // value / key scales behind their side's codes
  static constexpr int SF_ROW = K8 ? SLOT8 : SLOTROWS ? SLOT : SS;
  // What a sequence costs a partition beyond its units (locating it, loading its queries, the end-of-piece merge and
  // the output), in units: measured 3 to 4 microseconds per piece. The stream that is cut into equal partitions counts
  // every sequence as PIECE_COST + its units, so partitions that hold many short sequences get fewer units.
  static constexpr int PIECE_COST = UB == 2 ? 12 : 24;
  static constexpr int KS = D / 16;                    // k-steps of K Q^T == mma tiles of V^T P^T (per 16 tokens)
  static constexpr int NBL = D / 64;                   // 16-channel blocks of one key row held by one lane
  static constexpr int NH = D / 128;                   // 16-channel blocks of one value row held by one lane
  static constexpr int NCH = D == 256 ? 2 : 1;          // independent accumulators per score tile
  // token (row of a 16-token block) handled by row i of the 16-row score tile. With 72-byte rows (head_dim 128, slot
  // layout) bits 1 and 3 of i are swapped: then the key loads of a half warp (rows i = 4k .. 4k+3, 16 bytes apart
  // inside a row) and its value loads (rows i = j, j+2, j+4, j+6, 32 contiguous bytes of each) both touch every
  // shared-memory bank once. 144-byte rows need no permutation.
  __device__ static constexpr int tok(int i) {
    return (D == 128 && SLOTROWS) ? ((i & 5) | ((i & 2) << 2) | ((i & 8) >> 2)) : i;
  }
  // 16-channel block of a key row held by lane column c as its u-th block: NBL adjacent blocks per lane, so that
  // their scale bytes come with one load
  __device__ static constexpr int kblk(int c, int u) { return NBL * c + u; }
};

// QT: 8-row query tiles of one pass (1, or 2 at head_dim 128: sixteen query rows per kv head read the cache once)
template <int D, int LAYOUT, int QT = 1>
struct Smem {
  using G_ = Geo<D, LAYOUT>;
  static constexpr int RP = RPAD * QT;                              // query rows of one pass
  static constexpr int RING = TG * G_::NS * G_::STAGE;
  static constexpr int BARS = TG * G_::NS * 8;
  static constexpr int OROW = D + 4;                               // padded accumulator row (floats)
  static constexpr int MERGE = TG * RP * OROW * 4 + TG * RP * 2 * 4;
  static constexpr int COARSE = (kMaxBatch / 32 + 2) * 4;
  static constexpr int TOTAL = RING + BARS + MERGE + COARSE + 64;
};

template <int D, int LAYOUT, int QT = 1>
__global__ void __launch_bounds__(NTHREADS, QT == 2 ? 2 : Geo<D, LAYOUT>::MINB) decode_kernel(const DecodeParams p) {
  using Gm = Geo<D, LAYOUT>;
  using Sm = Smem<D, LAYOUT, QT>;
  constexpr int RP = Sm::RP;
  constexpr int NS = Gm::NS, UB = Gm::UB, UT = Gm::UT, LOG_UT = Gm::LOG_UT;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Sm::RING);
  float* obuf = reinterpret_cast<float*>(smem + Sm::RING + Sm::BARS);
  float* mbuf = obuf + TG * RP * Sm::OROW;
  float* lbuf = mbuf + TG * RP;
  int* coarse = reinterpret_cast<int*>(smem + Sm::RING + Sm::BARS + Sm::MERGE);
  __shared__ SplitSeq split[2];
  __shared__ int split_win[2];
  unsigned pending = 0, drawn = 0;                  // bit 0 / 1: the partition's first / last piece belongs to a split
                                                    // sequence; .. and its ticket has been drawn already

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, c = lane & 3;
  const int KVH = p.KVH, B = p.B;
  Header* hdr = reinterpret_cast<Header*>(p.ws);
  const int n_parts = gridDim.x, part = blockIdx.x;
  const WorkspaceLayout wl(n_parts, RP, D);
  int* tickets = reinterpret_cast<int*>(p.ws + wl.ticket_off);
  float* lse_ws = reinterpret_cast<float*>(p.ws + wl.lse_off);
  float* opart_ws = reinterpret_cast<float*>(p.ws + wl.opart_off);

  if (tid < TG * NS) mbar_init(bars + tid, Gm::ROWCOPY ? 32 : 1);   // (row copies: every lane of the warp arrives)
  if (tid < 2) split_win[tid] = 0;
  // Every global input may come from the preceding launch, so the kernel waits for it here. The caller may state that
  // the request metadata is older than that launch (hkv_set_option): then the partition search below, which reads only
  // seq_lens and query_start_loc, runs while the preceding launch is still draining, and the wait comes after it.
  const bool early = p.early_meta != 0;
  if (!early) pdl_wait();

  // ---- coarse prefix of the weight (units + piece cost) per request and head: coarse[k] = sum over b < 32 k
  constexpr int PC = Gm::PIECE_COST;
  auto wt = [](int U) { return U > 0 ? U + PC : 0; };
  const int ngrp = (B + 31) >> 5;
  for (int grp = w; grp < ngrp; grp += TG) {
    const int b = grp * 32 + lane;
    int u = b < B ? wt(load_req<LOG_UT>(p, b).U) : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
    if (lane == 0) coarse[grp + 1] = u;
  }
  __syncthreads();
  if (w == 0) {                                   // scan of up to kMaxBatch / 32 group sums
    const int per_lane = (ngrp + 31) >> 5;
    int s = 0;
    for (int i = 0; i < per_lane; ++i) {
      const int k = lane * per_lane + i;
      s += k < ngrp ? coarse[k + 1] : 0;
    }
    int incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    int run = incl - s;
    for (int i = 0; i < per_lane; ++i) {
      const int k = lane * per_lane + i;
      if (k < ngrp) {
        const int v = coarse[k + 1];
        coarse[k + 1] = run + v;                  // inclusive: coarse[k + 1] = units of requests < 32 (k + 1)
        run += v;
      }
    }
    if (lane == 0) coarse[0] = 0;
  }
  fence_barrier_init();
  __syncthreads();

  const long long total = (long long)coarse[ngrp] * KVH;
  const int per = (int)max(1ll, (total + n_parts - 1) / n_parts);
  const long long lo = (long long)part * per;
  const long long hi = min(total, lo + per);
  if (lo >= hi) {                                   // an idle partition
    if (early) pdl_wait();
    pdl_launch_dependents();
    return;
  }

  // ---- locate the request that holds stream position lo (warp-uniform, every warp for itself)
  int b0, base0;                                   // request and weight of earlier requests (per head)
  {
    int lo_g = 0, hi_g = ngrp;                     // largest grp with coarse[grp] * KVH <= lo
    while (hi_g - lo_g > 1) {
      const int mid = (lo_g + hi_g) >> 1;
      if ((long long)coarse[mid] * KVH <= lo) lo_g = mid; else hi_g = mid;
    }
    const int b = lo_g * 32 + lane;
    const int u = b < B ? wt(load_req<LOG_UT>(p, b).U) : 0;
    int incl = u;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, (long long)(coarse[lo_g] + incl) * KVH > lo);
    const int j = __ffs(hit) - 1;                  // first request whose end lies beyond lo
    b0 = lo_g * 32 + j;
    base0 = coarse[lo_g] + __shfl_sync(0xffffffffu, incl - u, j);
  }

  // ---- units (not cost slots) of the partition: request b with weighted start S holds, before stream position x,
  // floor(t / W) * U + max(0, t mod W - PC) units, t = min(x - S, KVH * W); 32 requests at a time
  int n_units = 0;
  for (int grp = b0 >> 5; grp < ngrp && (long long)coarse[grp] * KVH < hi; ++grp) {
    const int b = grp * 32 + lane;
    const int U = b < B ? load_req<LOG_UT>(p, b).U : 0, W = wt(U);
    int incl = W;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const long long S = (long long)(coarse[grp] + incl - W) * KVH;
    auto before = [&](long long x) -> long long {
      if (W == 0 || x <= S) return 0;
      const long long t = min(x - S, (long long)KVH * W);
      return (t / W) * U + max(0ll, t % W - PC);
    };
    int n = (int)(before(hi) - before(lo));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    n_units += n;
  }

  // ---- compute-side walker over the pieces of the partition (identical in every warp)
  struct Walker {
    int b, h;
    long long seq0;                                // stream position of (b, h): PC cost slots, then its units
    ReqInfo r;
  };
  auto seek = [&](Walker& wk, long long pos) {     // move to the sequence that holds pos (pos < total)
    while (true) {
      const long long end_h = wk.seq0 + wt(wk.r.U);
      if (pos < end_h) break;
      wk.seq0 = end_h;
      if (++wk.h == KVH) {
        wk.h = 0;
        do { wk.r = load_req<LOG_UT>(p, ++wk.b); } while (wk.r.U == 0);
      }
    }
  };
  Walker cw;
  cw.b = b0;
  cw.r = load_req<LOG_UT>(p, b0);
  cw.h = (int)((lo - (long long)base0 * KVH) / wt(cw.r.U));
  cw.seq0 = (long long)base0 * KVH + (long long)cw.h * wt(cw.r.U);

  // ---- fetch side: this warp's units are the partition-local indices w, w + TG, ..; the cursor below runs NS units
  // ahead of the compute loop. The common case (next unit in the same sequence, its page ids already in the warp's
  // 32-entry window) costs a shuffle per 16 tokens, one 64-bit multiply-add and the copy instructions of UB lanes.
  const int n_my = n_units > w ? (n_units - w + TG - 1) / TG : 0;
  const int n_tok = __ldg(p.qsl + B);              // query rows of the batch (bounds the query prefetch)
  // shared-memory addresses of this warp's ring and barriers, and the byte offsets of this lane's rows and blocks
  // inside a stage. They are constant for the whole kernel; passing them through an empty asm keeps the compiler from
  // re-deriving them from the thread index inside the main loop.
  uint32_t ring_a = smem_u32(ring + w * NS * Gm::STAGE), bars_a = smem_u32(bars + w * NS);
  const int r0 = Gm::tok(g), r1 = Gm::tok(g + 8);
  const int t00 = Gm::tok(2 * c);
  uint32_t koff_d = r0 * Gm::ROW + Gm::KB * Gm::kblk(c, 0), koff_s = Gm::SF_BASE + r0 * Gm::SF_ROW + Gm::kblk(c, 0);
  uint32_t voff_d = Gm::V_BASE + t00 * Gm::ROW + 8 * g, voff_s = Gm::V_BASE + Gm::SF_BASE + t00 * Gm::SF_ROW + g;
  asm volatile("" : "+r"(ring_a), "+r"(bars_a), "+r"(koff_d), "+r"(koff_s), "+r"(voff_d), "+r"(voff_s));
  constexpr int KR1 = Gm::tok(8) - Gm::tok(0);                            // r1 - r0 (the same for every g)
  constexpr int VR01 = Gm::tok(1) - Gm::tok(0), VR10 = Gm::tok(8) - Gm::tok(0),
                VR11 = Gm::tok(9) - Gm::tok(0);                           // t01 - t00, t10 - t00, t11 - t00 (for every c)

  int f_b = cw.b, f_h = cw.h, f_U = cw.r.U, f_L = cw.r.L;
  int f_blk = w + (int)max(0ll, lo - cw.seq0 - PC);  // unit (inside the cursor's sequence) to fetch next; may run past
  int f_fast_end = 0;                               // units below this bound take the fast path
  int f_idx = 0, pg = 0;                            // page ids of the warp's next 32 blocks of the sequence, one per lane
  unsigned f_n = 0;                                 // units fetched so far (of n_my)
  const uint8_t* f_k = p.kd + (long long)f_h * p.dsh;
  const uint8_t* f_v = p.vd + (long long)f_h * p.dsh;
  const uint8_t* f_ks = p.ksf + (long long)f_h * p.ssh;
  const uint8_t* f_vs = p.vsf + (long long)f_h * p.ssh;
  const int* f_bt = p.bt + (long long)f_b * p.MP;
  const int lps = 31 - __clz(p.PS);                 // page size is a power of two

  auto fetch_slow = [&](const uint32_t bar) -> bool {                 // true: the unit carries no bytes and has been dealt with here
    if (f_blk >= f_U) {                             // the cursor left its sequence: walk to the one that holds the unit
      do {
        f_blk -= f_U;
        if (++f_h == KVH) {
          f_h = 0;
          ReqInfo r;
          do { r = load_req<LOG_UT>(p, ++f_b); } while (r.U == 0);
          f_U = r.U;
          f_L = r.L;
        }
      } while (f_blk >= f_U);
      f_k = p.kd + (long long)f_h * p.dsh;
      f_v = p.vd + (long long)f_h * p.dsh;
      f_ks = p.ksf + (long long)f_h * p.ssh;
      f_vs = p.vsf + (long long)f_h * p.ssh;
      f_bt = p.bt + (long long)f_b * p.MP;
    }
    if (f_L == 0) {                                 // an empty context has one unit and nothing to read: complete the
      if (Gm::ROWCOPY || lane == 0) mbar_arrive_u32(bar);   // phase with plain arrivals so that both sides stay in step
      f_fast_end = 0;
      return true;
    }
    // refill the page window from the current unit: lane j holds the page of 16-token block j % UB of the warp's
    // (j / UB)-th next unit
    const int tok_l = (f_blk + (lane / UB) * TG) * UT + (lane % UB) * 16;
    pg = tok_l < f_L ? __ldg(f_bt + (tok_l >> lps)) : 0;
    f_idx = 0;
    f_fast_end = min(f_U, f_blk + (32 / UB) * TG);
    return false;
  };
  // fetches this warp's next unit into the stage at shared address st, completion on the barrier at address bar
  auto fetch_one = [&](const uint32_t bar, const uint32_t st) {
    bool empty = false;
    if (f_blk >= f_fast_end) empty = fetch_slow(bar);
    if (!empty) {
      int page[UB];                                             // page ids of the unit's 16-token blocks (warp-uniform)
#pragma unroll
      for (int bi = 0; bi < UB; ++bi) page[bi] = __shfl_sync(0xffffffffu, pg, f_idx + bi);
      f_idx += UB;
      const int tok0 = f_blk * UT;
      const int nb = min(UB, (f_L - tok0 + 15) >> 4);          // 16-token blocks of this unit that exist
      if (Gm::ROWCOPY) {
        // lane -> (side, token row) of every 16-token block: SLOT bytes from its own address, in 8- or 16-byte pieces
        constexpr int CB = D == 128 ? 8 : 16;
        const int side = lane >> 4, row = lane & 15;
        const uint8_t* base = side ? f_v : f_k;
#pragma unroll
        for (int bi = 0; bi < UB; ++bi) {
          if (bi < nb) {
            const unsigned pos0 = (unsigned)(tok0 + 16 * bi) & (unsigned)(p.PS - 1);
            const uint8_t* src = base + (unsigned long long)(unsigned)page[bi] * p.dsp +
                                 (unsigned long long)(pos0 + row) * p.dst;
            const uint32_t dsm = st + bi * (16 * Gm::SLOT) + side * Gm::TILE + row * Gm::SLOT;
#pragma unroll
            for (int j = 0; j < Gm::SLOT / CB; ++j) cp_async<CB>(dsm + j * CB, src + j * CB);
          }
        }
        cp_async_mbar_arrive_noinc(bar);                        // arrives once this lane's copies have landed
      } else if (elect_one()) {                                 // one lane arms the barrier and issues the copies
        mbar_expect_tx_u32(bar, nb * (Gm::STAGE / UB));
#pragma unroll
        for (int bi = 0; bi < UB; ++bi) {
          if (bi < nb) {
            const unsigned pos0 = (unsigned)(tok0 + 16 * bi) & (unsigned)(p.PS - 1);
            const unsigned long long doff = (unsigned long long)(unsigned)page[bi] * p.dsp + pos0 * (unsigned)Gm::SD_ROW;
            if (LAYOUT == 2) {
              bulk_g2s_u32(st + bi * (16 * Gm::SLOT8), f_k + doff, 16 * Gm::SLOT8, bar);
            } else if (LAYOUT == 0) {
              bulk_g2s_u32(st + bi * (16 * Gm::SLOT), f_k + doff, 16 * Gm::SLOT, bar);
              bulk_g2s_u32(st + bi * (16 * Gm::SLOT) + Gm::TILE, f_v + doff, 16 * Gm::SLOT, bar);
            } else {
              const unsigned long long soff = (unsigned long long)(unsigned)page[bi] * p.ssp + pos0 * (unsigned)Gm::SS;
              const uint32_t sd = st + bi * (16 * Gm::SD), ss = st + UT * Gm::SD + bi * (16 * Gm::SS);
              bulk_g2s_u32(sd, f_k + doff, 16 * Gm::SD, bar);
              bulk_g2s_u32(ss, f_ks + soff, 16 * Gm::SS, bar);
              bulk_g2s_u32(sd + Gm::TILE, f_v + doff, 16 * Gm::SD, bar);
              bulk_g2s_u32(ss + Gm::TILE, f_vs + soff, 16 * Gm::SS, bar);
            }
          }
        }
      }
    }
    f_blk += TG;
    ++f_n;
  };

  if (early) pdl_wait();                            // from here on: workspace writes, block tables, cache and query reads
  pdl_launch_dependents();

  unsigned c_n = 0;                                 // stages consumed so far
  uint32_t c_bar = bars_a, c_st = ring_a, c_par = 0;  // barrier, stage and phase parity of the next stage to consume
  auto advance = [&]() {
    ++c_n;
    c_bar += 8;
    c_st += Gm::STAGE;
    if (c_bar == bars_a + 8 * NS) {
      c_bar = bars_a;
      c_st = ring_a;
      c_par ^= 1;
    }
  };
  bool dead = false;                                // a bounded wait ran out: stop consuming
  while (f_n < NS && (int)f_n < n_my) fetch_one(bars_a + 8 * f_n, ring_a + f_n * Gm::STAGE);

  // one thread, after a CTA barrier behind which every thread has fenced its share of the partial: counts this piece
  // as finished; true when it was the sequence's last outstanding one (then the counter goes back to zero: every piece
  // has arrived, nobody touches it again in this launch)
  auto draw_ticket = [&](const SplitSeq& sq) -> int {
    const long long seq_u0 = sq.seq0 + PC;
    const int first = (int)(seq_u0 / per), last = (int)((seq_u0 + sq.U - 1) / per);
    __threadfence();
    const int win = atomicAdd(tickets + last, 1) == last - first;
    if (win) tickets[last] = 0;
    return win;
  };

  // ---- compute side: walk the pieces of the partition
  long long pos = lo;
  int piece_idx = 0, k_units = 0;                   // pieces and units of the partition dealt with so far
  while (pos < hi) {
    seek(cw, pos);
    // the sequence's units occupy [seq0 + PC, seq_end); the part of them inside [pos, hi) is this partition's piece
    const long long seq_u0 = cw.seq0 + PC, seq_end = seq_u0 + cw.r.U;
    const long long piece_lo = max(pos, seq_u0), piece_end = min(hi, seq_end);
    if (piece_lo >= piece_end) {                    // only cost slots of this sequence lie in the partition
      pos = min(hi, seq_end);
      continue;
    }
    const int blk0 = (int)(piece_lo - seq_u0);
    const int n_piece = (int)(piece_end - piece_lo);
    const int k0 = k_units;                         // partition-local index of the piece's first unit
    k_units += n_piece;
    const int b = cw.b, h = cw.h, L = cw.r.L, ql = cw.r.ql, q0 = cw.r.q0, G = p.G;
    const int R = min(RP, G * ql - p.row0);      // query rows of this pass: rows row0 .. row0 + R - 1 of the group
    const bool complete = blk0 == 0 && piece_end == seq_end;
    if (kQueryPrefetch && w == 0 && piece_end < hi) {
      // the partition goes on with the next sequence: ask for its query rows now (L2 prefetch, no registers held), so
      // that their load latency passes behind this piece instead of stalling all four warps at the start of the next
      long long row;                                 // first query row of the next sequence (clamped into the tensor)
      if (h + 1 < KVH) row = (long long)q0 * (KVH * G) + (h + 1) * G;
      else row = (long long)min(q0 + ql, n_tok - 1) * (KVH * G);
      const char* a = reinterpret_cast<const char*>(p.q + row * D) + lane * 128;
      if (lane * 128 < G * D * 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    }
    if (!complete && tid == 0) {
      // a piece of a split sequence: remember the sequence for the ticket round at the end of the partition (at most
      // two per partition: its first piece and, when the last sequence runs on into the next partition, its last)
      SplitSeq& sq = split[piece_idx == 0 ? 0 : 1];
      sq.h = h; sq.U = cw.r.U; sq.q0 = q0; sq.R = R; sq.seq0 = cw.seq0;
    }
    if (!complete) pending |= piece_idx == 0 ? 1u : 2u;
    // a split piece that is not the partition's last work draws its ticket as soon as it is stored: the latency passes
    // behind the SM's other CTAs, and the end of the partition is left with at most one sequence to settle
    const bool draw_now = !complete && piece_end < hi;

    // this warp's units of the piece: blk_first, blk_first + TG, .. < blk_end
    const int blk_first = blk0 + ((w - k0) % TG + TG) % TG, blk_end = blk0 + n_piece;
    // running max (raw score units) and sum of query rows 2c and 2c+1 over this lane's tokens
    // (per 8-row query tile q: rows 8 q + 2c and 8 q + 2c + 1)
    float m0[QT], m1[QT], l0[QT], l1[QT];
    float o[QT][Gm::KS][4];
#pragma unroll
    for (int q = 0; q < QT; ++q) {
      m0[q] = m1[q] = NEG_BIG;
      l0[q] = l1[q] = 0.0f;
#pragma unroll
      for (int j = 0; j < Gm::KS; ++j) o[q][j][0] = o[q][j][1] = o[q][j][2] = o[q][j][3] = 0.0f;
    }

    if (blk_first < blk_end && !dead) {
      // softmax scale in the log2 domain. A negative scale is moved into the query so that "max" stays a max.
      float sc = p.scale_log2 * __ldg(p.gk + h);
      const bool flip = sc < 0.0f;
      sc = fmaxf(fabsf(sc), 1e-30f);
      const float tau_raw = TAU / sc;
      // query fragments: row g of the (request, kv head) group, channels of this lane's key blocks, as f16
      uint32_t qa[QT][Gm::KS][2];
#pragma unroll
      for (int q = 0; q < QT; ++q) {
        const bool have = g + 8 * q < R;
        const int t = have ? (p.row0 + g + 8 * q) / G : 0, gq = have ? p.row0 + g + 8 * q - t * G : 0;
        const __nv_bfloat16* qrow = p.q + ((long long)(q0 + t) * (KVH * G) + h * G + gq) * D;
        constexpr int NQ = 16 * Gm::NBL;            // this lane's channels: NQ * c .. NQ * c + NQ - 1 of the row
        float qf[NQ];
#pragma unroll
        for (int u = 0; u < Gm::NBL; ++u) {
          uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
          if (have) {
            const uint4* src = reinterpret_cast<const uint4*>(qrow + 16 * Gm::kblk(c, u));
            x0 = __ldg(src);
            x1 = __ldg(src + 1);
          }
          const uint32_t ws[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            qf[16 * u + 2 * i] = __uint_as_float(ws[i] << 16);
            qf[16 * u + 2 * i + 1] = __uint_as_float(ws[i] & 0xffff0000u);
          }
        }
        if (p.signs != nullptr) {
          // keys were written rotated: q' = bf16(FWHT(q * signs) * head_dim^-0.5), the reference's rotate_q
          // (kv_fp4_ref.py:90-92), fp32 butterflies in its stage order. The four lanes of a quad hold one row.
          const float4* sg = reinterpret_cast<const float4*>(p.signs + NQ * c);
#pragma unroll
          for (int i = 0; i < NQ / 4; ++i) {
            const float4 s4 = __ldg(sg + i);
            qf[4 * i] = __fmul_rn(qf[4 * i], s4.x);
            qf[4 * i + 1] = __fmul_rn(qf[4 * i + 1], s4.y);
            qf[4 * i + 2] = __fmul_rn(qf[4 * i + 2], s4.z);
            qf[4 * i + 3] = __fmul_rn(qf[4 * i + 3], s4.w);
          }
#pragma unroll
          for (int hh = 1; hh < NQ; hh *= 2)
#pragma unroll
            for (int i = 0; i < NQ; ++i)
              if ((i & hh) == 0) {
                const float a = qf[i], b = qf[i + hh];
                qf[i] = __fadd_rn(a, b);
                qf[i + hh] = __fsub_rn(a, b);
              }
#pragma unroll
          for (int m = 1; m < 4; m *= 2) {          // stages h = NQ, 2 NQ: the partner is the lane with c ^ m
            const bool upper = (c & m) != 0;
#pragma unroll
            for (int i = 0; i < NQ; ++i) {
              const float o2 = __shfl_xor_sync(0xffffffffu, qf[i], m);
              qf[i] = upper ? __fsub_rn(o2, qf[i]) : __fadd_rn(qf[i], o2);
            }
          }
#pragma unroll
          for (int i = 0; i < NQ; ++i) qf[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(qf[i], p.rot_scale)));
        }
#pragma unroll
        for (int i = 0; i < NQ / 2; ++i) {
          float a = qf[2 * i], bq = qf[2 * i + 1];
          if (flip) { a = -a; bq = -bq; }
          qa[q][i >> 1][i & 1] = pack_f16x2_sat(a, bq);   // values beyond f16's range become +-65504
        }
      }
      // visible context of query rows 2c, 2c+1 (causal among the request's own query tokens)
      int lim0[QT], lim1[QT];
#pragma unroll
      for (int q = 0; q < QT; ++q) {
        const int ra = 8 * q + 2 * c, rb = ra + 1;
        lim0[q] = ra < R ? L - ql + (p.row0 + ra) / G + 1 : L;
        lim1[q] = rb < R ? L - ql + (p.row0 + rb) / G + 1 : L;
      }
      const int blk_mask = (L - ql + p.row0 / G + 1) >> LOG_UT;   // units below this one are visible to every row in full
      float mneg0[QT], mneg1[QT], thr0[QT], thr1[QT];   // p = 2^(s * sc + mneg)
#pragma unroll
      for (int q = 0; q < QT; ++q) {
        mneg0[q] = -m0[q] * sc; mneg1[q] = -m1[q] * sc;
        thr0[q] = m0[q] + tau_raw; thr1[q] = m1[q] + tau_raw;
      }

      // waits (bounded) for the next stage this warp consumes; false once a wait ran out
      // (the stage's addresses come back in bar and st: the unit fetched after it reuses them)
      auto wait_stage = [&](uint32_t& bar, uint32_t& st) -> bool {
        if (!mbar_try_wait_u32(c_bar, c_par)) {
          if (!mbar_wait_bounded_u32(c_bar, c_par)) {
            if (lane == 0) atomicExch(&hdr->status, HKV_ERR_DEVICE_WAIT);
            dead = true;
            return false;
          }
        }
        bar = c_bar;
        st = c_st;
        advance();
        return true;
      };

      // ---------------- S^T = K Q^T per 16-token block: rows = tokens, columns = query rows
      auto k_phase = [&](const uint32_t st, float (&x)[QT][UB][4]) {
        const uint32_t kd_ = st + koff_d, ks_ = st + koff_s;
#pragma unroll
        for (int bi = 0; bi < UB; ++bi) {
          float sa[QT][Gm::NCH][4];
#pragma unroll
          for (int q = 0; q < QT; ++q)
#pragma unroll
            for (int i = 0; i < Gm::NCH; ++i) sa[q][i][0] = sa[q][i][1] = sa[q][i][2] = sa[q][i][3] = 0.0f;
          if (Gm::K8) {
            // FP8 keys: 16 bytes per block and row, no block scale (the global scale is part of `sc`)
            const int dk8 = bi * 16 * Gm::ROW;
#pragma unroll
            for (int u = 0; u < Gm::NBL; ++u) {
              const uint4 a = lds128(kd_ + dk8 + 16 * u), b = lds128(kd_ + dk8 + KR1 * Gm::ROW + 16 * u);
              const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int v = 0; v < 4; ++v) {           // k-step v of the block: channels 4v .. 4v+3 of rows r0, r1
                uint32_t a0, a2, a1, a3;
                e4m3x4_to_f16x2(wa[v], a0, a2);
                e4m3x4_to_f16x2(wb[v], a1, a3);
#pragma unroll
                for (int q = 0; q < QT; ++q)
                  mma_f16(sa[q][v & (Gm::NCH - 1)], a0, a1, a2, a3, qa[q][4 * u + v][0], qa[q][4 * u + v][1]);
              }
            }
#pragma unroll
            for (int q = 0; q < QT; ++q)
#pragma unroll
              for (int i = 0; i < 4; ++i) x[q][bi][i] = Gm::NCH == 2 ? sa[q][0][i] + sa[q][Gm::NCH - 1][i] : sa[q][0][i];
            continue;
          }
          // codes and scales of this lane's NBL adjacent key blocks of rows r0 and r1
          const int dk = bi * 16 * Gm::ROW, sk = bi * 16 * Gm::SF_ROW;
          uint2 w0[Gm::NBL], w1[Gm::NBL];
          uint32_t h0[Gm::NBL / 2 + 1], h1[Gm::NBL / 2 + 1];   // f16x2 scale pairs (block 2j, block 2j+1) of r0 / r1
          if (Gm::NBL == 2) {
            w0[0] = lds64(kd_ + dk);
            w0[1] = lds64(kd_ + dk + 8);
            w1[0] = lds64(kd_ + dk + KR1 * Gm::ROW);
            w1[1] = lds64(kd_ + dk + KR1 * Gm::ROW + 8);
            h0[0] = e4m3x2_to_f16x2(lds16(ks_ + sk));
            h1[0] = e4m3x2_to_f16x2(lds16(ks_ + sk + KR1 * Gm::SF_ROW));
          } else {
#pragma unroll
            for (int j = 0; j < Gm::NBL / 2; ++j) {
              const uint4 a = lds128(kd_ + dk + 16 * j), b = lds128(kd_ + dk + KR1 * Gm::ROW + 16 * j);
              w0[2 * j] = make_uint2(a.x, a.y);
              w0[2 * j + 1] = make_uint2(a.z, a.w);
              w1[2 * j] = make_uint2(b.x, b.y);
              w1[2 * j + 1] = make_uint2(b.z, b.w);
            }
            e4m3x4_to_f16x2(lds32(ks_ + sk), h0[0], h0[1]);
            e4m3x4_to_f16x2(lds32(ks_ + sk + KR1 * Gm::SF_ROW), h1[0], h1[1]);
          }
#pragma unroll
          for (int u = 0; u < Gm::NBL; ++u) {
            const __half2 p0 = u32_as_h2(h0[u >> 1]), p1 = u32_as_h2(h1[u >> 1]);
            const __half2 sf0 = (u & 1) ? __high2half2(p0) : __low2half2(p0);
            const __half2 sf1 = (u & 1) ? __high2half2(p1) : __low2half2(p1);
            uint32_t e0[4], e1[4], e2[4], e3[4];
            e2m1x8_to_f16x2(w0[u].x, e0);
            e2m1x8_to_f16x2(w0[u].y, e1);
            e2m1x8_to_f16x2(w1[u].x, e2);
            e2m1x8_to_f16x2(w1[u].y, e3);
            // k-step v of this block: A = {row r0 k-low, row r1 k-low, row r0 k-high, row r1 k-high}
            // (the dequantised A fragments serve every query tile)
            const uint32_t A0[4] = {hmul2h(e0[0], sf0), hmul2h(e2[0], sf1), hmul2h(e0[1], sf0), hmul2h(e2[1], sf1)};
            const uint32_t A1[4] = {hmul2h(e0[2], sf0), hmul2h(e2[2], sf1), hmul2h(e0[3], sf0), hmul2h(e2[3], sf1)};
            const uint32_t A2[4] = {hmul2h(e1[0], sf0), hmul2h(e3[0], sf1), hmul2h(e1[1], sf0), hmul2h(e3[1], sf1)};
            const uint32_t A3[4] = {hmul2h(e1[2], sf0), hmul2h(e3[2], sf1), hmul2h(e1[3], sf0), hmul2h(e3[3], sf1)};
#pragma unroll
            for (int q = 0; q < QT; ++q) {
              mma_f16(sa[q][0], A0[0], A0[1], A0[2], A0[3], qa[q][4 * u + 0][0], qa[q][4 * u + 0][1]);
              mma_f16(sa[q][Gm::NCH - 1], A1[0], A1[1], A1[2], A1[3], qa[q][4 * u + 1][0], qa[q][4 * u + 1][1]);
              mma_f16(sa[q][0], A2[0], A2[1], A2[2], A2[3], qa[q][4 * u + 2][0], qa[q][4 * u + 2][1]);
              mma_f16(sa[q][Gm::NCH - 1], A3[0], A3[1], A3[2], A3[3], qa[q][4 * u + 3][0], qa[q][4 * u + 3][1]);
            }
          }
#pragma unroll
          for (int q = 0; q < QT; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) x[q][bi][i] = Gm::NCH == 2 ? sa[q][0][i] + sa[q][Gm::NCH - 1][i] : sa[q][0][i];
        }
      };

      // ---------------- online softmax (raw score units): this lane holds query rows 2c, 2c+1 of tokens r0, r1 of
      // every block; x[bi] = {(r0, row 2c), (r0, row 2c+1), (r1, row 2c), (r1, row 2c+1)}. Leaves P^T as the B
      // operand of the second product in pb.
      auto softmax = [&](const uint32_t st, const int blk, float (&x)[QT][UB][4], uint32_t (&pb)[QT][UB][2]) {
        const int tbase = blk * UT;
        if (blk >= blk_mask) {                        // warp-uniform: only the last unit(s) of a sequence
          // rows past the context hold arbitrary bytes: their scores become -inf below, and their value scales are
          // set to zero here, in shared memory, so that the value product needs no masking code
          if (lane < UT && tbase + lane >= L) {
            const uint32_t a = st + Gm::V_BASE + Gm::SF_BASE + lane * Gm::SF_ROW;
#pragma unroll
            for (int i = 0; i < Gm::SS; i += 8) sts64_zero(a + i);
            fence_proxy_async();                      // the stage's next bulk copy overwrites these bytes
          }
          __syncwarp();
          const float ninf = -__int_as_float(0x7f800000);
#pragma unroll
          for (int q = 0; q < QT; ++q)
#pragma unroll
            for (int bi = 0; bi < UB; ++bi) {
              const int ta = tbase + 16 * bi + r0, tb = tbase + 16 * bi + r1;
              x[q][bi][0] = ta < lim0[q] ? x[q][bi][0] : ninf;
              x[q][bi][1] = ta < lim1[q] ? x[q][bi][1] : ninf;
              x[q][bi][2] = tb < lim0[q] ? x[q][bi][2] : ninf;
              x[q][bi][3] = tb < lim1[q] ? x[q][bi][3] : ninf;
            }
        }
        // the running max moves only when some score exceeds it by more than TAU (then P stays below 2^TAU, inside
        // f16); the cross-lane maximum is needed only in that case
        float bm0[QT], bm1[QT];
        bool over = false;
#pragma unroll
        for (int q = 0; q < QT; ++q) {
          bm0[q] = fmaxf(x[q][0][0], x[q][0][2]);
          bm1[q] = fmaxf(x[q][0][1], x[q][0][3]);
#pragma unroll
          for (int bi = 1; bi < UB; ++bi) {
            bm0[q] = fmaxf(bm0[q], fmaxf(x[q][bi][0], x[q][bi][2]));
            bm1[q] = fmaxf(bm1[q], fmaxf(x[q][bi][1], x[q][bi][3]));
          }
          over |= (bm0[q] > thr0[q]) | (bm1[q] > thr1[q]);
        }
        if (__any_sync(0xffffffffu, over)) {
#pragma unroll
          for (int q = 0; q < QT; ++q) {
#pragma unroll
            for (int of = 4; of < 32; of <<= 1) {
              bm0[q] = fmaxf(bm0[q], __shfl_xor_sync(0xffffffffu, bm0[q], of));
              bm1[q] = fmaxf(bm1[q], __shfl_xor_sync(0xffffffffu, bm1[q], of));
            }
            const float n0 = fmaxf(m0[q], fmaxf(bm0[q], NEG_BIG)), n1 = fmaxf(m1[q], fmaxf(bm1[q], NEG_BIG));
            const float al0 = fast_exp2((m0[q] - n0) * sc), al1 = fast_exp2((m1[q] - n1) * sc);
            m0[q] = n0; m1[q] = n1;
            mneg0[q] = -n0 * sc; mneg1[q] = -n1 * sc;
            thr0[q] = n0 + tau_raw; thr1[q] = n1 + tau_raw;
            l0[q] *= al0; l1[q] *= al1;
#pragma unroll
            for (int j = 0; j < Gm::KS; ++j) {
              o[q][j][0] *= al0; o[q][j][1] *= al1; o[q][j][2] *= al0; o[q][j][3] *= al1;
            }
          }
        }
#pragma unroll
        for (int q = 0; q < QT; ++q)
#pragma unroll
          for (int bi = 0; bi < UB; ++bi) {
            const float p00 = fast_exp2(fmaf(x[q][bi][0], sc, mneg0[q])), p01 = fast_exp2(fmaf(x[q][bi][1], sc, mneg1[q])),
                        p10 = fast_exp2(fmaf(x[q][bi][2], sc, mneg0[q])), p11 = fast_exp2(fmaf(x[q][bi][3], sc, mneg1[q]));
            l0[q] += p00 + p10;
            l1[q] += p01 + p11;
            // transpose the two 8x8 (token, row) tiles
            pb[q][bi][0] = movmatrix_trans(pack_f16x2(p00, p01));
            pb[q][bi][1] = movmatrix_trans(pack_f16x2(p10, p11));
          }
      };

      // ---------------- O^T += V^T P^T : rows = channels of block g (+8), columns = query rows
      auto v_phase = [&](const uint32_t st, const uint32_t (&pb)[QT][UB][2]) {
        const uint32_t vd_ = st + voff_d, vs_ = st + voff_s;
#pragma unroll
        for (int bi = 0; bi < UB; ++bi) {
#pragma unroll
          for (int hf = 0; hf < Gm::NH; ++hf) {
            const int dv = bi * 16 * Gm::ROW + 64 * hf, sv = bi * 16 * Gm::SF_ROW + 8 * hf;
            const uint2 v00 = lds64(vd_ + dv);
            const uint2 v01 = lds64(vd_ + dv + VR01 * Gm::ROW);
            const uint2 v10 = lds64(vd_ + dv + VR10 * Gm::ROW);
            const uint2 v11 = lds64(vd_ + dv + VR11 * Gm::ROW);
            const uint32_t f00 = lds8(vs_ + sv), f01 = lds8(vs_ + sv + VR01 * Gm::SF_ROW);
            const uint32_t f10 = lds8(vs_ + sv + VR10 * Gm::SF_ROW), f11 = lds8(vs_ + sv + VR11 * Gm::SF_ROW);
            const __half2 sa = u32_as_h2(e4m3x2_to_f16x2(f00 | (f01 << 8))),
                          sb = u32_as_h2(e4m3x2_to_f16x2(f10 | (f11 << 8)));
            const uint32_t M = 0x0f0f0f0fu;
#pragma unroll
            for (int wv = 0; wv < 2; ++wv) {
              const uint32_t a0 = wv ? v00.y : v00.x, a1 = wv ? v01.y : v01.x, b0_ = wv ? v10.y : v10.x,
                             b1_ = wv ? v11.y : v11.x;
              // bytes of (token pair, channel): low nibble = first token of the pair, high nibble = second
              const uint32_t xe = (a0 & M) | ((a1 * 16u) & ~M), xo = ((a0 >> 4) & M) | (a1 & ~M);
              const uint32_t ye = (b0_ & M) | ((b1_ * 16u) & ~M), yo = ((b0_ >> 4) & M) | (b1_ & ~M);
              uint32_t ae[4], ao[4], be[4], bo[4];   // [channel pair] -> f16x2 over (first, second) token
              e2m1x8_to_f16x2(xe, ae);
              e2m1x8_to_f16x2(xo, ao);
              e2m1x8_to_f16x2(ye, be);
              e2m1x8_to_f16x2(yo, bo);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t a0_ = hmul2h(ae[i], sa), a1_ = hmul2h(ao[i], sa), a2_ = hmul2h(be[i], sb), a3_ = hmul2h(bo[i], sb);
#pragma unroll
                for (int q = 0; q < QT; ++q) mma_f16(o[q][8 * hf + 4 * wv + i], a0_, a1_, a2_, a3_, pb[q][bi][0], pb[q][bi][1]);
              }
            }
          }
        }
      };

      uint32_t bar, st;
      if (L == 0) {                                   // the single unit of an empty context carries nothing
        for (int blk = blk_first; blk < blk_end; blk += TG) {
          if (!wait_stage(bar, st)) break;
          if ((int)f_n < n_my) fetch_one(bar, st);
        }
      } else if (wait_stage(bar, st)) {
        for (int blk = blk_first;;) {
          float x[QT][UB][4];
          uint32_t pb[QT][UB][2];
          k_phase(st, x);
          softmax(st, blk, x, pb);
          v_phase(st, pb);
          __syncwarp();
          if ((int)f_n < n_my) fetch_one(bar, st);
          blk += TG;
          if (blk >= blk_end || !wait_stage(bar, st)) break;
        }
      }
    }

    // ---------------- merge the TG warps' states of this piece and write it out
    {
      float sc = p.scale_log2 * __ldg(p.gk + h);
      sc = fmaxf(fabsf(sc), 1e-30f);
      float* ob = obuf + (size_t)w * RP * Sm::OROW;
#pragma unroll
      for (int q = 0; q < QT; ++q) {
#pragma unroll
        for (int of = 4; of < 32; of <<= 1) {
          l0[q] += __shfl_xor_sync(0xffffffffu, l0[q], of);
          l1[q] += __shfl_xor_sync(0xffffffffu, l1[q], of);
        }
        const int ra = 8 * q + 2 * c;              // this lane's rows of the tile: ra, ra + 1
        if (g == 0) {
          mbuf[w * RP + ra] = m0[q] * sc;          // log2 units from here on
          mbuf[w * RP + ra + 1] = m1[q] * sc;
          lbuf[w * RP + ra] = l0[q];
          lbuf[w * RP + ra + 1] = l1[q];
        }
#pragma unroll
        for (int hf = 0; hf < Gm::NH; ++hf)
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int ch = 16 * (g + 8 * hf) + 2 * jj;
            const float* a = o[q][8 * hf + jj];
            *reinterpret_cast<float2*>(ob + ra * Sm::OROW + ch) = make_float2(a[0], a[2]);
            *reinterpret_cast<float2*>(ob + (ra + 1) * Sm::OROW + ch) = make_float2(a[1], a[3]);
          }
      }
      __syncthreads();
      const float gvh = __ldg(p.gv + h);
      const int slot_id = part * 2 + (piece_idx == 0 ? 0 : 1);
      // a thread stays on one query row (4 rows x 32 threads, or 8 x 16), so the warps' weights are worked out once
      const int tpr = R <= RP / 2 ? NTHREADS / (RP / 2) : NTHREADS / RP;   // threads per row
      const int row = tid / tpr;
      if (row < R) {
        float mx = -3.0e38f;
#pragma unroll
        for (int ww = 0; ww < TG; ++ww) mx = fmaxf(mx, mbuf[ww * RP + row]);
        float den = 0.0f, wgt[TG];
#pragma unroll
        for (int ww = 0; ww < TG; ++ww) {
          wgt[ww] = fast_exp2(mbuf[ww * RP + row] - mx);
          den += lbuf[ww * RP + row] * wgt[ww];
        }
        const float inv = den > 0.0f ? gvh / den : 0.0f;
        const float* orow = obuf + (size_t)row * Sm::OROW;
        float* dst_p = nullptr;
        __nv_bfloat16* dst_o = nullptr;
        if (complete) {
          const int t = (p.row0 + row) / G, gq = p.row0 + row - t * G;
          dst_o = p.out + ((long long)(q0 + t) * (KVH * G) + h * G + gq) * D;
        } else {
          dst_p = opart_ws + ((size_t)slot_id * RP + row) * D;
          if (tid == row * tpr) lse_ws[slot_id * RP + row] = den > 0.0f ? log2f(den) + mx : -__int_as_float(0x7f800000);
        }
        for (int ch = (tid - row * tpr) * 2; ch < D; ch += 2 * tpr) {
          float n0 = 0.0f, n1 = 0.0f;
#pragma unroll
          for (int ww = 0; ww < TG; ++ww) {
            const float2 v = *reinterpret_cast<const float2*>(orow + (size_t)ww * RP * Sm::OROW + ch);
            n0 += v.x * wgt[ww];
            n1 += v.y * wgt[ww];
          }
          if (complete)
            *reinterpret_cast<__nv_bfloat162*>(dst_o + ch) = __floats2bfloat162_rn(n0 * inv * p.v_scale, n1 * inv * p.v_scale);
          else
            *reinterpret_cast<float2*>(dst_p + ch) = make_float2(n0 * inv, n1 * inv);
        }
      }
      if (draw_now) __threadfence();                 // this thread's part of the partial, visible device-wide
      __syncthreads();
      if (draw_now) {
        if (tid == 0) split_win[0] = draw_ticket(split[0]);
        drawn |= 1u;
      }
    }
    pos = piece_end;
    ++piece_idx;
  }

  // ---- ticket round of the split sequences this partition holds a piece of: the CTA that finishes a sequence's last
  // outstanding piece merges all of them (log-sum-exp weights, partition order) and writes the output rows. The
  // partial was written by many threads: each makes its own writes visible device-wide, the CTA barrier orders them
  // before the thread that draws the ticket, and the merging CTA reads the partials past the L1 (ld.global.cg).
  if (pending) {
    const unsigned late = pending & ~drawn;          // CTA-uniform: the pieces that ended with the partition
    if (late) __threadfence();
    __syncthreads();
    if (tid < 2 && (late >> tid & 1u)) split_win[tid] = draw_ticket(split[tid]);
    if (late) __syncthreads();
#pragma unroll 1
    for (int i = 0; i < 2; ++i) {
      if (!split_win[i]) continue;
      __threadfence();
      const SplitSeq sq = split[i];
      const long long seq_u0 = sq.seq0 + PC;
      const int first = (int)(seq_u0 / per), last = (int)((seq_u0 + sq.U - 1) / per);
      const int first_slot = (long long)first * per >= sq.seq0 ? 0 : 1;
      for (int rb = 0; rb < sq.R; rb += RPAD)
        merge_split<D, RP, NTHREADS, RPAD>(lse_ws, opart_ws, first, last, first_slot, sq.R, p.row0, p.G,
                                          p.out + ((long long)sq.q0 * (KVH * p.G) + sq.h * p.G) * D,
                                          (long long)KVH * p.G * D, p.v_scale, rb);
    }
  }

  // a warp that gave up may still have copies in flight: wait for them (bounded) before the CTA's shared memory is
  // released
  if (dead) {
    while (c_n < f_n) {
      (void)mbar_wait_bounded_u32(c_bar, c_par);
      advance();
    }
  }
}

// ----------------------------------------------------------------------------------------------------- host side
int record_cuda(cudaError_t e);

struct DeviceInfo {
  int sms = 0;
  int ctas_per_sm[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};    // [D == 256][LAYOUT]
  int ctas_two_tiles = 0;                            // decode_kernel<128, 0, 2>: sixteen query rows per pass
  std::atomic<bool> ready{false};                    // set (release) after the fields above, under g_setup_mutex
};
static DeviceInfo g_dev[64];
static std::mutex g_setup_mutex;                     // serialises the once-per-device set-up of concurrent host threads
static std::atomic<int> g_early_metadata{0};

template <int D, int LAYOUT, int QT = 1>
static cudaError_t setup_variant(int& ctas) {
  auto k = decode_kernel<D, LAYOUT, QT>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D, LAYOUT, QT>::TOTAL);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, k, NTHREADS, Smem<D, LAYOUT, QT>::TOTAL);
}

static int device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda(e);
  if (dev < 0 || dev >= 64) return HKV_ERR_RANGE;
  DeviceInfo& di = g_dev[dev];
  if (!di.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!di.ready.load(std::memory_order_relaxed)) {
      e = cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<128, 0>(di.ctas_per_sm[0][0])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<128, 1>(di.ctas_per_sm[0][1])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<256, 0>(di.ctas_per_sm[1][0])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<256, 1>(di.ctas_per_sm[1][1])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<256, 2>(di.ctas_per_sm[1][2])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<128, 3>(di.ctas_per_sm[0][3])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<256, 3>(di.ctas_per_sm[1][3])) != cudaSuccess) return record_cuda(e);
      if ((e = setup_variant<128, 0, 2>(di.ctas_two_tiles)) != cudaSuccess) return record_cuda(e);
      di.ready.store(true, std::memory_order_release);
    }
  }
  *out = &di;
  return HKV_OK;
}

// upper bound of partitions for any layout of this head_dim on this device
static int max_parts(const DeviceInfo& di, int D) {
  const int i = D == 256;
  return min(kMaxParts, di.sms * max(max(1, di.ctas_per_sm[i][3]),
                                     max(di.ctas_per_sm[i][0], max(di.ctas_per_sm[i][1], di.ctas_per_sm[i][2]))));
}

}  // namespace hkv

extern "C" size_t hkv_decode_workspace_bytes(int B, int KVH, int G, int D, int qlmax) {
  using namespace hkv;
  if (B < 1 || B > kMaxBatch || KVH < 1 || G < 1 || qlmax < 1 || G * qlmax > kMaxRows || (D != 128 && D != 256)) return 0;
  DeviceInfo* di;
  if (device_info(&di) != HKV_OK) return 0;
  size_t need = WorkspaceLayout(max_parts(*di, D), RPAD, D).total;
  if (D == 128 && G * qlmax > RPAD)                 // head-major pages may take the two-tile kernel (16 rows per pass)
    need = std::max(need, WorkspaceLayout(std::min(kMaxParts, di->sms * std::max(1, di->ctas_two_tiles)), 2 * RPAD, D).total);
  return need;
}

static int decode_impl(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                       const int64_t strides[6], int PS, const int32_t* block_tables, int MP, const int32_t* seq_lens,
                       const int32_t* query_start_loc, int B, int KVH, int G, int D, int qlmax, float sm_scale,
                       float v_scale, const float* gk, const float* gv, void* workspace, size_t workspace_bytes,
                       int splits, const float* signs, int k8, void* out, void* stream) {
  using namespace hkv;
  if (B < 0 || MP < 0) return HKV_ERR_RANGE;
  if (B == 0) return HKV_OK;
  if (!q || !kd || !ksf || !vd || !vsf || !strides || !block_tables || !seq_lens || !query_start_loc || !gk || !gv ||
      !workspace || !out)
    return HKV_ERR_NULL;
  if (D != 128 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (KVH < 1 || G < 1 || qlmax < 1 || G * qlmax > kMaxRows) return HKV_ERR_UNSUPPORTED;
  if (PS < 16 || (PS & (PS - 1)) != 0) return HKV_ERR_UNSUPPORTED;   // 16, 32, 64, ..
  if (B > kMaxBatch) return HKV_ERR_RANGE;
  if (splits < 0) return HKV_ERR_RANGE;
  if (splits > 64) return HKV_ERR_SPLITS;
  const int SD = D / 2, SS = D / 16, SLOT = SD + SS;
  const int64_t dsp = strides[0], dst = strides[1], dsh = strides[2], ssp = strides[3], sst = strides[4],
                ssh = strides[5];
  int layout;
  if (k8) {
    // K8V4 slot: [D key bytes | D/2 value codes | D/16 value scales] per token, heads outermost (head_dim 256 only)
    const int SLOT8 = D + SD + SS;
    if (D != 256 || signs) return HKV_ERR_UNSUPPORTED;
    if (dst != SLOT8 || sst != SLOT8 || dsp != ssp || dsh != ssh || (const uint8_t*)vd != (const uint8_t*)kd + D ||
        (const uint8_t*)vsf != (const uint8_t*)vd + SD)
      return HKV_ERR_UNSUPPORTED;
    layout = 2;
  } else if (dst == SLOT && sst == SLOT && dsp == ssp && dsh == ssh && (const uint8_t*)ksf == (const uint8_t*)kd + SD &&
      (const uint8_t*)vsf == (const uint8_t*)vd + SD)
    layout = 0;
  else if (dst == SD && sst == SS)
    layout = 1;
  else if (sst == dst && dsp == ssp && dsh == ssh && (const uint8_t*)ksf == (const uint8_t*)kd + SD &&
           (const uint8_t*)vsf == (const uint8_t*)vd + SD)
    layout = 3;   // rows of [codes | scales] at any position / head strides, e.g. positions outermost inside a page (NHD)
  else
    return HKV_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)out) & 15) return HKV_ERR_ALIGN;
  if (layout == 3) {
    // every token row is copied on its own in 8-byte (head_dim 128) or 16-byte (256) pieces
    const int a = D == 128 ? 7 : 15;
    if (((uintptr_t)kd | (uintptr_t)vd | (uintptr_t)dsp | (uintptr_t)dst | (uintptr_t)dsh) & a) return HKV_ERR_ALIGN;
    if (dst < 0 || dst >= (1ll << 31)) return HKV_ERR_RANGE;
  } else {
    if (((uintptr_t)kd | (uintptr_t)vd) & 15) return HKV_ERR_ALIGN;
    if ((dsp | dsh) & 15) return HKV_ERR_ALIGN;
  }
  if (dsp < 0 || ssp < 0 || dsp >= (1ll << 31) || ssp >= (1ll << 31)) return HKV_ERR_RANGE;   // a page is far below 2 GB
  if (layout == 1 && ((((uintptr_t)ksf | (uintptr_t)vsf) & 15) || ((ssp | ssh) & 15))) return HKV_ERR_ALIGN;
  if ((uintptr_t)workspace & 255) return HKV_ERR_ALIGN;
  DeviceInfo* di;
  int rc = device_info(&di);
  if (rc != HKV_OK) return rc;
  // head_dim 128, head-major slot pages, more than 8 query rows per kv head: the two-tile kernel serves 16 rows per pass
  const bool two = D == 128 && layout == 0 && G * qlmax > RPAD && di->ctas_two_tiles > 0;
  const int rows_per_pass = two ? 2 * RPAD : RPAD;
  const int cps = two ? di->ctas_two_tiles : di->ctas_per_sm[D == 256][layout];
  if (cps < 1) return HKV_ERR_UNSUPPORTED;
  (void)max_parts;
  long long n_parts = std::min<long long>((long long)di->sms * cps, kMaxParts);
  if (splits > 0) n_parts = std::min<long long>(n_parts, (long long)B * KVH * splits);
  if (n_parts < 1) n_parts = 1;
  if (workspace_bytes < WorkspaceLayout((int)n_parts, rows_per_pass, D).total) return HKV_ERR_WORKSPACE;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q;
  p.kd = (const uint8_t*)kd; p.ksf = (const uint8_t*)ksf; p.vd = (const uint8_t*)vd; p.vsf = (const uint8_t*)vsf;
  p.dsp = (unsigned)dsp; p.dsh = dsh; p.ssp = (unsigned)ssp; p.ssh = ssh; p.dst = (unsigned)dst;
  p.bt = block_tables; p.seq_lens = seq_lens; p.qsl = query_start_loc;
  p.gk = gk; p.gv = gv;
  p.ws = (uint8_t*)workspace;
  p.out = (__nv_bfloat16*)out;
  p.MP = MP; p.B = B; p.KVH = KVH; p.G = G; p.qlmax = qlmax; p.PS = PS;
  p.early_meta = g_early_metadata.load(std::memory_order_relaxed);
  p.max_len = (int)std::min<long long>((long long)MP * PS, 0x7fffffffll);
  if (signs && ((uintptr_t)signs & 15)) return HKV_ERR_ALIGN;
  p.signs = signs;
  p.rot_scale = (float)(1.0 / sqrt((double)D));
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.v_scale = v_scale;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)n_parts;
  void (*k)(const DecodeParams) =
      two ? decode_kernel<128, 0, 2> :
      D == 128 ? (layout == 0 ? decode_kernel<128, 0> : layout == 1 ? decode_kernel<128, 1> : decode_kernel<128, 3>)
               : (layout == 0 ? decode_kernel<256, 0> : layout == 1 ? decode_kernel<256, 1>
                  : layout == 2 ? decode_kernel<256, 2> : decode_kernel<256, 3>);
  const size_t smem_bytes = two ? (size_t)Smem<128, 0, 2>::TOTAL : D == 128 ? (size_t)Smem<128, 0>::TOTAL
                                     : layout == 2 ? (size_t)Smem<256, 2>::TOTAL : (size_t)Smem<256, 0>::TOTAL;
  static_assert(Smem<128, 0>::TOTAL == Smem<128, 1>::TOTAL && Smem<256, 0>::TOTAL == Smem<256, 1>::TOTAL &&
                Smem<128, 0>::TOTAL == Smem<128, 3>::TOTAL && Smem<256, 0>::TOTAL == Smem<256, 3>::TOTAL,
                "layouts share a size");
  // More query rows per kv head than a pass serves (large groups, several draft tokens) take several passes: every
  // pass is one launch over the cache (split sequences are merged inside it).
  for (int row0 = 0; row0 < G * qlmax; row0 += rows_per_pass) {
    p.row0 = row0;
    rc = record_cuda(launch_pdl(k, dim3(grid), dim3(NTHREADS), smem_bytes, st, p));
    if (rc != HKV_OK) return rc;
  }
  return HKV_OK;
}

extern "C" int hkv_decode(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                          const int64_t strides[6], int PS, const int32_t* block_tables, int MP,
                          const int32_t* seq_lens, const int32_t* query_start_loc, int B, int KVH, int G, int D,
                          int qlmax, float sm_scale, float v_scale, const float* gk, const float* gv, void* workspace,
                          size_t workspace_bytes, int splits, void* out, void* stream) {
  return decode_impl(q, kd, ksf, vd, vsf, strides, PS, block_tables, MP, seq_lens, query_start_loc, B, KVH, G, D, qlmax,
                     sm_scale, v_scale, gk, gv, workspace, workspace_bytes, splits, nullptr, 0, out, stream);
}

extern "C" int hkv_decode_rot(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                              const int64_t strides[6], int PS, const int32_t* block_tables, int MP,
                              const int32_t* seq_lens, const int32_t* query_start_loc, int B, int KVH, int G, int D,
                              int qlmax, float sm_scale, float v_scale, const float* gk, const float* gv,
                              void* workspace, size_t workspace_bytes, int splits, const float* signs, void* out,
                              void* stream) {
  if (B > 0 && !signs) return HKV_ERR_NULL;
  return decode_impl(q, kd, ksf, vd, vsf, strides, PS, block_tables, MP, seq_lens, query_start_loc, B, KVH, G, D, qlmax,
                     sm_scale, v_scale, gk, gv, workspace, workspace_bytes, splits, signs, 0, out, stream);
}

extern "C" int hkv_decode_k8(const void* q, const void* kd, const void* vd, const void* vsf, const int64_t strides[6],
                             int PS, const int32_t* block_tables, int MP, const int32_t* seq_lens,
                             const int32_t* query_start_loc, int B, int KVH, int G, int D, int qlmax, float sm_scale,
                             float v_scale, const float* gk, const float* gv, void* workspace, size_t workspace_bytes,
                             int splits, void* out, void* stream) {
  return decode_impl(q, kd, kd, vd, vsf, strides, PS, block_tables, MP, seq_lens, query_start_loc, B, KVH, G, D, qlmax,
                     sm_scale, v_scale, gk, gv, workspace, workspace_bytes, splits, nullptr, 1, out, stream);
}

extern "C" int hkv_combine(const void* workspace, size_t workspace_bytes, const int32_t* query_start_loc, int B,
                           int KVH, int G, int D, int qlmax, float v_scale, void* out, void* stream) {
  using namespace hkv;
  // The log-sum-exp combine runs inside the decode launch (merge_split above): when hkv_decode's kernels have finished,
  // `out` is complete. This entry point is kept so that callers written against the three-call sequence of the
  // reference (write, decode, combine) keep working; it checks its arguments like before and launches nothing.
  (void)v_scale; (void)stream;
  if (B < 0) return HKV_ERR_RANGE;
  if (B == 0) return HKV_OK;
  if (!workspace || !query_start_loc || !out) return HKV_ERR_NULL;
  if (D != 128 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (KVH < 1 || G < 1 || qlmax < 1 || G * qlmax > kMaxRows) return HKV_ERR_UNSUPPORTED;
  if (((uintptr_t)workspace & 255) || ((uintptr_t)out & 15)) return HKV_ERR_ALIGN;
  if (workspace_bytes < WorkspaceLayout(1, RPAD, D).total) return HKV_ERR_WORKSPACE;
  return HKV_OK;
}

extern "C" int hkv_set_option(int option, int value) {
  using namespace hkv;
  if (option != HKV_OPT_EARLY_METADATA) return HKV_ERR_UNSUPPORTED;
  if (value != 0 && value != 1) return HKV_ERR_RANGE;
  g_early_metadata.store(value, std::memory_order_relaxed);
  return HKV_OK;
}

namespace hkv {
// One warp waits, with the decode kernel's bounded wait but a caller-given limit, on a barrier that nothing completes,
// and reports the way the decode kernel does. It never hangs: the wait gives up after `cycles` SM clocks.
__global__ void selftest_wait_kernel(uint8_t* ws, long long cycles) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  fence_barrier_init();
  __syncthreads();
  if (!mbar_wait_bounded_u32(smem_u32(&bar), 0, cycles)) {
    if (threadIdx.x == 0) atomicExch(&reinterpret_cast<Header*>(ws)->status, HKV_ERR_DEVICE_WAIT);
  }
}
}  // namespace hkv

extern "C" int hkv_selftest_wait_timeout(void* workspace, int64_t cycles, void* stream) {
  using namespace hkv;
  if (!workspace) return HKV_ERR_NULL;
  if (cycles < 0 || cycles > (1ll << 31)) return HKV_ERR_RANGE;     // at most about a second
  selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint8_t*)workspace, cycles);
  return record_cuda(cudaGetLastError());
}

extern "C" int hkv_workspace_status(void* workspace, int* status, void* stream) {
  using namespace hkv;
  if (!workspace || !status) return HKV_ERR_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return record_cuda(e);
  if ((e = cudaMemsetAsync(workspace, 0, sizeof(int), st)) != cudaSuccess) return record_cuda(e);
  return record_cuda(cudaStreamSynchronize(st));
}

// ------------------------------------------------------------------------------------------ decode without a workspace
namespace hkv {
// Scratch of the workspace-free entry point: partition descriptors, log2-sum-exp values and fp32 partials of one
// decode call. 5 MiB hold 444 partitions at head_dim 128 (3.7 MB) and 296 at head_dim 256 (4.9 MB), which is what a
// 148-SM device uses. Every GPU that loads this library carries the array until the process exits.
constexpr size_t kNoAllocScratchBytes = 5u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// device address of the array per device ordinal; the symbol's name above is only a host-side handle
static std::atomic<void*> g_noalloc_ptr[64] = {};
}  // namespace hkv

extern "C" int hkv_decode_noalloc(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                                  const int64_t strides[6], int PS, const int32_t* block_tables, int MP,
                                  const int32_t* seq_lens, const int32_t* query_start_loc, int B, int KVH, int G, int D,
                                  int qlmax, float sm_scale, float v_scale, const float* gk, const float* gv, int splits,
                                  void* out, void* stream) {
  using namespace hkv;
  if (B < 0 || MP < 0 || splits < 0) return HKV_ERR_RANGE;
  if (B == 0) return HKV_OK;
  if (D != 128 && D != 256) return HKV_ERR_UNSUPPORTED;
  if (KVH < 1 || G < 1 || qlmax < 1 || G * qlmax > kMaxRows) return HKV_ERR_UNSUPPORTED;
  if (splits > 64) return HKV_ERR_SPLITS;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda(e);
  if (dev < 0 || dev >= 64) return HKV_ERR_RANGE;
  void* ws = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (ws == nullptr) {                              // set-up, once per device, with that device current
    e = cudaGetSymbolAddress(&ws, g_noalloc_scratch);
    if (e != cudaSuccess) return record_cuda(e);
    if (ws == nullptr) return HKV_ERR_CUDA;
    g_noalloc_ptr[dev].store(ws, std::memory_order_release);   // (two threads racing here store the same address)
  }
  DeviceInfo* di;
  const int rc0 = device_info(&di);
  if (rc0 != HKV_OK) return rc0;
  // the scratch a call needs grows with the number of stream partitions, which is bounded by the device's resident
  // CTAs and by B * KVH * splits
  long long n_parts = std::min<long long>(
      (long long)max_parts(*di, D), kMaxParts);
  if (splits > 0) n_parts = std::min<long long>(n_parts, (long long)B * KVH * splits);
  if (n_parts < 1) n_parts = 1;
  if (WorkspaceLayout((int)n_parts, RPAD, D).total > kNoAllocScratchBytes) return HKV_ERR_NOALLOC_LIMIT;
  const int rc = hkv_decode(q, kd, ksf, vd, vsf, strides, PS, block_tables, MP, seq_lens, query_start_loc, B, KVH, G, D,
                            qlmax, sm_scale, v_scale, gk, gv, ws, kNoAllocScratchBytes, splits, out, stream);
  return rc;
}

extern "C" int hkv_decode_noalloc_status(int* status, void* stream) {
  using namespace hkv;
  if (!status) return HKV_ERR_NULL;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda(e);
  if (dev < 0 || dev >= 64) return HKV_ERR_RANGE;
  void* ws = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (ws == nullptr) {                              // no hkv_decode_noalloc call on this device yet: nothing to report
    *status = HKV_OK;
    return HKV_OK;
  }
  return hkv_workspace_status(ws, status, stream);
}
