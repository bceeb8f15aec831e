/*
 * hkv: NVFP4 paged KV-cache kernels for NVIDIA B200 (sm_100a) behind a plain C ABI.
 *
 * Cache format (per token, kv head and side K or V; head_dim D in {128, 256}):
 *   data : D/2 bytes of E2M1 codes, element 2j in the low nibble of byte j
 *   sf   : D/16 bytes, one E4M3 scale per 16 consecutive elements
 *   g    : one fp32 global scale per (kv head, side), passed by the caller (gk, gv)
 *   value = e2m1(code) * e4m3(sf) * g
 * The four parts of a cache (K data, K scales, V data, V scales) are described the way the reference's kernels take
 * them: a base pointer per part plus byte strides of a [page, position, head, byte] view,
 *   strides = {data page, data position, data head, scale page, scale position, scale head}
 * (reference: nvidia-sm120/horizon_kvfp4/kernels/kv_fp4_serving.py:873-886 `flat_views`, :37 `Strides`).
 *
 * Every function returns HKV_OK or a negative error code, launches on the given CUDA stream, never allocates, never
 * synchronises and never reads device data on the host, so a sequence of calls can be captured in a CUDA graph.
 * Host-detectable misuse (null or misaligned pointers, unsupported head_dim / group size / page size, a workspace that
 * is too small) is rejected before anything is launched.
 * Host threads: the once-per-device set-up that the first decode call on a device performs is serialised internally,
 * so several host threads may make their first calls at the same time.
 */
#ifndef HKV_H_
#define HKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HKV_OK 0
#define HKV_ERR_NULL (-1)         /* a required pointer is null */
#define HKV_ERR_ALIGN (-2)        /* a pointer or stride misses the alignment the kernels need */
#define HKV_ERR_UNSUPPORTED (-3)  /* head_dim, group size (G * qlmax > 64), page size or layout outside the supported set */
#define HKV_ERR_SPLITS (-4)       /* more than 64 splits requested */
#define HKV_ERR_WORKSPACE (-5)    /* workspace too small */
#define HKV_ERR_RANGE (-6)        /* a size is negative or too large */
#define HKV_ERR_CUDA (-7)         /* a CUDA runtime call failed; hkv_last_cuda_error() has the code */
#define HKV_ERR_DEVICE_WAIT (-8)  /* a bounded wait inside a kernel ran out (read back by hkv_workspace_status) */
#define HKV_ERR_NOALLOC_LIMIT (-9) /* hkv_decode_noalloc: the call needs more than the built-in scratch */

/* library version (major * 10000 + minor * 100 + patch) and a text for an error code */
int hkv_version(void);
const char* hkv_error_string(int code);
int hkv_last_cuda_error(void);

/*
 * Quantize-on-write: bf16 K / V rows -> E2M1 codes + E4M3 block scales, scattered to slot = page * PS + position.
 * Replaces `write` / `hz4::write_task` (kv_fp4_serving.py:994-1005, :618-700) and is bit-exact to `write_reference`
 * (kv_fp4_ref.py:233-245) without the optional key rotation.
 *   key, val : bf16, logical (n_tokens >= n_slots, KVH, D); element strides ks0/vs0 (token) and ks1/vs1 (head), last
 *              dimension contiguous and 16-byte aligned rows
 *   slots    : int64[n_slots]; a negative slot skips the token
 *   gk, gv   : fp32[KVH] global scales
 *   search   : 1 = choose the block scale among 4 candidates by squared error (the reference's default), 0 = plain
 */
int hkv_write(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1, void* kd,
              void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS, const int64_t* slots, int64_t n_slots,
              const float* gk, const float* gv, int KVH, int D, int search, void* stream);

/*
 * Workspace for hkv_decode on the current device: bytes needed for a batch of up to B requests.
 * The size depends on the device (number of SMs) and on (B, KVH, G, D, qlmax) only, never on context lengths, so one
 * allocation made outside graph capture serves every step. Replaces the sizing loop at backend.py:263-277.
 * Returns 0 for unsupported arguments.
 * The workspace must be ZERO-FILLED once before its first use (cudaMemsetAsync): it holds the per-sequence ticket
 * counters of the in-kernel combine, which every launch leaves at zero again. After a launch that reported
 * HKV_ERR_DEVICE_WAIT the counters are undefined: zero-fill the workspace again before reusing it.
 */
size_t hkv_decode_workspace_bytes(int B, int KVH, int G, int D, int qlmax);

/*
 * Paged split-K flash-decoding over the FP4 cache. Replaces `decode_ragged` / `hz4::attn_task_rg`
 * (kv_fp4_serving.py:894-915, :99-511):
 *   out[qsl[b] + t, h*G + g, :] = softmax_j(q . k_j * sm_scale * gk[h]) @ v_j * gv[h] * v_scale,  j < L_b - ql_b + t + 1
 * The concatenated (request, kv head) token streams are cut into equal partitions, one per resident CTA; a sequence
 * that lies inside one partition is written to `out` directly, the others leave normalised fp32 partials and
 * log2-sum-exp values in the workspace, and the CTA that finishes a sequence's last outstanding piece merges them in
 * partition order inside the same launch (the reference's `hz4::combine_rg`, kv_fp4_serving.py:518-558, as a second
 * launch): `out` is complete when the call's kernels have finished, and the result does not depend on which CTA
 * merged. `splits` (1..64, or 0 = automatic) bounds the number of partitions to B * KVH * splits like the reference's
 * grid (kv_fp4_serving.py:889-891); it depends on the batch size only.
 *   q            : bf16 (n_tokens, KVH*G, D) contiguous
 *   block_tables : int32 (B, MP); seq_lens int32 (B); query_start_loc int32 (B + 1)
 *   requests with 0 or more than qlmax query tokens are skipped and their output rows left untouched
 *   out          : bf16 (>= n_tokens, KVH*G, D) contiguous
 * A pass over the cache serves 8 query rows per kv head, or 16 at head_dim 128 over head-major slot pages (the reference
 * serves up to 32 rows in one launch, backend.py:237). G * qlmax within one pass is one launch. Up to 64 rows are
 * accepted: the call then makes ceil(G * qlmax / rows per pass) launches.
 */
int hkv_decode(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
               const int64_t strides[6], int PS, const int32_t* block_tables, int MP, const int32_t* seq_lens,
               const int32_t* query_start_loc, int B, int KVH, int G, int D, int qlmax, float sm_scale, float v_scale,
               const float* gk, const float* gv, void* workspace, size_t workspace_bytes, int splits, void* out,
               void* stream);

/*
 * Kept for callers written against the reference's three launches (write, decode, combine: `hz4::combine_rg`,
 * kv_fp4_serving.py:518-558, launched at :913-914). The log-sum-exp merge now runs inside hkv_decode's launch, so this
 * call checks its arguments and launches nothing.
 */
int hkv_combine(const void* workspace, size_t workspace_bytes, const int32_t* query_start_loc, int B, int KVH, int G,
                int D, int qlmax, float v_scale, void* out, void* stream);

/*
 * Decode + combine for callers that cannot allocate device memory. This entry point has no counterpart in the
 * reference, whose backend always allocates its workspace with torch.
 *
 * Who needs it: an inference server usually hands nearly all device memory to one pool at start-up, and a component
 * that is loaded afterwards (a plugin, a sidecar runtime written in another language, code that runs while another
 * library is capturing a CUDA graph) finds cudaMalloc either failing for lack of memory or forbidden outright. Such a
 * caller passes the same inputs and the output buffer as for hkv_decode, but no workspace: the scratch is
 * a 5 MiB array built into the library (HKV_NOALLOC_SCRATCH_BYTES), resident on every GPU that loads it.
 *
 * Limits and rules:
 *   - The scratch holds the partials of at most 444 partitions at head_dim 128 or 296 at head_dim 256 (what a 148-SM
 *     GPU uses). A call that would need more returns HKV_ERR_NOALLOC_LIMIT and launches nothing; a smaller `splits`
 *     (partitions <= B * KVH * splits) brings it under the limit.
 *   - The first call on a device looks up the array's device address and configures the kernels. Make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array. Two calls whose kernels can overlap on the GPU (different streams
 *     without an ordering between them) race on it; order them on one stream or with events. Nothing in the array has
 *     to be cleared between calls: every call rewrites the partials it reads and leaves the ticket counters of the
 *     in-kernel combine at zero, which is also how the array starts.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Arguments as for hkv_decode (without workspace, workspace_bytes); `out` is complete when the call's kernels finish.
 */
#define HKV_NOALLOC_SCRATCH_BYTES (5u << 20)
int hkv_decode_noalloc(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                       const int64_t strides[6], int PS, const int32_t* block_tables, int MP, const int32_t* seq_lens,
                       const int32_t* query_start_loc, int B, int KVH, int G, int D, int qlmax, float sm_scale,
                       float v_scale, const float* gk, const float* gv, int splits, void* out, void* stream);

/*
 * Status word of the built-in scratch of hkv_decode_noalloc on the current device (HKV_OK or HKV_ERR_DEVICE_WAIT), read
 * and cleared like hkv_workspace_status does for a caller's workspace; synchronises the stream. No counterpart in the
 * reference.
 */
int hkv_decode_noalloc_status(int* status, void* stream);

/*
 * The same two operations with the reference's optional key rotation (kv_fp4_ref.py:31-35, :55-92): `signs` is a
 * fixed vector of +-1 per channel (fp32[D], 16-byte aligned; the reference's `hadamard_signs`).
 *   hkv_write_rot  quantises k' = FWHT(k * signs) * D^-0.5, computed in fp32 with the reference's butterfly order, from
 *                  the fp32 result (values are not rotated): bit-exact to `write_reference(..., signs=signs)`
 *                  (kv_fp4_ref.py:233-241; `hz4::write_task<.., HAD = 1>` kv_fp4_serving.py:621-641).
 *   hkv_decode_rot rotates every query row the same way inside the kernel, rounded once to bf16 like `rotate_q`
 *                  (kv_fp4_ref.py:90-92; the fused rotation of kv_fp4_serving.py:146-189), so q' . k' = q . k and the
 *                  model's math is unchanged.
 * All other arguments as for hkv_write / hkv_decode.
 */
int hkv_write_rot(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1, void* kd,
                  void* ksf, void* vd, void* vsf, const int64_t strides[6], int PS, const int64_t* slots,
                  int64_t n_slots, const float* gk, const float* gv, int KVH, int D, int search, const float* signs,
                  void* stream);
int hkv_decode_rot(const void* q, const void* kd, const void* ksf, const void* vd, const void* vsf,
                   const int64_t strides[6], int PS, const int32_t* block_tables, int MP, const int32_t* seq_lens,
                   const int32_t* query_start_loc, int B, int KVH, int G, int D, int qlmax, float sm_scale,
                   float v_scale, const float* gk, const float* gv, void* workspace, size_t workspace_bytes,
                   int splits, const float* signs, void* out, void* stream);

/*
 * Exact dequantisation of cached tokens into dense bf16 or fp16 rows (n_tokens, KVH, D), the input of a prefill
 * attention over a cached prefix: value = e2m1(code) * e4m3(block scale), WITHOUT the global scales gk / gv (the
 * product is exact in both output types; the caller folds the global scales into its softmax scale and its output).
 * Replaces `dequant_tokens` / `hz4::dequant_task` (kv_fp4_serving.py:918-925, :577-609) and `dequant_multi` /
 * `hz4::dequant_multi_task` (kv_fp4_serving.py:1008-1016, :700-740).
 *   rows == NULL, cu == NULL : one request. `block_tables` points at ITS block-table row; positions
 *                              [start, start + n_tokens) of its context go to output rows [0, n_tokens).
 *   rows, cu given           : requests rows[r], r < n_rows, with their full contexts packed: output rows
 *                              [cu[r], cu[r + 1]) hold positions 0 .. cu[r + 1] - cu[r] - 1 of request rows[r];
 *                              cu[0] == 0, cu[n_rows] == n_tokens; `block_tables` is the (B, MP) table; `start` unused.
 *   out_k, out_v             : (n_tokens, KVH, D) contiguous, bf16 (out_f16 == 0) or fp16 (out_f16 == 1), 16-byte aligned
 * Any of the cache layouts hkv_write accepts (code rows 8-byte aligned). A scale byte 0x7f / 0xff (never written by
 * hkv_write) gives NaN.
 */
int hkv_dequant(const void* kd, const void* ksf, const void* vd, const void* vsf, const int64_t strides[6], int PS,
                const int32_t* block_tables, int MP, const int32_t* rows, const int32_t* cu, int n_rows, int64_t start,
                int64_t n_tokens, void* out_k, void* out_v, int KVH, int D, int out_f16, void* stream);

/*
 * The three operations on the reference's K8V4 slot (kv_fp4_ref.py:283-321; `HORIZON_KVFP4_K8`), head_dim 256 only:
 * per (token, kv head) 400 bytes = [256 signed E4M3 key bytes | 128 value code bytes | 16 value scale bytes], cache
 * (pages, KVH, PS, 400) with heads outermost. kd / vd / vsf point at the key bytes, value codes and value scales of
 * (page 0, position 0, head 0); strides = {page, position, head} byte strides of kd and vd, then of vsf.
 *   hkv_write_k8   keys e4m3(k / gk[h]) (IEEE division, round to nearest even, saturating at +-448, what vLLM's fp8 cache
 *                  holds), values like hkv_write: byte-exact to `write_reference_k8` (kv_fp4_ref.py:301-311)
 *   hkv_decode_k8  like hkv_decode with key = e4m3 value * gk[h]. The slots of a head's 16
 *                  tokens must be contiguous (dst == 400)
 *   hkv_dequant_k8 like hkv_dequant; keys are the E4M3 values themselves (no gk)
 */
int hkv_write_k8(const void* key, const void* val, int64_t ks0, int64_t ks1, int64_t vs0, int64_t vs1, void* kd, void* vd,
                 void* vsf, const int64_t strides[6], int PS, const int64_t* slots, int64_t n_slots, const float* gk,
                 const float* gv, int KVH, int D, int search, void* stream);
int hkv_decode_k8(const void* q, const void* kd, const void* vd, const void* vsf, const int64_t strides[6], int PS,
                  const int32_t* block_tables, int MP, const int32_t* seq_lens, const int32_t* query_start_loc, int B,
                  int KVH, int G, int D, int qlmax, float sm_scale, float v_scale, const float* gk, const float* gv,
                  void* workspace, size_t workspace_bytes, int splits, void* out, void* stream);
int hkv_dequant_k8(const void* kd, const void* vd, const void* vsf, const int64_t strides[6], int PS,
                   const int32_t* block_tables, int MP, const int32_t* rows, const int32_t* cu, int n_rows, int64_t start,
                   int64_t n_tokens, void* out_k, void* out_v, int KVH, int D, int out_f16, void* stream);

/*
 * Process-wide options. No counterpart in the reference.
 *   HKV_OPT_EARLY_METADATA (0 = off, the default; 1 = on): the caller states that `seq_lens` and `query_start_loc` of
 *     every later hkv_decode / hkv_decode_noalloc call are complete before the kernel that PRECEDES the call on its
 *     stream starts (an inference engine writes them once per step, long before the attention layers run; hkv_write never
 *     writes them). hkv_decode then reads these two arrays while the preceding kernel is still running and waits for
 *     it only afterwards, before it touches the block tables, the cache, the queries or the workspace. With the option
 *     off every input may be produced by the directly preceding kernel.
 * Returns HKV_ERR_UNSUPPORTED for an unknown option and HKV_ERR_RANGE for a value outside its set.
 */
#define HKV_OPT_EARLY_METADATA 1
int hkv_set_option(int option, int value);

/*
 * Self-test of the failure path, no counterpart in the reference: one warp waits on a barrier that nothing will ever
 * complete, with the decode kernel's bounded wait and a limit of `cycles` SM clocks (at most 2^31, about a second), gives
 * up and records HKV_ERR_DEVICE_WAIT in the workspace header, where hkv_workspace_status finds it. The kernel always
 * terminates and the context stays usable; nothing faults.
 */
int hkv_selftest_wait_timeout(void* workspace, int64_t cycles, void* stream);

/*
 * Self-test of the narrow-float conversions the kernels stand on, no counterpart in the reference (whose CPU tests
 * pin the equivalent bit formulas exhaustively: scripts/kernels/kvfp4/test_kvfp4_cpu.py:54-99, :390-434,
 * test_kvfp4_serving_cpu.py:47-110). Writes to `out` (device memory, 8-byte aligned, HKV_SELFTEST_CODEC_BYTES):
 *   uint64 [0]  how many of the 2^31 - 2^23 + 1 non-negative fp32 bit patterns 0 .. +inf get a different E2M1 code from
 *               the hardware conversion the write kernel uses (cvt.rn.satfinite.e2m1x2.f32) than from the reference's
 *               threshold chain (kv_fp4_ref.py:122-130); must be 0
 *   uint64 [1]  the same count over the NaN patterns above +inf
 *   uint64 [2]  how many (value, scale) pairs get a different quotient from the write kernel's three multiply-adds with
 *               the scale's reciprocal than from an IEEE division (any bit where the quotient is >= 0.125, the E2M1
 *               code everywhere); must be 0. Scales: every E4M3 code 1..126 times 64 global scales (few mantissa bits,
 *               full mantissas, n / 2688, mantissas of all ones); values: the bf16 patterns of 17 binades around the
 *               scale, hashed fp32 quotients in [0, 8), the seven rounding boundaries with their neighbours
 *   uint64 [3]  the number of pairs compared (about 6 * 10^7)
 *   uint64 [4]  how many blocks of 16 values get different codes, or a squared error that differs in any bit, from the
 *               write kernel's packed fp32 pair arithmetic than from IEEE divisions, the threshold chain and the
 *               reference's chain of single fp32 multiplies, subtractions and additions in index order
 *               (kv_fp4_ref.py:148-156); must be 0
 *   uint64 [5]  the number of blocks compared (about 2 * 10^6)
 *   uint64 [6], [7]  zero
 *   uint16 [16 * 256]  f16 bits of cvt.rn.f16x2.e2m1x2(code) * cvt.rn.f16x2.e4m3x2(scale byte), index code * 256 + byte:
 *               the dequantised value the decode and dequantisation kernels form
 * A few milliseconds of GPU time; asynchronous on the stream like every other call.
 */
#define HKV_SELFTEST_CODEC_BYTES (64 + 16 * 256 * 2)
int hkv_selftest_codec(void* out, size_t out_bytes, void* stream);

/*
 * Issue-rate probe, no counterpart in the reference: times, with the SM clock counter, unrolled sequences of the
 * instruction kinds the decode and write kernels are made of, `warps_per_subpartition` (1..8) warps per SM sub-partition, one block
 * per SM. Results in `scratch` (device memory, 8-byte aligned, HKV_PROBE_SCRATCH_BYTES): int64 cycles[12][256], entry
 * [mode][sm] = cycles that SM's block took for 2048 repetitions per warp of
 *   mode 0: 8 cvt.rn.f16x2.e2m1x2   1: 8 mul.f16x2   2: 8 fma.f32   3: 8 lop3   4: 4 conversions + 4 multiplies
 *   mode 5: 4 conversions + 4 multiplies + 1 integer add (the decode kernel's dequantise group without its mma)
 *   mode 6: mode 5 + one mma.sync.m16n8k16 (10 instructions per repetition)
 *   mode 7: 8 mul.f32   8: 8 mul.f32x2   9: 8 cvt.rn.satfinite.e2m1x2.f32   10: 8 cvt.f32.f16   11: 8 prmt
 * cycles / (2048 * instructions per repetition * warps_per_subpartition) = cycles per warp instruction and
 * sub-partition. `python -m horizon_kernels_b200.microbench pipes` prints them. Asynchronous on the stream.
 */
#define HKV_PROBE_SCRATCH_BYTES (12 * 256 * 8 + 256 * 1024 * 4)
int hkv_probe_issue_rates(void* scratch, size_t scratch_bytes, int warps_per_subpartition, void* stream);

/*
 * Copies the workspace's device status word to *status (HKV_OK or HKV_ERR_DEVICE_WAIT) and clears it. Synchronises the
 * stream: a debugging aid, not for the hot path.
 */
int hkv_workspace_status(void* workspace, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HKV_H_ */
