/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement (plain C, fp32 IEEE without contraction for the quantiser, fp64 for attention) of the NVFP4
 * KV-cache path of the reference `nvidia-sm120/horizon_kvfp4`. Only the parity tests, the smoke check and the CPU
 * baseline leg of the benchmark may load this library; the CUDA library never links or calls it.
 *
 * Parity status: PINNED. The functions below are checked (tests/test_oracle.py) against golden vectors produced by
 * running the reference's own PyTorch implementation (`nvidia-sm120/horizon_kvfp4/kernels/kv_fp4_ref.py`) and against
 * the known-answer properties of the reference's CPU test script (`nvidia-sm120/scripts/kernels/kvfp4/test_kvfp4_cpu.py`
 * T1-T3, T3b, T6).
 *
 * Each function names the reference lines it restates. Build with -ffp-contract=off and without -ffast-math: every
 * quantiser step must be one IEEE fp32 operation (kv_fp4_ref.py:15-25).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define HKVO_BLOCK 16

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bf16_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 >= 0 -> e4m3fn byte, round to nearest even, saturating at 448; NaN -> 0x7f.
 * Restates e4m3_encode (kv_fp4_ref.py:94-97): clamp(max=448) then torch's float8_e4m3fn cast. */
uint8_t hkvo_e4m3_encode(float x) {
  if (x != x) return 0x7f;
  if (x >= 448.0f) return 0x7e;
  if (x <= 0.0f) return 0;
  if (x < 0.015625f) {                 /* below the smallest normal 2^-6: multiples of 2^-9 */
    float r = nearbyintf(x * 512.0f);  /* exact scaling, then RNE in the default rounding mode */
    return (uint8_t)r;                 /* 8 == 0x08 == 2^-6, the smallest normal */
  }
  uint32_t u = f32_bits(x);
  uint32_t lsb = (u >> 20) & 1u;
  u += 0x7ffffu + lsb;                 /* RNE to 3 mantissa bits (a carry moves into the exponent) */
  int e = (int)(u >> 23) - 127;
  uint32_t m = (u >> 20) & 7u;
  return (uint8_t)(((e + 7) << 3) | m);
}

/* e4m3fn byte -> value; 0x7f / 0xff are NaN. Restates e4m3_decode / e4m3_table (kv_fp4_ref.py:100-116). */
double hkvo_e4m3_decode(uint8_t c) {
  int s = c >> 7, e = (c >> 3) & 15, m = c & 7;
  double v;
  if (e == 15 && m == 7) v = NAN;
  else if (e == 0) v = m / 8.0 * ldexp(1.0, -6);
  else v = (1.0 + m / 8.0) * ldexp(1.0, e - 7);
  return s ? -v : v;
}

/* y >= 0 -> 3-bit magnitude code, nearest even on {0,.5,1,1.5,2,3,4,6}, saturating (kv_fp4_ref.py:122-130).
 * A NaN fails every comparison and falls through to 7, as in the reference's chain of torch.where. */
uint8_t hkvo_e2m1_mag(float y) {
  if (y <= 0.25f) return 0;
  if (y < 0.75f) return 1;
  if (y <= 1.25f) return 2;
  if (y < 1.75f) return 3;
  if (y <= 2.5f) return 4;
  if (y < 3.5f) return 5;
  if (y <= 5.0f) return 6;
  return 7;
}

static const float E2M1_GRID[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* 4-bit code (bit 3 = sign) -> value (kv_fp4_ref.py:133-136) */
float hkvo_e2m1_value(uint8_t code) {
  float v = E2M1_GRID[code & 7];
  return (code & 8) ? -v : v;
}

static inline uint8_t block_mag(float ax, float s) {       /* _block_codes, kv_fp4_ref.py:142-145 */
  if (!(s > 0.0f)) return 0;
  volatile float y = ax / s;
  return hkvo_e2m1_mag(y);
}

static float block_sse(const float* x, float s) {           /* _block_sse, kv_fp4_ref.py:148-156 */
  volatile float acc = 0.0f;
  for (int i = 0; i < HKVO_BLOCK; ++i) {
    float ax = fabsf(x[i]);
    volatile float p = E2M1_GRID[block_mag(ax, s)] * s;
    volatile float d = p - ax;
    volatile float sq = d * d;
    if (i == 0) acc = sq; else acc = acc + sq;
  }
  return acc;
}

/* One block of 16 values (kv_fp4_ref.py:159-186 for one block): 8 code bytes + 1 scale byte. */
void hkvo_quantize_block(const float* x, float g, int search, uint8_t* data, uint8_t* sf_out) {
  float amax = 0.0f;
  int nan_seen = 0;
  for (int i = 0; i < HKVO_BLOCK; ++i) {
    float a = fabsf(x[i]);
    if (a != a) nan_seen = 1;
    if (a > amax) amax = a;
  }
  if (nan_seen) amax = NAN;                                  /* torch amax propagates NaN */
  volatile float g6 = g * 6.0f;
  volatile float q6 = amax / g6;
  uint8_t sf = hkvo_e4m3_encode(q6);
  if (search) {
    int c0 = sf;
    volatile float g4 = g * 4.0f;
    volatile float q4 = amax / g4;
    uint8_t cand[4];
    cand[0] = sf;
    cand[1] = (uint8_t)(c0 + 1 > 126 ? 126 : c0 + 1);
    cand[2] = (uint8_t)(c0 - 1 < 0 ? 0 : c0 - 1);
    cand[3] = hkvo_e4m3_encode(q4);
    volatile float s0 = (float)hkvo_e4m3_decode(sf) * g;
    float best = block_sse(x, s0);
    for (int k = 1; k < 4; ++k) {
      volatile float sk = (float)hkvo_e4m3_decode(cand[k]) * g;
      float e = block_sse(x, sk);
      if (e < best) { best = e; sf = cand[k]; }
    }
  }
  volatile float s = (float)hkvo_e4m3_decode(sf) * g;
  uint8_t code[HKVO_BLOCK];
  for (int i = 0; i < HKVO_BLOCK; ++i)
    code[i] = (uint8_t)(block_mag(fabsf(x[i]), s) | (x[i] < 0.0f ? 8 : 0));
  for (int j = 0; j < HKVO_BLOCK / 2; ++j) data[j] = (uint8_t)(code[2 * j] | (code[2 * j + 1] << 4));
  *sf_out = sf;
}

/* quantize_rows (kv_fp4_ref.py:159-186): x (n_rows, D) fp32, g one value per row -> data (n_rows, D/2),
 * sf (n_rows, D/16). */
void hkvo_quantize_rows(const float* x, long long n_rows, int D, const float* g_row, int search, uint8_t* data,
                        uint8_t* sf) {
  const int nb = D / HKVO_BLOCK;
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < n_rows; ++r)
    for (int b = 0; b < nb; ++b)
      hkvo_quantize_block(x + r * D + b * HKVO_BLOCK, g_row[r], search, data + r * (D / 2) + b * 8, sf + r * nb + b);
}

/* dequantize_rows (kv_fp4_ref.py:189-199) in fp64: code * e4m3(sf) (* g_row when g_row != NULL) */
void hkvo_dequantize_rows(const uint8_t* data, const uint8_t* sf, long long n_rows, int D, const double* g_row,
                          double* out) {
  const int nb = D / HKVO_BLOCK;
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < n_rows; ++r)
    for (int b = 0; b < nb; ++b) {
      double s = hkvo_e4m3_decode(sf[r * nb + b]);
      for (int j = 0; j < 8; ++j) {
        uint8_t by = data[r * (D / 2) + b * 8 + j];
        double v0 = hkvo_e2m1_value(by & 15) * s, v1 = hkvo_e2m1_value(by >> 4) * s;
        if (g_row) { v0 *= g_row[r]; v1 *= g_row[r]; }
        out[r * D + b * 16 + 2 * j] = v0;
        out[r * D + b * 16 + 2 * j + 1] = v1;
      }
    }
}

/* rotate (kv_fp4_ref.py:55-87): out = FWHT(x * signs) * D^-0.5 in fp32, butterflies in the reference's stage order
 * (h = 1, 2, 4, .., D/2; for every i with (i & h) == 0: (x[i], x[i+h]) = (x[i] + x[i+h], x[i] - x[i+h])).
 * `scale` is D^-0.5 rounded to fp32 by the caller. x and out may be the same array. */
void hkvo_rotate_row(const float* x, const float* signs, int D, float scale, float* out) {
  for (int i = 0; i < D; ++i) { volatile float v = x[i] * signs[i]; out[i] = v; }
  for (int h = 1; h < D; h *= 2)
    for (int i = 0; i < D; ++i)
      if ((i & h) == 0) {
        volatile float a = out[i], b = out[i + h];
        volatile float s = a + b, d = a - b;
        out[i] = s;
        out[i + h] = d;
      }
  for (int i = 0; i < D; ++i) { volatile float v = out[i] * scale; out[i] = v; }
}
void hkvo_rotate_rows(const float* x, long long n_rows, int D, const float* signs, float scale, float* out) {
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < n_rows; ++r) hkvo_rotate_row(x + r * D, signs, D, scale, out + r * D);
}

/* The four cache parts as [page, position, head, byte] views of one byte buffer (kv_fp4_ref.py:215-230 and
 * backend.py:279-300): byte offsets of the parts plus data strides (page, position, head) and scale strides. */
typedef struct {
  long long kd, ksf, vd, vsf;          /* offsets of the four parts from the cache base */
  long long dsp, dst, dsh;             /* data strides: page, position, head */
  long long ssp, sst, ssh;             /* scale strides */
  int PS;
  int k8;                              /* 1: K8V4 slot (kv_fp4_ref.py:283-321): keys are D signed e4m3 bytes at kd (no
                                          block scales, ksf unused), values stay e2m1 codes + e4m3 block scales */
} hkvo_layout;

/* fp8_encode_signed (kv_fp4_ref.py:296-298): fp32 -> e4m3fn byte, round to nearest even, saturating to +-448; the sign
 * bit survives for -0.0 and for negative values that round to zero */
static uint8_t e4m3_encode_signed(float x) {
  return (uint8_t)((signbit(x) ? 0x80 : 0) | hkvo_e4m3_encode(fabsf(x)));
}
static double e4m3_decode_signed(uint8_t b) { return (b & 0x80 ? -1.0 : 1.0) * hkvo_e4m3_decode(b & 0x7f); }

/* write_reference (kv_fp4_ref.py:233-245): key/value (NT, KVH, D) bf16 with element strides (token, head), slot < 0
 * skipped, one global scale per kv head and side. signs != NULL: the keys are rotated first (hkvo_rotate_row) and
 * quantised from the fp32 result; values are never rotated. */
void hkvo_write_rot(const uint16_t* key, const uint16_t* val, long long ks0, long long ks1, long long vs0,
                    long long vs1, uint8_t* cache, const hkvo_layout* lay, const long long* slots, long long n_slots,
                    const float* gk, const float* gv, int KVH, int D, int search, const float* signs, float rot_scale) {
  const int nb = D / HKVO_BLOCK;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < n_slots; ++t) {
    long long sl = slots[t];
    if (sl < 0) continue;
    long long p = sl / lay->PS, o = sl % lay->PS;
    float row[512];
    for (int side = 0; side < 2; ++side)
      for (int h = 0; h < KVH; ++h) {
        const uint16_t* src = side ? val + t * vs0 + h * vs1 : key + t * ks0 + h * ks1;
        uint8_t* dd = cache + (side ? lay->vd : lay->kd) + p * lay->dsp + o * lay->dst + h * lay->dsh;
        uint8_t* ds = cache + (side ? lay->vsf : lay->ksf) + p * lay->ssp + o * lay->sst + h * lay->ssh;
        float g = side ? gv[h] : gk[h];
        for (int i = 0; i < D; ++i) row[i] = bf16_f32(src[i]);
        if (lay->k8 && side == 0) {                    /* write_reference_k8 (kv_fp4_ref.py:301-311): e4m3(k / gk) */
          for (int i = 0; i < D; ++i) { volatile float y = row[i] / g; dd[i] = e4m3_encode_signed(y); }
          continue;
        }
        if (signs && side == 0) hkvo_rotate_row(row, signs, D, rot_scale, row);
        for (int b = 0; b < nb; ++b) hkvo_quantize_block(row + b * 16, g, search, dd + b * 8, ds + b);
      }
  }
}
void hkvo_write(const uint16_t* key, const uint16_t* val, long long ks0, long long ks1, long long vs0, long long vs1,
                uint8_t* cache, const hkvo_layout* lay, const long long* slots, long long n_slots, const float* gk,
                const float* gv, int KVH, int D, int search) {
  hkvo_write_rot(key, val, ks0, ks1, vs0, vs1, cache, lay, slots, n_slots, gk, gv, KVH, D, search, 0, 0.0f);
}

/* attention_reference (kv_fp4_ref.py:260-280) with per-request query lengths (kv_fp4_serving.py:5-11): fp64 attention
 * over the dequantised cache. q (NT, HQ, D) bf16; request b owns query tokens [qsl[b], qsl[b+1]); token t of a request
 * with ql tokens and length L sees positions < L - ql + t + 1. out (NT, HQ, D) fp64; rows of requests with no query
 * tokens are left untouched. Returns the number of cached (token, kv head) pairs visited. */
long long hkvo_attention(const uint16_t* q, const uint8_t* cache, const hkvo_layout* lay, const int* bt, int MP,
                         const int* seq_lens, const int* qsl, int B, int KVH, int G, int D, double sm_scale,
                         const float* gk, const float* gv, double v_scale, double* out) {
  const int HQ = KVH * G, nb = D / HKVO_BLOCK;
  long long visited = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1) reduction(+ : visited)
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < KVH; ++h) {
      const int q0 = qsl[b], ql = qsl[b + 1] - q0, L = seq_lens[b];
      if (ql <= 0) continue;
      double* K = (double*)malloc((size_t)(L > 0 ? L : 1) * D * sizeof(double));
      double* V = (double*)malloc((size_t)(L > 0 ? L : 1) * D * sizeof(double));
      double* sc = (double*)malloc((size_t)(L > 0 ? L : 1) * sizeof(double));
      for (int j = 0; j < L; ++j) {                          /* gather, kv_fp4_ref.py:248-257 */
        long long page = bt[(long long)b * MP + j / lay->PS], pos = j % lay->PS;
        for (int side = 0; side < 2; ++side) {
          const uint8_t* dd = cache + (side ? lay->vd : lay->kd) + page * lay->dsp + pos * lay->dst + h * lay->dsh;
          const uint8_t* ds = cache + (side ? lay->vsf : lay->ksf) + page * lay->ssp + pos * lay->sst + h * lay->ssh;
          double* dst = (side ? V : K) + (size_t)j * D;
          if (lay->k8 && side == 0) {                  /* gather_k8 (kv_fp4_ref.py:314-321) */
            for (int i = 0; i < D; ++i) dst[i] = e4m3_decode_signed(dd[i]);
            continue;
          }
          for (int bb = 0; bb < nb; ++bb) {
            double s = hkvo_e4m3_decode(ds[bb]);
            for (int i = 0; i < 8; ++i) {
              uint8_t by = dd[bb * 8 + i];
              dst[bb * 16 + 2 * i] = hkvo_e2m1_value(by & 15) * s;
              dst[bb * 16 + 2 * i + 1] = hkvo_e2m1_value(by >> 4) * s;
            }
          }
        }
      }
      visited += L;
      for (int t = 0; t < ql; ++t) {
        int lim = L - ql + t + 1;
        if (lim > L) lim = L;
        for (int g = 0; g < G; ++g) {
          const uint16_t* qq = q + ((long long)(q0 + t) * HQ + h * G + g) * D;
          double* o = out + ((long long)(q0 + t) * HQ + h * G + g) * D;
          double mx = -INFINITY;
          for (int j = 0; j < lim; ++j) {
            double d = 0.0;
            const double* kj = K + (size_t)j * D;
            for (int c = 0; c < D; ++c) d += (double)bf16_f32(qq[c]) * kj[c];
            d = d * (double)gk[h] * sm_scale;
            sc[j] = d;
            if (d > mx) mx = d;
          }
          double den = 0.0;
          for (int j = 0; j < lim; ++j) { sc[j] = exp(sc[j] - mx); den += sc[j]; }
          for (int c = 0; c < D; ++c) o[c] = 0.0;
          for (int j = 0; j < lim; ++j) {
            double p = sc[j] / den;
            const double* vj = V + (size_t)j * D;
            for (int c = 0; c < D; ++c) o[c] += p * vj[c];
          }
          for (int c = 0; c < D; ++c) o[c] = o[c] * (double)gv[h] * v_scale;   /* all zeros when lim <= 0 */
        }
      }
      free(K); free(V); free(sc);
    }
  return visited;
}

int hkvo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void hkvo_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* array forms of the scalar codecs, for exhaustive tests */
void hkvo_e4m3_encode_n(const float* x, long long n, uint8_t* out) { for (long long i = 0; i < n; ++i) out[i] = hkvo_e4m3_encode(x[i]); }
void hkvo_e4m3_decode_n(const uint8_t* c, long long n, double* out) { for (long long i = 0; i < n; ++i) out[i] = hkvo_e4m3_decode(c[i]); }
void hkvo_e2m1_mag_n(const float* y, long long n, uint8_t* out) { for (long long i = 0; i < n; ++i) out[i] = hkvo_e2m1_mag(y[i]); }
void hkvo_e2m1_value_n(const uint8_t* c, long long n, float* out) { for (long long i = 0; i < n; ++i) out[i] = hkvo_e2m1_value(c[i]); }
