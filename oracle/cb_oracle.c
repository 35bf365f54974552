/*
 * CPU oracle, C restatement (TEST INFRASTRUCTURE ONLY).
 *
 * The same algorithm as oracle/cb_oracle.py, written in plain C with OpenMP so that
 * (a) the parity tests can check full-size layers in seconds and (b) the benchmark
 * has a CPU baseline that uses every host core.  Nothing that ships links this file.
 *
 * Follows, in the reference project:
 *   bit extraction / value decode / weight rounding   tests/cb_torch_reference.py:33-178
 *   full mode                                         docs/SPEC.md:97-101
 *   scale planes                                      gridbook/codec.py:170-194
 *   activation buckets                                gridbook/codec.py:248-260, 428-437
 *   linear = bf16 weights, fp32 product, bf16 output  tests/cb_torch_reference.py:307-330
 * Parity is pinned by tests/test_oracle_c.py against the reference-generated fixtures.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GBO_API __attribute__((visibility("default")))

enum { GRID_FP4 = 0, GRID_FP8 = 1 };
enum { MODE_PRODUCT = 0, MODE_SIGNED = 1, MODE_FULL = 2 };
enum { SCALE_NONE = 0, SCALE_V1 = 1, SCALE_V2 = 2 };

typedef struct {
  int grid, mode, k_bits, n_sub, type_size, scale_coding;
} gbo_format;

static inline float bits_to_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

static inline float bf16_round(float x) {
  uint32_t b = f32_to_bits(x);
  if ((b & 0x7FFFFFFFu) > 0x7F800000u) return x;              /* NaN */
  b = (b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u;
  return bits_to_f32(b);
}

static float e4m3_lut[256];
static int lut_ready = 0;
static void init_lut(void) {
  if (lut_ready) return;
  for (int b = 0; b < 256; ++b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + m / 8.0f, e - 7);
    if (e == 15 && m == 7) v = NAN;
    e4m3_lut[b] = (b & 0x80) ? -v : v;
  }
  lut_ready = 1;
}

/* fp32 -> E4M3, one rounding to nearest even; |f| < 480. */
static inline uint8_t f32_to_e4m3(float f) {
  uint32_t u = f32_to_bits(f);
  uint32_t sign = (u >> 24) & 0x80u;
  u &= 0x7FFFFFFFu;
  uint32_t r;
  if (u >= (1087u << 20)) r = 0x7F;
  else if (u < (121u << 23)) {
    float shifted = bits_to_f32(u) + 16384.0f;
    r = f32_to_bits(shifted) - f32_to_bits(16384.0f);
  } else {
    uint32_t odd = (u >> 20) & 1u;
    u += 0x7FFFFu + odd;
    r = (u >> 20) - (120u << 3);
  }
  return (uint8_t)((r & 0x7Fu) | sign);
}

GBO_API int gbo_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* One row: packed bytes -> K served weights (bf16 values held as fp32). */
static void decode_row(const uint8_t* row, int64_t avail, const float* cb, const float* compose,
                       float wscale, const gbo_format* f, int64_t K, float* w) {
  const int n_sb = (int)(K / 256);
  const int k = f->k_bits;
  int widths[4] = {0, 0, 0, 0}, shifts[4] = {0, 0, 0, 0}, bases[4] = {0, 0, 0, 0};
  const int n_sub = f->mode == MODE_PRODUCT ? f->n_sub : 1;
  const int sub_dim = 8 / n_sub;
  if (f->mode == MODE_PRODUCT) {
    int off = 0, base = 0;
    for (int i = 0; i < n_sub; ++i) {
      widths[i] = k / n_sub + (i < k % n_sub ? 1 : 0);
      shifts[i] = off; bases[i] = base;
      off += widths[i]; base += (1 << widths[i]) * sub_dim;
    }
  }
  for (int s = 0; s < n_sb; ++s) {
    const uint8_t* sb = row + (int64_t)s * f->type_size;
    const int64_t sb_avail = avail - (int64_t)s * f->type_size;
    float gscale[16];
    if (f->grid == GRID_FP4) {
      const uint8_t* plane = sb + 4 * k;
      if (f->scale_coding == SCALE_V1) {
        for (int g = 0; g < 16; ++g) gscale[g] = e4m3_lut[plane[g]];
      } else {
        const int e = plane[0];
        for (int g = 0; g < 16; ++g) {
          const int nib = (plane[1 + (g >> 1)] >> ((g & 1) * 4)) & 15;
          gscale[g] = compose[e * 16 + nib];
        }
      }
    }
    for (int v = 0; v < 32; ++v) {
      const int bit = v * k, byte0 = bit >> 3, sh = bit & 7;
      uint64_t win = 0;
      for (int i = 0; i < 8; ++i)
        if (byte0 + i < sb_avail) win |= (uint64_t)sb[byte0 + i] << (8 * i);
      const uint64_t code = (win >> sh) & ((k >= 64) ? ~0ull : ((1ull << k) - 1ull));
      float val[8];
      if (f->mode == MODE_FULL) {
        for (int j = 0; j < 8; ++j) val[j] = cb[code * 8 + j];
      } else if (f->mode == MODE_SIGNED) {
        for (int j = 0; j < 8; ++j) {
          const float m = cb[(code >> 8) * 8 + j];
          val[j] = ((code >> j) & 1) ? -m : m;
        }
      } else {
        for (int i = 0; i < n_sub; ++i) {
          const uint64_t idx = (code >> shifts[i]) & ((1ull << widths[i]) - 1ull);
          for (int t = 0; t < sub_dim; ++t) val[i * sub_dim + t] = cb[bases[i] + idx * sub_dim + t];
        }
      }
      const float sc = f->grid == GRID_FP4 ? gscale[v >> 1] : wscale;
      float* dst = w + (int64_t)s * 256 + v * 8;
      for (int j = 0; j < 8; ++j) dst[j] = bf16_round(val[j] * sc);
    }
  }
}

/* [nrows, K] served weights of rows [row0, row0+nrows). */
GBO_API void gbo_reconstruct(const uint8_t* qw, int64_t row_stride, const float* cb,
                             const int32_t* cb_row_offset, const float* compose,
                             const float* weight_scale, const gbo_format* f, int64_t N, int64_t K,
                             int64_t row0, int64_t nrows, float* out) {
  init_lut();
  const int64_t row_bytes = (K / 256) * f->type_size;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t n = row0 + r;
    const int64_t avail = (N - 1 - n) * row_stride + row_bytes;
    decode_row(qw + n * row_stride, avail, cb + (cb_row_offset ? cb_row_offset[n] : 0), compose,
               weight_scale ? weight_scale[n] : 1.0f, f, K, out + r * K);
  }
}

/* y[M,N] = bf16( global_scale * sum_k x[m,k] * W[n,k] ), W = bf16 served weights, fp32 sums. */
GBO_API void gbo_linear(const float* x, int64_t M, const uint8_t* qw, int64_t row_stride,
                        const float* cb, const int32_t* cb_row_offset, const float* compose,
                        const float* weight_scale, float global_scale, const gbo_format* f,
                        int64_t N, int64_t K, float* y) {
  init_lut();
  const int64_t row_bytes = (K / 256) * f->type_size;
#pragma omp parallel
  {
    float* w = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      const int64_t avail = (N - 1 - n) * row_stride + row_bytes;
      decode_row(qw + n * row_stride, avail, cb + (cb_row_offset ? cb_row_offset[n] : 0), compose,
                 weight_scale ? weight_scale[n] : 1.0f, f, K, w);
      for (int64_t m = 0; m < M; ++m) {
        const float* xr = x + m * K;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int64_t k8 = 0; k8 < K; k8 += 8)
          for (int j = 0; j < 8; ++j) acc[j] += xr[k8 + j] * w[k8 + j];
        const float sum = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        y[m * N + n] = bf16_round(sum * global_scale);
      }
    }
    free(w);
  }
}

static const float kGrid[15] = {-6.f, -4.f, -3.f, -2.f, -1.5f, -1.f, -.5f, 0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};

/* Group-16 E2M1 round-to-nearest QDQ; scale_div != 0 divides amax by 6, else multiplies by fp32(1/6). */
GBO_API void gbo_fp4_act_qdq(const float* x, int64_t M, int64_t K, int scale_div, float* out) {
  const volatile float inv6 = 1.0f / 6.0f;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < M * (K / 16); ++g) {
    const float* v = x + g * 16;
    float amax = 0.f;
    int has_nan = 0;
    for (int i = 0; i < 16; ++i) { amax = fmaxf(amax, fabsf(v[i])); has_nan |= isnan(v[i]); }
    /* torch.amax spreads a NaN over the group (gridbook/codec.py:254); C's fmaxf would drop it */
    amax = has_nan ? NAN : fmaxf(amax, 1e-8f);
    const float scale = scale_div ? amax / 6.0f : amax * inv6;
    for (int i = 0; i < 16; ++i) {
      const float xg = v[i] / scale;
      int idx = 15;
      for (int j = 14; j >= 0; --j) if (kGrid[j] >= xg) idx = j;
      const float lo = kGrid[idx > 0 ? idx - 1 : 0], hi = kGrid[idx < 15 ? idx : 14];
      const float q = fabsf(hi - xg) < fabsf(xg - lo) ? hi : lo;
      out[g * 16 + i] = bf16_round(q * scale);
    }
  }
}

/* Per-token dynamic E4M3 QDQ. */
GBO_API void gbo_fp8_act_qdq(const float* x, int64_t M, int64_t K, int scale_div, float* out) {
  init_lut();
  const volatile float inv448 = 1.0f / 448.0f;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float* v = x + m * K;
    float amax = 0.f;
    int has_nan = 0;
    for (int64_t i = 0; i < K; ++i) { amax = fmaxf(amax, fabsf(v[i])); has_nan |= isnan(v[i]); }
    float scale = scale_div ? amax / 448.0f : amax * inv448;
    /* torch's amax and clamp both keep a NaN (gridbook/codec.py:433-435): the row becomes NaN */
    scale = has_nan ? NAN : fmaxf(scale, 1.0f / (448.0f * 512.0f));
    for (int64_t i = 0; i < K; ++i) {
      float q = v[i] / scale;
      if (isnan(q)) { out[m * K + i] = NAN; continue; }
      q = fminf(fmaxf(q, -448.0f), 448.0f);
      out[m * K + i] = bf16_round(e4m3_lut[f32_to_e4m3(q)] * scale);
    }
  }
}
