/*
 * C restatement of the int8-KV-cache attention path (TEST INFRASTRUCTURE: the checker and the
 * timed CPU baseline; the product never links or calls it).
 *
 * Follows kbwal/inference-engine qwen3-1.7b/kernels.py:
 *   kv_quantize_rows        :460-480, :798-811   scale = max(absmax,1e-6)/127, rint, clamp +-127
 *   kv_norm_rope            :410-436, :579-633   per-head RMSNorm + half-split rotation, fp32
 *   kv_decode_attention     :128-264             computed the plain way: dequantize, fp32 softmax,
 *                                                fp32 P.V, round to bf16 (OpenMP over entry x kv head)
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/build_c.py).  No fast-math:
 * every operation is a separately rounded IEEE fp32 operation, and the 64-element sums use the
 * same pairwise order as the numpy restatement (oracle/oracle.py), so the two agree bit for bit
 * on codes, scales and rotated values.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x7FFFFFu)) return x; /* NaN */
  u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
  memcpy(&x, &u, 4);
  return x;
}

static float pairwise_sum64(const float* a) {
  float r[8];
  for (int j = 0; j < 8; ++j) r[j] = a[j];
  for (int i = 1; i < 8; ++i)
    for (int j = 0; j < 8; ++j) r[j] = r[j] + a[8 * i + j];
  return ((r[0] + r[1]) + (r[2] + r[3])) + ((r[4] + r[5]) + (r[6] + r[7]));
}

void kv_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int kv_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* x [rows, D] -> codes int8 [rows, D], scales [rows] */
void kv_quantize_rows(const float* x, int64_t rows, int D, int8_t* codes, float* scales) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * D;
    float amax = 0.0f;
    for (int d = 0; d < D; ++d) {
      float a = fabsf(row[d]);
      if (a > amax) amax = a;
    }
    float s = (amax > 1e-6f ? amax : 1e-6f) / 127.0f;
    scales[r] = s;
    for (int d = 0; d < D; ++d) {
      float c = rintf(row[d] / s);
      if (c > 127.0f) c = 127.0f;
      if (c < -127.0f) c = -127.0f;
      codes[r * D + d] = (int8_t)c;
    }
  }
}

/* x [T, H, 128], w [128], cos/sin [T, 64] -> out [T, H, 128] (fp32, not rounded) */
void kv_norm_rope(const float* x, int64_t T, int H, const float* w, const float* cos_t, const float* sin_t, float eps,
                  float* out) {
  enum { D = 128, HALF = 64 };
  for (int64_t t = 0; t < T; ++t)
    for (int h = 0; h < H; ++h) {
      const float* row = x + (t * H + h) * D;
      float sq[D];
      for (int d = 0; d < D; ++d) sq[d] = row[d] * row[d];
      float ss = pairwise_sum64(sq) + pairwise_sum64(sq + HALF);
      float rstd = 1.0f / sqrtf(ss / (float)D + eps);
      float* o = out + (t * H + h) * D;
      for (int d = 0; d < HALF; ++d) {
        float y1 = (row[d] * rstd) * w[d];
        float y2 = (row[d + HALF] * rstd) * w[d + HALF];
        float c = cos_t[t * HALF + d], s = sin_t[t * HALF + d];
        o[d] = y1 * c - y2 * s;
        o[d + HALF] = y1 * s + y2 * c;
      }
    }
}

/* Decode attention over a paged int8 cache.
 * q [B, Hq, 128] fp32 (bf16 values); k,v int8 [num_pages, Hkv, P, 128]; scales [num_pages, Hkv, P];
 * table int32 [B, max_pages]; entry b attends tokens [0, cached_lens[b]].  out [B, Hq, 128] fp32
 * holding bf16-rounded values; rows >= num_decoding untouched. */
void kv_decode_attention(const float* q, const int8_t* k, const int8_t* v, const float* k_scale, const float* v_scale,
                         const int32_t* table, int max_pages, const int32_t* cached_lens, int B, int num_decoding,
                         int Hq, int Hkv, int P, float scale, float* out) {
  enum { D = 128 };
  const int G = Hq / Hkv;
  const int nd = num_decoding < B ? num_decoding : B;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < nd; ++b)
    for (int h = 0; h < Hkv; ++h) {
      const int n = cached_lens[b] + 1;
      float* s = (float*)malloc((size_t)n * G * sizeof(float));
      float m[8], l[8], acc[8][D];
      for (int g = 0; g < G; ++g) m[g] = -INFINITY;
      for (int t = 0; t < n; ++t) {
        const int64_t page = table[(int64_t)b * max_pages + t / P];
        const int64_t row = ((page * Hkv + h) * P + t % P);
        const int8_t* kc = k + row * D;
        const float ks = k_scale[row];
        float kd[D];
        for (int d = 0; d < D; ++d) kd[d] = (float)kc[d] * ks;
        for (int g = 0; g < G; ++g) {
          const float* qr = q + ((int64_t)b * Hq + h * G + g) * D;
          float dot = 0.0f;
          for (int d = 0; d < D; ++d) dot += qr[d] * kd[d];
          dot *= scale;
          s[(size_t)g * n + t] = dot;
          if (dot > m[g]) m[g] = dot;
        }
      }
      for (int g = 0; g < G; ++g) {
        l[g] = 0.0f;
        for (int d = 0; d < D; ++d) acc[g][d] = 0.0f;
      }
      for (int t = 0; t < n; ++t) {
        const int64_t page = table[(int64_t)b * max_pages + t / P];
        const int64_t row = ((page * Hkv + h) * P + t % P);
        const int8_t* vc = v + row * D;
        const float vs = v_scale[row];
        float vd[D];
        for (int d = 0; d < D; ++d) vd[d] = (float)vc[d] * vs;
        for (int g = 0; g < G; ++g) {
          const float p = expf(s[(size_t)g * n + t] - m[g]);
          l[g] += p;
          for (int d = 0; d < D; ++d) acc[g][d] += p * vd[d];
        }
      }
      for (int g = 0; g < G; ++g) {
        float* o = out + ((int64_t)b * Hq + h * G + g) * D;
        for (int d = 0; d < D; ++d) o[d] = bf16_round(acc[g][d] / l[g]);
      }
      free(s);
    }
}
