/*
 * CPU restatement (plain C, OpenMP) of the reference's decode-path arithmetic, used as the parity
 * checker's fast twin and as the timed CPU baseline.  TEST / BENCH INFRASTRUCTURE ONLY: nothing
 * under dmlx_b200/ links or loads this file.
 *
 * It follows the reference's *structure*, including the work the reference does on every decode
 * step and the GPU path avoids:
 *   - gather every page of a sequence into one contiguous K/V array
 *     (src/kvcache/paged.zig:705-802: mlx_slice per page + mlx_concatenate),
 *   - repeat each KV head for its group of query heads (src/models/llama.zig:240-241,303-323),
 *   - scores = q K^T / sqrt(D), softmax, scores V (src/models/llama.zig:249-270).
 * Parity is unpinned against MLX itself (not vendored in the reference tree); the Python oracle
 * (oracle/ref_math.py), which is pinned on the reference's golden vectors, cross-checks this file
 * in tests/test_oracle_c.py.
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Pool layout: [page][kv_head][32][D] bf16.  q: [n_seq][Hq][D] f32.  out: [n_seq][Hq][D] f32.
 * block_table: [n_seq][max_pages].  Returns 0, or -1 on allocation failure. */
int ref_paged_attention_decode(const uint16_t* k_pool, const uint16_t* v_pool, const int32_t* block_table,
                               int32_t max_pages, const int32_t* ctx, int32_t n_seq, int32_t hq, int32_t hkv,
                               int32_t d, const float* q, float* out) {
  const int g = hq / hkv;
  int fail = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int s = 0; s < n_seq; ++s) {
    const int len = ctx[s];
    if (len <= 0) {
      memset(out + (size_t)s * hq * d, 0, sizeof(float) * hq * d);
      continue;
    }
    /* gather: contiguous [Hkv][len][D] (paged.zig:705-802) */
    float* kc = (float*)malloc(sizeof(float) * (size_t)hkv * len * d);
    float* vc = (float*)malloc(sizeof(float) * (size_t)hkv * len * d);
    /* repeatHeads: [Hq][len][D] (llama.zig:303-323) */
    float* kr = (float*)malloc(sizeof(float) * (size_t)hq * len * d);
    float* vr = (float*)malloc(sizeof(float) * (size_t)hq * len * d);
    float* sc = (float*)malloc(sizeof(float) * (size_t)len);
    if (!kc || !vc || !kr || !vr || !sc) { fail = 1; free(kc); free(vc); free(kr); free(vr); free(sc); continue; }
    for (int t = 0; t < len; ++t) {
      const int page = block_table[(size_t)s * max_pages + t / 32], slot = t % 32;
      for (int h = 0; h < hkv; ++h) {
        const size_t src = (((size_t)page * hkv + h) * 32 + slot) * d;
        float* kd = kc + ((size_t)h * len + t) * d;
        float* vd = vc + ((size_t)h * len + t) * d;
        for (int i = 0; i < d; ++i) { kd[i] = bf16_to_f32(k_pool[src + i]); vd[i] = bf16_to_f32(v_pool[src + i]); }
      }
    }
    for (int h = 0; h < hq; ++h) {
      memcpy(kr + (size_t)h * len * d, kc + (size_t)(h / g) * len * d, sizeof(float) * (size_t)len * d);
      memcpy(vr + (size_t)h * len * d, vc + (size_t)(h / g) * len * d, sizeof(float) * (size_t)len * d);
    }
    const float scale = 1.0f / sqrtf((float)d);
    for (int h = 0; h < hq; ++h) {
      const float* qh = q + ((size_t)s * hq + h) * d;
      float mx = -INFINITY;
      for (int t = 0; t < len; ++t) {
        const float* kt = kr + ((size_t)h * len + t) * d;
        float acc = 0.f;
        for (int i = 0; i < d; ++i) acc += qh[i] * kt[i];
        sc[t] = acc * scale;
        if (sc[t] > mx) mx = sc[t];
      }
      float sum = 0.f;
      for (int t = 0; t < len; ++t) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
      float* o = out + ((size_t)s * hq + h) * d;
      for (int i = 0; i < d; ++i) o[i] = 0.f;
      for (int t = 0; t < len; ++t) {
        const float p = sc[t] / sum;
        const float* vt = vr + ((size_t)h * len + t) * d;
        for (int i = 0; i < d; ++i) o[i] += p * vt[i];
      }
    }
    free(kc); free(vc); free(kr); free(vr); free(sc);
  }
  return fail ? -1 : 0;
}

/* y[T][N] = x[T][K] . dequant(W)^T, affine 4-bit group 64: packed uint32 [N][K/8] (nibble j of a word
 * = column 8w+j), scales/biases f32 [N][K/64]  (call sites src/models/llama.zig:127,367,596). */
void ref_qmm_affine4(const uint32_t* packed, const float* scales, const float* biases, int32_t n, int32_t k,
                     const float* x, int32_t t_rows, float* y) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n; ++r) {
    float* wrow = (float*)malloc(sizeof(float) * k);
    for (int c = 0; c < k; ++c) {
      const uint32_t word = packed[(size_t)r * (k / 8) + c / 8];
      const float qv = (float)((word >> (4 * (c % 8))) & 0xF);
      wrow[c] = qv * scales[(size_t)r * (k / 64) + c / 64] + biases[(size_t)r * (k / 64) + c / 64];
    }
    for (int t = 0; t < t_rows; ++t) {
      const float* xr = x + (size_t)t * k;
      float acc = 0.f;
      for (int c = 0; c < k; ++c) acc += xr[c] * wrow[c];
      y[(size_t)t * n + r] = acc;
    }
    free(wrow);
  }
}

/* MXFP4: bytes [N][K/2], low nibble = even column; E8M0 scale per 32 columns
 * (src/models/deepseek_v4_loader.zig:839-920). */
void ref_qmm_mxfp4(const uint8_t* packed, const uint8_t* scales, int32_t n, int32_t k, const float* x,
                   int32_t t_rows, float* y) {
  static const float tab[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, 0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n; ++r) {
    float* wrow = (float*)malloc(sizeof(float) * k);
    for (int c = 0; c < k; ++c) {
      const uint8_t b = packed[(size_t)r * (k / 2) + c / 2];
      const float v = tab[(c & 1) ? (b >> 4) : (b & 0xF)];
      wrow[c] = v * exp2f((float)scales[(size_t)r * (k / 32) + c / 32] - 127.f);
    }
    for (int t = 0; t < t_rows; ++t) {
      const float* xr = x + (size_t)t * k;
      float acc = 0.f;
      for (int c = 0; c < k; ++c) acc += xr[c] * wrow[c];
      y[(size_t)t * n + r] = acc;
    }
    free(wrow);
  }
}

/* Use `n` OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1). */
void ref_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int ref_num_threads(void) {
  int n = 1;
#pragma omp parallel
  {
#pragma omp single
    n =
#ifdef _OPENMP
        omp_get_num_threads();
#else
        1;
#endif
  }
  return n;
}
