/*
 * CPU restatement in plain C of paged single-token decode with fused append --
 * TEST INFRASTRUCTURE ONLY (the checker and the timed CPU baseline; nothing in
 * the shipped package links or calls it).
 *
 * Semantics follow the reference project's NumPy test oracle,
 * tests/softmax_attention/test_paged.py:80-206 (append at cache_seqlens + t
 * through the block table, f32 scores = scale * q.k, optional softcap
 * softcap * tanh(s / softcap), causal / left-window mask on the bottom-right
 * diagonal, softmax with an optional sink logit in the denominator, natural-log
 * lse), on the merged [k0, v0, k1, v1, ...] bf16 layout of
 * flywheel_tpu/softmax_attention/kv_layout.py:39-46.  It is checked against
 * oracle/paged_attention.py (itself pinned to golden vectors) in
 * tests/test_oracle_c.py.  One OpenMP task per (request, kv head).
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t v) {
  uint32_t bits = (uint32_t)v << 16;
  float f;
  memcpy(&f, &bits, sizeof f);
  return f;
}

/*
 * q:      (batch, q_len, heads, d) bf16          out: (batch, q_len, heads, d) f32
 * pool:   (pages, page_size, 2*kv_heads, d) bf16 (updated in place by the append)
 * k_new, v_new: (batch, q_len, kv_heads, d) bf16 or NULL
 * lse:    (batch, heads, q_len) f32 or NULL; sinks: (heads,) f32 or NULL
 * window_left < 0: unbounded.  threads > 0 sets the OpenMP team size for this
 * call (the environment's OMP_NUM_THREADS is read only when the runtime loads,
 * and launchers such as torchrun set it to 1); 0 leaves it alone.  Returns 0.
 */
int fw_ref_paged_decode(const uint16_t* q, uint16_t* pool, const uint16_t* k_new, const uint16_t* v_new,
                        const int32_t* cache_seqlens, const int32_t* block_table, const float* sinks,
                        float* out, float* lse, int batch, int q_len, int heads, int kv_heads, int d,
                        int page_size, int pages_per_seq, int causal, int window_left, float scale,
                        float softcap, int threads) {
  const int group = heads / kv_heads;
  if (threads > 0) omp_set_num_threads(threads);
  const size_t row = (size_t)2 * kv_heads * d;
  /* append: whole merged rows, bits moved as they are */
  if (k_new != NULL) {
    for (int b = 0; b < batch; ++b)
      for (int t = 0; t < q_len; ++t) {
        const int pos = cache_seqlens[b] + t;
        const size_t page = (size_t)block_table[(size_t)b * pages_per_seq + pos / page_size];
        uint16_t* dst = pool + (page * page_size + pos % page_size) * row;
        for (int h = 0; h < kv_heads; ++h) {
          memcpy(dst + (size_t)(2 * h) * d, k_new + (((size_t)b * q_len + t) * kv_heads + h) * d, 2 * d);
          memcpy(dst + (size_t)(2 * h + 1) * d, v_new + (((size_t)b * q_len + t) * kv_heads + h) * d, 2 * d);
        }
      }
  }
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < kv_heads; ++h) {
      const int total = cache_seqlens[b] + (k_new != NULL ? q_len : 0);
      const int rows = q_len * group;
      float* qf = (float*)malloc(sizeof(float) * rows * d);
      float* acc = (float*)calloc((size_t)rows * d, sizeof(float));
      float* m = (float*)malloc(sizeof(float) * rows);
      float* l = (float*)calloc(rows, sizeof(float));
      float* kf = (float*)malloc(sizeof(float) * 2 * d);
      for (int r = 0; r < rows; ++r) {
        const int t = r / group, g = r % group;
        const uint16_t* src = q + (((size_t)b * q_len + t) * heads + h * group + g) * d;
        for (int i = 0; i < d; ++i) qf[(size_t)r * d + i] = bf16_to_f32(src[i]);
        m[r] = -INFINITY;
      }
      for (int pos = 0; pos < total; ++pos) {
        const size_t page = (size_t)block_table[(size_t)b * pages_per_seq + pos / page_size];
        const uint16_t* kv = pool + (page * page_size + pos % page_size) * row + (size_t)(2 * h) * d;
        for (int i = 0; i < 2 * d; ++i) kf[i] = bf16_to_f32(kv[i]);
        for (int r = 0; r < rows; ++r) {
          const int diag = total - q_len + r / group;
          if ((causal && pos > diag) || (window_left >= 0 && pos < diag - window_left)) continue;
          float s = 0.f;
          const float* qr = qf + (size_t)r * d;
          for (int i = 0; i < d; ++i) s += qr[i] * kf[i];
          s *= scale;
          if (softcap > 0.f) s = softcap * tanhf(s / softcap);
          if (s > m[r]) { /* move the running maximum */
            const float a = expf(m[r] - s);
            l[r] *= a;
            for (int i = 0; i < d; ++i) acc[(size_t)r * d + i] *= a;
            m[r] = s;
          }
          const float p = expf(s - m[r]);
          l[r] += p;
          const float* vr = kf + d;
          for (int i = 0; i < d; ++i) acc[(size_t)r * d + i] += p * vr[i];
        }
      }
      for (int r = 0; r < rows; ++r) {
        const int t = r / group, g = r % group, head = h * group + g;
        float top = m[r], den = l[r];
        if (sinks != NULL && sinks[head] != -INFINITY) {
          const float s = sinks[head];
          if (top == -INFINITY) { top = s; den = 1.f; }
          else if (s > top) { den = den * expf(top - s) + 1.f; for (int i = 0; i < d; ++i) acc[(size_t)r * d + i] *= expf(m[r] - s); top = s; }
          else den += expf(s - top);
        }
        float* dst = out + (((size_t)b * q_len + t) * heads + head) * d;
        const int seen = m[r] != -INFINITY;
        for (int i = 0; i < d; ++i) dst[i] = seen ? acc[(size_t)r * d + i] / den : 0.f;
        if (lse != NULL) lse[((size_t)b * heads + head) * q_len + t] = top == -INFINITY ? -INFINITY : top + logf(den);
      }
      free(qf); free(acc); free(m); free(l); free(kf);
    }
  return 0;
}
