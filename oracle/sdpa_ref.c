/*
 * Plain-C restatement of dense non-causal forward attention. TEST INFRASTRUCTURE ONLY: used
 * to cross-check oracle/sdpa_oracle.py and as a CPU timing arm; the product never links it.
 *
 * Follows the streaming form of the reference kernel
 * (IaroslavElistratov/b200-attention, kernels/5_minor/18_tma_l2_promotion.cu): per query row a
 * running maximum and running sum over key blocks (:701-719, here with an exact rebase on every
 * block), un-normalised accumulation of P V (:229-251), division by the row sum at the end
 * (:859-873), and additionally the natural-log LSE (research/causal_gqa_2cta.cu:783-793).
 * Everything is fp32; inputs are bf16 bit patterns (uint16).
 *
 * Layout: q [bh, len_q, 128], k/v [bh, len_kv, 128] contiguous; o [bh, len_q, 128] fp32;
 * lse [bh, len_q] fp32 (may be NULL). Rows [row_begin, row_end) of every (batch*head) are
 * computed. OpenMP over (bh, row) when compiled with -fopenmp.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HEAD_DIM 128
#define KEY_BLOCK 256

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

int sdpa_ref_forward(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* o, float* lse,
                     int64_t bh, int64_t len_q, int64_t len_kv, float scale, int64_t row_begin,
                     int64_t row_end) {
  if (!q || !k || !v || !o || bh < 1 || len_q < 1 || len_kv < 1) return 1;
  if (row_begin < 0 || row_end > len_q || row_begin >= row_end) return 2;
  const int64_t rows = row_end - row_begin;
  int failed = 0;

#pragma omp parallel
  {
    /* per-thread fp32 copies of one key block and one value block */
    float* kb = (float*)malloc(sizeof(float) * KEY_BLOCK * HEAD_DIM);
    float* vb = (float*)malloc(sizeof(float) * KEY_BLOCK * HEAD_DIM);
    if (!kb || !vb) {
#pragma omp atomic write
      failed = 1;
    } else {
#pragma omp for collapse(2) schedule(dynamic, 1)
      for (int64_t h = 0; h < bh; ++h) {
        for (int64_t r0 = 0; r0 < rows; r0 += 64) {
          const int64_t r1 = r0 + 64 < rows ? r0 + 64 : rows;
          float m[64], l[64];
          float acc[64][HEAD_DIM];
          float qrow[64][HEAD_DIM];
          for (int64_t r = r0; r < r1; ++r) {
            m[r - r0] = -INFINITY;
            l[r - r0] = 0.0f;
            memset(acc[r - r0], 0, sizeof acc[0]);
            const uint16_t* qp = q + ((h * len_q) + row_begin + r) * HEAD_DIM;
            for (int d = 0; d < HEAD_DIM; ++d) qrow[r - r0][d] = bf16_to_f32(qp[d]);
          }
          for (int64_t j0 = 0; j0 < len_kv; j0 += KEY_BLOCK) {
            const int64_t nb = j0 + KEY_BLOCK < len_kv ? KEY_BLOCK : len_kv - j0;
            const uint16_t* kp = k + (h * len_kv + j0) * HEAD_DIM;
            const uint16_t* vp = v + (h * len_kv + j0) * HEAD_DIM;
            for (int64_t t = 0; t < nb * HEAD_DIM; ++t) {
              kb[t] = bf16_to_f32(kp[t]);
              vb[t] = bf16_to_f32(vp[t]);
            }
            for (int64_t r = r0; r < r1; ++r) {
              float s[KEY_BLOCK];
              float mx = m[r - r0];
              const float* qr = qrow[r - r0];
              for (int64_t j = 0; j < nb; ++j) {
                const float* kr = kb + j * HEAD_DIM;
                float dot = 0.0f;
                for (int d = 0; d < HEAD_DIM; ++d) dot += qr[d] * kr[d];
                s[j] = dot * scale;
                if (s[j] > mx) mx = s[j];
              }
              const float alpha = expf(m[r - r0] - mx);
              float sum = 0.0f;
              float* a = acc[r - r0];
              for (int d = 0; d < HEAD_DIM; ++d) a[d] *= alpha;
              for (int64_t j = 0; j < nb; ++j) {
                const float p = expf(s[j] - mx);
                sum += p;
                const float* vr = vb + j * HEAD_DIM;
                for (int d = 0; d < HEAD_DIM; ++d) a[d] += p * vr[d];
              }
              l[r - r0] = l[r - r0] * alpha + sum;
              m[r - r0] = mx;
            }
          }
          for (int64_t r = r0; r < r1; ++r) {
            float* op = o + ((h * rows) + r) * HEAD_DIM;
            const float inv = 1.0f / l[r - r0];
            for (int d = 0; d < HEAD_DIM; ++d) op[d] = acc[r - r0][d] * inv;
            if (lse) lse[h * rows + r] = m[r - r0] + logf(l[r - r0]);
          }
        }
      }
    }
    free(kb);
    free(vb);
  }
  return failed ? 3 : 0;
}
