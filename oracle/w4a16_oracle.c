/*
 * CPU restatement (C, OpenMP) of GlowQ's corrected W4A16 linear.  TEST INFRASTRUCTURE ONLY:
 * it is the checker and the timed CPU baseline, never part of the shipped path.
 *
 * Follows the reference's CPU-capable path:
 *   - nibble order and zero-point packing      src/cuda_w4a16/linear.py:42-54, 75-85
 *   - dequantised weight half((code-z)*s)      src/cuda_w4a16/linear.py:248-253, csrc/gemm_w4a16.cu:44-49
 *   - chunked dequantise-then-matmul forward   src/cuda_w4a16/linear.py:229-238
 *   - low-rank correction z += alpha*(xR^T)L^T src/step3_eval_dataset.py:470-511
 * evaluated with fp32 accumulation and no intermediate fp16 rounding of r or of the
 * correction, i.e. the fp32 result the parity tolerances are quoted against.
 * Checked against the numpy oracle (itself pinned to outputs of the reference) in tests/.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline int nib(const int32_t *row, int idx) {
  return (int)(((uint32_t)row[idx >> 3] >> ((idx & 7) * 4)) & 0xFu);
}

/* out_w[OC, IC] fp16 = half((code - zero) * scale); bit-exact definition. */
int glowq_oracle_dequant(const int32_t *qweight, const uint16_t *scales_bits, const int32_t *qzeros,
                         uint16_t *out_bits, int OC, int IC, int group_size, int weight_stride_i32,
                         int zero_stride_i32, int scale_stride) {
  const f16 *scales = (const f16 *)scales_bits;
  f16 *out = (f16 *)out_bits;
  if (group_size <= 0 || group_size % 8) return 1;
#pragma omp parallel for schedule(static)
  for (int oc = 0; oc < OC; ++oc) {
    const int32_t *wrow = qweight + (size_t)oc * weight_stride_i32;
    const int32_t *zrow = qzeros + (size_t)oc * zero_stride_i32;
    for (int k = 0; k < IC; ++k) {
      int g = k / group_size;
      float v = (float)(nib(wrow, k) - nib(zrow, g)) * (float)scales[(size_t)oc * scale_stride + g];
      out[(size_t)oc * IC + k] = (f16)v;
    }
  }
  return 0;
}

/* y[M, OC] fp32 = x . dequant(Q)^T (+bias) + alpha * (x . R^T) . L^T
 * r_io: optional [M, rank] fp32 buffer; r_mode 0 = no correction, 1 = compute r = x R^T and store
 * it there (cache "set"), 2 = read r from there (cache "hit").  */
int glowq_oracle_corrected_forward(const uint16_t *x_bits, const int32_t *qweight, const uint16_t *scales_bits,
                                   const int32_t *qzeros, const uint16_t *bias_bits, const uint16_t *R_bits,
                                   const uint16_t *L_bits, float *r_io, int r_mode, float alpha, float *y, int M,
                                   int IC, int OC, int rank, int group_size, int weight_stride_i32,
                                   int zero_stride_i32, int scale_stride, int num_threads) {
  const f16 *x = (const f16 *)x_bits, *scales = (const f16 *)scales_bits, *bias = (const f16 *)bias_bits;
  const f16 *R = (const f16 *)R_bits, *L = (const f16 *)L_bits;
  if (group_size <= 0 || group_size % 8) return 1;
  if (r_mode != 0 && (rank <= 0 || !r_io || !L)) return 2;
  if (r_mode == 1 && !R) return 2;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
  float *xf = (float *)malloc((size_t)M * IC * sizeof(float));
  if (!xf) return 3;
  for (size_t i = 0; i < (size_t)M * IC; ++i) xf[i] = (float)x[i];

  if (r_mode == 1) {
#pragma omp parallel for schedule(static)
    for (int j = 0; j < rank; ++j) {
      for (int m = 0; m < M; ++m) {
        float acc = 0.f;
        const f16 *rr = R + (size_t)j * IC;
        const float *xm = xf + (size_t)m * IC;
        for (int k = 0; k < IC; ++k) acc += (float)rr[k] * xm[k];
        r_io[(size_t)m * rank + j] = acc;
      }
    }
  }

#pragma omp parallel
  {
    float *wrow_f = (float *)malloc((size_t)IC * sizeof(float));
#pragma omp for schedule(static)
    for (int oc = 0; oc < OC; ++oc) {
      const int32_t *wrow = qweight + (size_t)oc * weight_stride_i32;
      const int32_t *zrow = qzeros + (size_t)oc * zero_stride_i32;
      for (int k = 0; k < IC; ++k) {
        int g = k / group_size;
        f16 w = (f16)((float)(nib(wrow, k) - nib(zrow, g)) * (float)scales[(size_t)oc * scale_stride + g]);
        wrow_f[k] = (float)w;
      }
      for (int m = 0; m < M; ++m) {
        const float *xm = xf + (size_t)m * IC;
        float acc = 0.f;
        for (int k = 0; k < IC; ++k) acc += wrow_f[k] * xm[k];
        if (bias) acc += (float)bias[oc];
        if (r_mode != 0 && alpha != 0.f) {
          float c = 0.f;
          const f16 *lr = L + (size_t)oc * rank;
          const float *rm = r_io + (size_t)m * rank;
          for (int j = 0; j < rank; ++j) c += (float)lr[j] * rm[j];
          acc += alpha * c;
        }
        y[(size_t)m * OC + oc] = acc;
      }
    }
    free(wrow_f);
  }
  free(xf);
  return 0;
}

int glowq_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
