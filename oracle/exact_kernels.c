/*
 * TEST INFRASTRUCTURE - CPU restatement helpers for the parity oracle.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may use
 * this file; the product path never does.
 *
 * Exact scalar loops that numpy cannot express:
 *   - the per-K-block promotion of the block-quantised GEMM,
 *       total = fmaf(float(partial), scale, total)          (bq.cu:190-195 of the reference)
 *     needs a correctly rounded fused multiply-add;
 *   - int8 x int8 -> int32 products with exact accumulation (int8.cu mode 0 of the reference).
 * Compile with -ffp-contract=off so nothing else is fused.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

/* total[i] = fmaf(partial[i], scale[i], total[i]) */
void oracle_fma_accumulate(float* total, const float* partial, const float* scale, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) total[i] = fmaf(partial[i], scale[i], total[i]);
}

/* c (m x n, int32) = a (m x k, int8) * b (n x k, int8)^T over k in [k0, k1) */
void oracle_i8_gemm_nt(const int8_t* a, const int8_t* b, int32_t* c, int m, int n, int k, int k0,
                       int k1) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) {
      int32_t acc = 0;
      const int8_t* ar = a + (size_t)i * k;
      const int8_t* br = b + (size_t)j * k;
      for (int kk = k0; kk < k1; ++kk) acc += (int32_t)ar[kk] * (int32_t)br[kk];
      c[(size_t)i * n + j] = acc;
    }
  }
}
