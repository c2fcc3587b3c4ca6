/* CPU port of the annotated loops (oracle; test infrastructure, never linked into
 * the product).  Each function restates one reference loop in C with the element
 * arithmetic of the jitted loop: float32 elements; a float64 accumulator for
 * shared(...) scalars, which the front end turns into 1-element float64 arrays
 * (appy/frontend/process_shared.py:37-41); in-loop locals take the float32 type of
 * the products added to them (NumPy scalar promotion); and the loop's own iteration
 * order, so vec_add is bit-identical to NumPy and the reductions are sequential sums.
 * Rows / ranges are split over OpenMP threads when built with -fopenmp; reductions
 * then combine per-thread partials in thread order.
 *
 *   vec_add      examples/01-vec_add.py:7-13
 *   vec_sum      examples/02-vec_sum.py:5-11   (b is float64: frontend/process_shared.py:37-41)
 *   masked_sum   examples/04-masked_sum.py:7-23
 *   spmv         examples/03-spmv.py:5-16
 *   gemv         examples/05-gemv.py:7-17
 *   spmm         examples/06-spmm.py:4-11
 */
#include <stdint.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of OpenMP threads for the loops below.  A launcher may have set OMP_NUM_THREADS=1 for
 * every child process; the timed CPU baseline states its thread count instead of inheriting one. */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void oracle_vec_add_f32(const float* a, const float* b, float* c, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) c[i] = a[i] + b[i];
}

double oracle_vec_sum_f32(const float* a, int64_t n, double init) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t i = 0; i < n; ++i) total += (double)a[i];
  return init + total;
}

double oracle_masked_sum_f32(const float* a, const uint8_t* mask, int64_t n, double init) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t i = 0; i < n; ++i)
    if (mask[i]) total += (double)a[i];
  return init + total;
}

/* s starts as a Python float and becomes float32 after the first `s += f32 * f32`
 * (NumPy scalar promotion), so the row sum is a sequential float32 sum. */
void oracle_spmv_f32(const float* data, const int32_t* indptr, const int32_t* indices,
                     const float* x, float* y, int64_t row_lo, int64_t row_hi) {
#pragma omp parallel for schedule(dynamic, 1024)
  for (int64_t i = row_lo; i < row_hi; ++i) {
    float s = 0.0f;
    for (int32_t k = indptr[i]; k < indptr[i + 1]; ++k) s += data[k] * x[indices[k]];
    y[i] = s;
  }
}

void oracle_gemv_f32(float alpha, const float* A, int64_t lda, const float* x, float* y,
                     int64_t row_lo, int64_t row_hi, int64_t ncols) {
#pragma omp parallel for schedule(static)
  for (int64_t i = row_lo; i < row_hi; ++i) {
    float yi = 0.0f;
    const float* row = A + i * lda;
    for (int64_t j = 0; j < ncols; ++j) yi += alpha * row[j] * x[j];
    y[i] = yi;
  }
}

void oracle_spmm_f32(const float* data, const int32_t* indptr, const int32_t* indices,
                     const float* B, int64_t ldb, float* C, int64_t ldc, int64_t row_lo,
                     int64_t row_hi, int ncols) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t i = row_lo; i < row_hi; ++i) {
    float* c = C + i * ldc;
    for (int j = 0; j < ncols; ++j) c[j] = 0.0f;
    for (int32_t k = indptr[i]; k < indptr[i + 1]; ++k) {
      const float v = data[k];
      const float* b = B + (int64_t)indices[k] * ldb;
      for (int j = 0; j < ncols; ++j) c[j] += v * b[j];
    }
  }
}
