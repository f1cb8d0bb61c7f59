// BLAS entry points for the compiled reference CPU backend (oracle/_ref).
//
// TEST INFRASTRUCTURE ONLY.  The reference links MATLAB's libmwblas
// (Makefile:115), which is not part of its source tree.  These are the eight
// Fortran-convention routines it calls (matlab/src/bits/impl/blashelper.hpp:
// 89-141,160-212), with ptrdiff_t integers.
//
// Default: a plain column-major implementation whose summation order is
// fixed (reduction index ascending), so golden vectors made with it are
// reproducible on any machine.
// Optional: mcnref_use_openblas(path, threads) loads an ILP64 OpenBLAS (the
// one bundled with numpy exports scipy_sgemm_64_ and friends, whose 64-bit
// integers match ptrdiff_t) and forwards gemm/gemv to it; used only for the
// timed CPU baseline.
#include "blas.h"
#include <dlfcn.h>
#include <cstdio>
#include <cstring>
#include <vector>

namespace {

typedef void (*sgemm_fn)(char const*, char const*, ptrdiff_t const*, ptrdiff_t const*, ptrdiff_t const*,
                         float const*, float const*, ptrdiff_t const*, float const*, ptrdiff_t const*,
                         float const*, float*, ptrdiff_t const*);
typedef void (*dgemm_fn)(char const*, char const*, ptrdiff_t const*, ptrdiff_t const*, ptrdiff_t const*,
                         double const*, double const*, ptrdiff_t const*, double const*, ptrdiff_t const*,
                         double const*, double*, ptrdiff_t const*);
typedef void (*sgemv_fn)(char const*, ptrdiff_t const*, ptrdiff_t const*, float const*, float const*,
                         ptrdiff_t const*, float const*, ptrdiff_t const*, float const*, float*, ptrdiff_t const*);
typedef void (*dgemv_fn)(char const*, ptrdiff_t const*, ptrdiff_t const*, double const*, double const*,
                         ptrdiff_t const*, double const*, ptrdiff_t const*, double const*, double*, ptrdiff_t const*);
typedef void (*setthreads_fn)(int);

sgemm_fn ob_sgemm = nullptr;
dgemm_fn ob_dgemm = nullptr;
sgemv_fn ob_sgemv = nullptr;
dgemv_fn ob_dgemv = nullptr;

inline bool isT(char const* t) { return *t == 't' || *t == 'T' || *t == 'c' || *t == 'C'; }

// C(m x n) = alpha * op(A) * op(B) + beta * C, column-major.
// Each C(i,j) is the sum over l = 0..k-1 in ascending order, accumulated in T.
template <typename T>
void gemm_plain(char const* ta, char const* tb, ptrdiff_t m, ptrdiff_t n, ptrdiff_t k, T alpha,
                T const* a, ptrdiff_t lda, T const* b, ptrdiff_t ldb, T beta, T* c, ptrdiff_t ldc)
{
  bool at = isT(ta), bt = isT(tb);
  std::vector<T> col(m > 0 ? m : 1);
  for (ptrdiff_t j = 0; j < n; ++j) {
    for (ptrdiff_t i = 0; i < m; ++i) col[i] = 0;
    if (!at) {
      for (ptrdiff_t l = 0; l < k; ++l) {
        T bv = bt ? b[j + l * ldb] : b[l + j * ldb];
        T const* ac = a + l * lda;
        for (ptrdiff_t i = 0; i < m; ++i) col[i] += ac[i] * bv;
      }
    } else {
      for (ptrdiff_t i = 0; i < m; ++i) {
        T const* ar = a + i * lda;
        T s = 0;
        if (!bt) { T const* bc = b + j * ldb; for (ptrdiff_t l = 0; l < k; ++l) s += ar[l] * bc[l]; }
        else     { for (ptrdiff_t l = 0; l < k; ++l) s += ar[l] * b[j + l * ldb]; }
        col[i] = s;
      }
    }
    T* cc = c + j * ldc;
    if (beta == T(0)) { for (ptrdiff_t i = 0; i < m; ++i) cc[i] = alpha * col[i]; }
    else              { for (ptrdiff_t i = 0; i < m; ++i) cc[i] = alpha * col[i] + beta * cc[i]; }
  }
}

// y = alpha * op(A) * x + beta * y, A is m x n column-major.
template <typename T>
void gemv_plain(char const* t, ptrdiff_t m, ptrdiff_t n, T alpha, T const* a, ptrdiff_t lda,
                T const* x, ptrdiff_t incx, T beta, T* y, ptrdiff_t incy)
{
  if (isT(t)) {
    for (ptrdiff_t j = 0; j < n; ++j) {
      T s = 0;
      T const* ac = a + j * lda;
      for (ptrdiff_t i = 0; i < m; ++i) s += ac[i] * x[i * incx];
      y[j * incy] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[j * incy];
    }
  } else {
    for (ptrdiff_t i = 0; i < m; ++i) {
      T s = 0;
      for (ptrdiff_t j = 0; j < n; ++j) s += a[i + j * lda] * x[j * incx];
      y[i * incy] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[i * incy];
    }
  }
}

}  // namespace

extern "C" {

// Returns 1 when the library was loaded and all four symbols resolved.
int mcnref_use_openblas(char const* path, int threads)
{
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return 0;
  sgemm_fn s = (sgemm_fn)dlsym(h, "scipy_sgemm_64_");
  dgemm_fn d = (dgemm_fn)dlsym(h, "scipy_dgemm_64_");
  sgemv_fn sv = (sgemv_fn)dlsym(h, "scipy_sgemv_64_");
  dgemv_fn dv = (dgemv_fn)dlsym(h, "scipy_dgemv_64_");
  if (!s || !d || !sv || !dv) return 0;
  setthreads_fn st = (setthreads_fn)dlsym(h, "scipy_openblas_set_num_threads64_");
  if (st && threads > 0) st(threads);
  ob_sgemm = s; ob_dgemm = d; ob_sgemv = sv; ob_dgemv = dv;
  return 1;
}

void mcnref_use_plain_blas(void) { ob_sgemm = nullptr; ob_dgemm = nullptr; ob_sgemv = nullptr; ob_dgemv = nullptr; }
int mcnref_blas_is_openblas(void) { return ob_sgemm != nullptr; }

void sgemm(char const* ta, char const* tb, ptrdiff_t const* m, ptrdiff_t const* n, ptrdiff_t const* k,
           float const* alpha, float const* a, ptrdiff_t const* lda, float const* b, ptrdiff_t const* ldb,
           float const* beta, float* c, ptrdiff_t const* ldc)
{
  if (ob_sgemm) { ob_sgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); return; }
  gemm_plain<float>(ta, tb, *m, *n, *k, *alpha, a, *lda, b, *ldb, *beta, c, *ldc);
}
void dgemm(char const* ta, char const* tb, ptrdiff_t const* m, ptrdiff_t const* n, ptrdiff_t const* k,
           double const* alpha, double const* a, ptrdiff_t const* lda, double const* b, ptrdiff_t const* ldb,
           double const* beta, double* c, ptrdiff_t const* ldc)
{
  if (ob_dgemm) { ob_dgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); return; }
  gemm_plain<double>(ta, tb, *m, *n, *k, *alpha, a, *lda, b, *ldb, *beta, c, *ldc);
}
void sgemv(char const* t, ptrdiff_t const* m, ptrdiff_t const* n, float const* alpha, float const* a,
           ptrdiff_t const* lda, float const* x, ptrdiff_t const* incx, float const* beta, float* y,
           ptrdiff_t const* incy)
{
  if (ob_sgemv) { ob_sgemv(t, m, n, alpha, a, lda, x, incx, beta, y, incy); return; }
  gemv_plain<float>(t, *m, *n, *alpha, a, *lda, x, *incx, *beta, y, *incy);
}
void dgemv(char const* t, ptrdiff_t const* m, ptrdiff_t const* n, double const* alpha, double const* a,
           ptrdiff_t const* lda, double const* x, ptrdiff_t const* incx, double const* beta, double* y,
           ptrdiff_t const* incy)
{
  if (ob_dgemv) { ob_dgemv(t, m, n, alpha, a, lda, x, incx, beta, y, incy); return; }
  gemv_plain<double>(t, *m, *n, *alpha, a, *lda, x, *incx, *beta, y, *incy);
}
void saxpy(ptrdiff_t const* n, float const* alpha, float const* x, ptrdiff_t const* incx, float* y,
           ptrdiff_t const* incy)
{ for (ptrdiff_t i = 0; i < *n; ++i) y[i * *incy] += *alpha * x[i * *incx]; }
void daxpy(ptrdiff_t const* n, double const* alpha, double const* x, ptrdiff_t const* incx, double* y,
           ptrdiff_t const* incy)
{ for (ptrdiff_t i = 0; i < *n; ++i) y[i * *incy] += *alpha * x[i * *incx]; }
void sscal(ptrdiff_t const* n, float const* alpha, float* x, ptrdiff_t const* incx)
{ for (ptrdiff_t i = 0; i < *n; ++i) x[i * *incx] *= *alpha; }
void dscal(ptrdiff_t const* n, double const* alpha, double* x, ptrdiff_t const* incx)
{ for (ptrdiff_t i = 0; i < *n; ++i) x[i * *incx] *= *alpha; }

}  // extern "C"
