/* Stand-in for MATLAB's <blas.h>, which the reference CPU backend includes
 * (matlab/src/bits/impl/blashelper.hpp:18) and which is not shipped with it.
 *
 * TEST INFRASTRUCTURE ONLY: this header exists so that the unmodified
 * reference sources can be compiled into oracle/_ref/libmcn_ref.so.
 *
 * The reference calls the Fortran entry points with ptrdiff_t integer
 * arguments (blashelper.hpp:89-141).  The definitions live in
 * oracle/ref_blas.cpp: a plain column-major implementation by default, or
 * an ILP64 OpenBLAS loaded at run time when mcnref_use_openblas() is called.
 */
#ifndef MCN_REF_SHIM_BLAS_H
#define MCN_REF_SHIM_BLAS_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
void sgemm(char const *ta, char const *tb, ptrdiff_t const *m, ptrdiff_t const *n, ptrdiff_t const *k,
           float const *alpha, float const *a, ptrdiff_t const *lda, float const *b, ptrdiff_t const *ldb,
           float const *beta, float *c, ptrdiff_t const *ldc);
void dgemm(char const *ta, char const *tb, ptrdiff_t const *m, ptrdiff_t const *n, ptrdiff_t const *k,
           double const *alpha, double const *a, ptrdiff_t const *lda, double const *b, ptrdiff_t const *ldb,
           double const *beta, double *c, ptrdiff_t const *ldc);
void sgemv(char const *t, ptrdiff_t const *m, ptrdiff_t const *n, float const *alpha,
           float const *a, ptrdiff_t const *lda, float const *x, ptrdiff_t const *incx,
           float const *beta, float *y, ptrdiff_t const *incy);
void dgemv(char const *t, ptrdiff_t const *m, ptrdiff_t const *n, double const *alpha,
           double const *a, ptrdiff_t const *lda, double const *x, ptrdiff_t const *incx,
           double const *beta, double *y, ptrdiff_t const *incy);
void saxpy(ptrdiff_t const *n, float const *alpha, float const *x, ptrdiff_t const *incx,
           float *y, ptrdiff_t const *incy);
void daxpy(ptrdiff_t const *n, double const *alpha, double const *x, ptrdiff_t const *incx,
           double *y, ptrdiff_t const *incy);
void sscal(ptrdiff_t const *n, float const *alpha, float *x, ptrdiff_t const *incx);
void dscal(ptrdiff_t const *n, double const *alpha, double *x, ptrdiff_t const *incx);
#ifdef __cplusplus
}
#endif
#endif
