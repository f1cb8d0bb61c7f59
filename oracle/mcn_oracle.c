/* Plain-C restatement of the reference CPU backend for the training hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker: it is loaded by
 * tests/, by the smoke check and by the CPU-baseline leg of the benchmark,
 * never by the library itself.  The product path is CUDA only and fails
 * loudly when its extension is missing.
 *
 * Each function follows the reference file:line quoted beside it in
 * mcn_oracle_impl.h (paths relative to matlab/src/bits/ of the reference).
 * Parity pin: tests/test_oracle_pinned.py checks every function against
 * golden vectors produced by the reference's own compiled CPU code
 * (tests/golden/, made by tests/golden/make_golden.py) and against the
 * known-answer identities of the reference's test suite.
 *
 * Scalar, single-threaded, IEEE arithmetic: build with -ffp-contract=off and
 * without -ffast-math.  dtype: 0 = float, 1 = double.  Return value: 0 on
 * success, otherwise the numeric vl::ErrorCode (5 = out of memory).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define T float
#define FN(x) x##_f32
#include "mcn_oracle_impl.h"
#undef T
#undef FN

#define T double
#define FN(x) x##_f64
#include "mcn_oracle_impl.h"
#undef T
#undef FN

#define F(p) ((float*)(p))
#define D(p) ((double*)(p))
#define CF(p) ((float const*)(p))
#define CD(p) ((double const*)(p))

int mcno_conv_forward(int dt, void* y, void const* x, void const* f, void const* b, int const* shape, int const* prm)
{ return dt ? conv_forward_f64(D(y), CD(x), CD(f), CD(b), shape, prm) : conv_forward_f32(F(y), CF(x), CF(f), CF(b), shape, prm); }

int mcno_conv_backward(int dt, void* dx, void* df, void* db, void const* x, void const* f, void const* dy,
                       int const* shape, int const* prm)
{ return dt ? conv_backward_f64(D(dx), D(df), D(db), CD(x), CD(f), CD(dy), shape, prm)
            : conv_backward_f32(F(dx), F(df), F(db), CF(x), CF(f), CF(dy), shape, prm); }

int mcno_fc_forward(int dt, void* y, void const* x, void const* f, void const* b, int const* shape)
{ return dt ? fc_forward_f64(D(y), CD(x), CD(f), CD(b), shape) : fc_forward_f32(F(y), CF(x), CF(f), CF(b), shape); }

int mcno_fc_backward(int dt, void* dx, void* df, void* db, void const* x, void const* f, void const* dy, int const* shape)
{ return dt ? fc_backward_f64(D(dx), D(df), D(db), CD(x), CD(f), CD(dy), shape)
            : fc_backward_f32(F(dx), F(df), F(db), CF(x), CF(f), CF(dy), shape); }

int mcno_convt_forward(int dt, void* y, void const* x, void const* f, void const* b, int const* shape, int const* prm)
{ return dt ? convt_forward_f64(D(y), CD(x), CD(f), CD(b), shape, prm) : convt_forward_f32(F(y), CF(x), CF(f), CF(b), shape, prm); }

int mcno_convt_backward(int dt, void* dx, void* df, void* db, void const* x, void const* f, void const* dy,
                        int const* shape, int const* prm)
{ return dt ? convt_backward_f64(D(dx), D(df), D(db), CD(x), CD(f), CD(dy), shape, prm)
            : convt_backward_f32(F(dx), F(df), F(db), CF(x), CF(f), CF(dy), shape, prm); }

int mcno_bias_forward(int dt, void* y, double ymult, void const* x, double xmult, void const* b, double bmult,
                      int H, int W, int K, int N)
{ return dt ? bias_forward_f64(D(y), ymult, CD(x), xmult, CD(b), bmult, H, W, K, N)
            : bias_forward_f32(F(y), ymult, CF(x), xmult, CF(b), bmult, H, W, K, N); }

int mcno_bias_backward(int dt, void* dx, double dxmult, void* db, double dbmult, double xmult, double bmult,
                       void const* dy, int H, int W, int K, int N)
{ return dt ? bias_backward_f64(D(dx), dxmult, D(db), dbmult, xmult, bmult, CD(dy), H, W, K, N)
            : bias_backward_f32(F(dx), dxmult, F(db), dbmult, xmult, bmult, CF(dy), H, W, K, N); }

int mcno_bnorm_forward(int dt, void* y, void* mom, void const* x, void const* g, void const* b,
                       int H, int W, int C, int N, double eps)
{ return dt ? bnorm_forward_f64(D(y), D(mom), CD(x), CD(g), CD(b), H, W, C, N, eps)
            : bnorm_forward_f32(F(y), F(mom), CF(x), CF(g), CF(b), H, W, C, N, eps); }

int mcno_bnorm_forward_moment(int dt, void* y, void const* mom, void const* x, void const* g, void const* b,
                              int H, int W, int C, int N, double eps)
{ return dt ? bnorm_forward_moment_f64(D(y), CD(mom), CD(x), CD(g), CD(b), H, W, C, N, eps)
            : bnorm_forward_moment_f32(F(y), CF(mom), CF(x), CF(g), CF(b), H, W, C, N, eps); }

int mcno_bnorm_backward(int dt, void* dx, void* dg, void* db, void* mom, void const* x, void const* g,
                        void const* b, void const* dy, int H, int W, int C, int N, double eps)
{ return dt ? bnorm_backward_f64(D(dx), D(dg), D(db), D(mom), CD(x), CD(g), CD(b), CD(dy), H, W, C, N, eps)
            : bnorm_backward_f32(F(dx), F(dg), F(db), F(mom), CF(x), CF(g), CF(b), CF(dy), H, W, C, N, eps); }

int mcno_bnorm_backward_moment(int dt, void* dx, void* dg, void* db, void const* mom, void const* x,
                               void const* g, void const* b, void const* dy, int H, int W, int C, int N, double eps)
{ return dt ? bnorm_backward_moment_f64(D(dx), D(dg), D(db), CD(mom), CD(x), CD(g), CD(b), CD(dy), H, W, C, N, eps)
            : bnorm_backward_moment_f32(F(dx), F(dg), F(db), CF(mom), CF(x), CF(g), CF(b), CF(dy), H, W, C, N, eps); }

int mcno_pool_forward(int dt, void* y, void const* x, int H, int W, int C, int N, int const* prm)
{ return dt ? pool_forward_f64(D(y), CD(x), H, W, C, N, prm) : pool_forward_f32(F(y), CF(x), H, W, C, N, prm); }

int mcno_pool_backward(int dt, void* dx, void const* x, void const* dy, int H, int W, int C, int N, int const* prm)
{ return dt ? pool_backward_f64(D(dx), CD(x), CD(dy), H, W, C, N, prm)
            : pool_backward_f32(F(dx), CF(x), CF(dy), H, W, C, N, prm); }

int mcno_roipool_bounds(int dt, int* bounds, int* images, void const* rois, int H, int W, int N, int numROIs,
                        int S0, int S1, double const* tf)
{ return dt ? roipool_bounds_f64(bounds, images, CD(rois), H, W, N, numROIs, S0, S1, tf)
            : roipool_bounds_f32(bounds, images, CF(rois), H, W, N, numROIs, S0, S1, tf); }

int mcno_roipool_forward(int dt, void* y, void const* x, void const* rois, int H, int W, int C, int N,
                         int numROIs, int S0, int S1, double const* tf, int method)
{ return dt ? roipool_forward_f64(D(y), CD(x), CD(rois), H, W, C, N, numROIs, S0, S1, tf, method)
            : roipool_forward_f32(F(y), CF(x), CF(rois), H, W, C, N, numROIs, S0, S1, tf, method); }

int mcno_roipool_backward(int dt, void* dx, void const* x, void const* rois, void const* dy, int H, int W, int C,
                          int N, int numROIs, int S0, int S1, double const* tf, int method)
{ return dt ? roipool_backward_f64(D(dx), CD(x), CD(rois), CD(dy), H, W, C, N, numROIs, S0, S1, tf, method)
            : roipool_backward_f32(F(dx), CF(x), CF(rois), CF(dy), H, W, C, N, numROIs, S0, S1, tf, method); }

int mcno_sampler_forward(int dt, void* y, void const* x, void const* grid, int H, int W, int C, int N,
                         int Ho, int Wo, int Ng)
{ return dt ? sampler_forward_f64(D(y), CD(x), CD(grid), H, W, C, N, Ho, Wo, Ng)
            : sampler_forward_f32(F(y), CF(x), CF(grid), H, W, C, N, Ho, Wo, Ng); }

int mcno_sampler_backward(int dt, void* dx, void* dgrid, void const* x, void const* grid, void const* dy,
                          int H, int W, int C, int N, int Ho, int Wo, int Ng)
{ return dt ? sampler_backward_f64(D(dx), D(dgrid), CD(x), CD(grid), CD(dy), H, W, C, N, Ho, Wo, Ng)
            : sampler_backward_f32(F(dx), F(dgrid), CF(x), CF(grid), CF(dy), H, W, C, N, Ho, Wo, Ng); }

int mcno_relu_forward(int dt, void* y, void const* x, size_t n)
{ return dt ? relu_forward_f64(D(y), CD(x), n) : relu_forward_f32(F(y), CF(x), n); }

int mcno_relu_backward(int dt, void* dx, void const* x, void const* dy, size_t n)
{ return dt ? relu_backward_f64(D(dx), CD(x), CD(dy), n) : relu_backward_f32(F(dx), CF(x), CF(dy), n); }

int mcno_softmaxloss_forward(int dt, void* loss, void const* x, void const* labels, int H, int W, int C, int N)
{ return dt ? softmaxloss_forward_f64(D(loss), CD(x), CD(labels), H, W, C, N)
            : softmaxloss_forward_f32(F(loss), CF(x), CF(labels), H, W, C, N); }

int mcno_softmaxloss_backward(int dt, void* dx, void const* x, void const* labels, double dzdy, int H, int W, int C, int N)
{ return dt ? softmaxloss_backward_f64(D(dx), CD(x), CD(labels), dzdy, H, W, C, N)
            : softmaxloss_backward_f32(F(dx), CF(x), CF(labels), (float)dzdy, H, W, C, N); }

int mcno_lrn_forward(int dt, void* y, void const* x, int H, int W, int C, int N, double const* prm)
{ return dt ? lrn_forward_f64(D(y), CD(x), H, W, C, N, (int)prm[0], prm[1], prm[2], prm[3])
            : lrn_forward_f32(F(y), CF(x), H, W, C, N, (int)prm[0], prm[1], prm[2], prm[3]); }

int mcno_lrn_backward(int dt, void* dx, void const* x, void const* dy, int H, int W, int C, int N, double const* prm)
{ return dt ? lrn_backward_f64(D(dx), CD(x), CD(dy), H, W, C, N, (int)prm[0], prm[1], prm[2], prm[3])
            : lrn_backward_f32(F(dx), CF(x), CF(dy), H, W, C, N, (int)prm[0], prm[1], prm[2], prm[3]); }

int mcno_softmax(int dt, void* out, void const* x, void const* dz, int H, int W, int C, int N)
{ return dt ? softmax_f64(D(out), CD(x), dz ? CD(dz) : 0, H, W, C, N) : softmax_f32(F(out), CF(x), dz ? CF(dz) : 0, H, W, C, N); }
