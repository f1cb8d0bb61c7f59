// C entry points onto the UNMODIFIED reference CPU backend.
//
// TEST INFRASTRUCTURE ONLY: compiled together with the reference's own
// sources (matlab/src/bits/*.cpp, impl/im2row_cpu.cpp, impl/copy_cpu.cpp)
// into oracle/_ref/libmcn_ref.so by oracle/build_oracle.py.  It plays the
// part of the MEX gateways, which cannot be compiled without MATLAB: it wraps
// caller-owned host buffers as vl::Tensor views, applies the gateways' output
// shape formulas (matlab/src/vl_nnconv.cu:324-331, vl_nnpool.cu:240-247) and
// calls the operator classes (bits/nnconv.hpp:23-52, nnfullyconnected.hpp:
// 20-37, nnbias.hpp:20-35, nnbnorm.hpp:22-59, nnpooling.hpp:21-49,
// nnroipooling.hpp:23-45, nnbilinearsampler.hpp:21-36).
//
// dtype: 0 = single, 1 = double (the reference instantiates both when built
// with ENABLE_DOUBLE, bits/impl/dispatcher.hpp:91-93).  Null pointers become
// null tensors, which the operators skip (bits/nnconv.cu:190-212).
// Every function returns the vl::ErrorCode as int.
#include "data.hpp"
#include "nnconv.hpp"
#include "nnfullyconnected.hpp"
#include "nnbias.hpp"
#include "nnbnorm.hpp"
#include "nnpooling.hpp"
#include "nnroipooling.hpp"
#include "nnbilinearsampler.hpp"
#include "nnnormalize.hpp"
#include <array>
#include <cstring>

namespace {

vl::Context& ctx() { static vl::Context c; return c; }

vl::Tensor view(void const* p, int dtype, size_t h, size_t w, size_t c, size_t n)
{
  if (!p) return vl::Tensor();
  vl::DataType dt = dtype ? vl::VLDT_Double : vl::VLDT_Float;
  vl::TensorShape shape(h, w, c, n);
  return vl::Tensor(shape, dt, vl::VLDT_CPU, const_cast<void*>(p),
                    shape.getNumElements() * vl::getDataTypeSizeInBytes(dt));
}

inline int outdim(int in, int padA, int padB, int f, int dil, int stride)
{ return (in + padA + padB - ((f - 1) * dil + 1)) / stride + 1; }

}  // namespace

extern "C" {

char const* mcnref_last_error(void) { return ctx().getLastErrorMessage().c_str(); }

// shape = {H,W,C,N, FH,FW,FC,K}; prm = {strideY,strideX,padT,padB,padL,padR,dilY,dilX}
int mcnref_conv_forward(int dtype, void* y, void const* x, void const* f, void const* b,
                        int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FC = shape[6], K = shape[7];
  int Ho = outdim(H, prm[2], prm[3], FH, prm[6], prm[0]);
  int Wo = outdim(W, prm[4], prm[5], FW, prm[7], prm[1]);
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, FH, FW, FC, K);
  vl::Tensor B = view(b, dtype, 1, 1, 1, K), Y = view(y, dtype, Ho, Wo, K, N);
  vl::nn::Convolution op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5], prm[6], prm[7]);
  return op.forward(Y, 0, X, 1, F, B);
}

int mcnref_conv_backward(int dtype, void* dx, void* df, void* db, void const* x, void const* f,
                         void const* dy, int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FC = shape[6], K = shape[7];
  int Ho = outdim(H, prm[2], prm[3], FH, prm[6], prm[0]);
  int Wo = outdim(W, prm[4], prm[5], FW, prm[7], prm[1]);
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, FH, FW, FC, K);
  vl::Tensor DY = view(dy, dtype, Ho, Wo, K, N);
  vl::Tensor DX = view(dx, dtype, H, W, C, N), DF = view(df, dtype, FH, FW, FC, K), DB = view(db, dtype, 1, 1, 1, K);
  vl::nn::Convolution op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5], prm[6], prm[7]);
  return op.backward(DX, DF, DB, X, F, DY);
}

// Convolution transpose (bits/nnconv.hpp:54-80): shape = {H,W,C,N, FH,FW,FD,FN}; prm = {upsampleY,upsampleX,cropT,cropB,
// cropL,cropR,numGroups}; output extent as in the gateway (matlab/src/vl_nnconvt.cu:293-296).
int mcnref_convt_forward(int dtype, void* y, void const* x, void const* f, void const* b, int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FD = shape[6], FN = shape[7];
  int Ho = (H - 1) * prm[0] - (prm[2] + prm[3]) + FH, Wo = (W - 1) * prm[1] - (prm[4] + prm[5]) + FW, K = FD * prm[6];
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, FH, FW, FD, FN);
  vl::Tensor B = view(b, dtype, 1, 1, 1, K), Y = view(y, dtype, Ho, Wo, K, N);
  vl::nn::ConvolutionTranspose op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5]);
  return op.forward(Y, X, F, B);
}

int mcnref_convt_backward(int dtype, void* dx, void* df, void* db, void const* x, void const* f, void const* dy,
                          int const* shape, int const* prm)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], FH = shape[4], FW = shape[5], FD = shape[6], FN = shape[7];
  int Ho = (H - 1) * prm[0] - (prm[2] + prm[3]) + FH, Wo = (W - 1) * prm[1] - (prm[4] + prm[5]) + FW, K = FD * prm[6];
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, FH, FW, FD, FN), DY = view(dy, dtype, Ho, Wo, K, N);
  vl::Tensor DX = view(dx, dtype, H, W, C, N), DF = view(df, dtype, FH, FW, FD, FN), DB = view(db, dtype, 1, 1, 1, K);
  vl::nn::ConvolutionTranspose op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5]);
  return op.backward(DX, DF, DB, X, F, DY);
}

// Fully-connected mode (output 1x1): shape = {H,W,C,N, FH,FW,FC,K} with FH=H, FW=W, FC=C.
int mcnref_fc_forward(int dtype, void* y, void const* x, void const* f, void const* b, int const* shape)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], K = shape[7];
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, shape[4], shape[5], shape[6], K);
  vl::Tensor B = view(b, dtype, 1, 1, 1, K), Y = view(y, dtype, 1, 1, K, N);
  vl::nn::FullyConnected op(ctx());
  return op.forward(Y, X, F, B);
}

int mcnref_fc_backward(int dtype, void* dx, void* df, void* db, void const* x, void const* f,
                       void const* dy, int const* shape)
{
  int H = shape[0], W = shape[1], C = shape[2], N = shape[3], K = shape[7];
  vl::Tensor X = view(x, dtype, H, W, C, N), F = view(f, dtype, shape[4], shape[5], shape[6], K);
  vl::Tensor DY = view(dy, dtype, 1, 1, K, N);
  vl::Tensor DX = view(dx, dtype, H, W, C, N), DF = view(df, dtype, shape[4], shape[5], shape[6], K);
  vl::Tensor DB = view(db, dtype, 1, 1, 1, K);
  vl::nn::FullyConnected op(ctx());
  return op.backward(DX, DF, DB, X, F, DY);
}

int mcnref_bias_forward(int dtype, void* y, double ymult, void const* x, double xmult, void const* b,
                        double bmult, int H, int W, int K, int N)
{
  vl::Tensor Y = view(y, dtype, H, W, K, N), X = view(x, dtype, H, W, K, N), B = view(b, dtype, 1, 1, 1, K);
  vl::nn::Bias op(ctx());
  return op.forward(Y, ymult, X, xmult, B, bmult);
}

int mcnref_bias_backward(int dtype, void* dx, double dxmult, void* db, double dbmult, double xmult,
                         double bmult, void const* dy, int H, int W, int K, int N)
{
  vl::Tensor DX = view(dx, dtype, H, W, K, N), DB = view(db, dtype, 1, 1, 1, K), DY = view(dy, dtype, H, W, K, N);
  vl::nn::Bias op(ctx());
  return op.backward(DX, dxmult, DB, dbmult, xmult, bmult, DY);
}

// moments: 2*C values, [mean(0..C-1), sigma(C..2C-1)] (vl_nnbnorm.cu:210-213); may be NULL.
int mcnref_bnorm_forward(int dtype, void* y, void* moments, void const* x, void const* g, void const* b,
                         int H, int W, int C, int N, double eps)
{
  vl::Tensor Y = view(y, dtype, H, W, C, N), M = view(moments, dtype, C, 2, 1, 1), X = view(x, dtype, H, W, C, N);
  vl::Tensor G = view(g, dtype, C, 1, 1, 1), B = view(b, dtype, C, 1, 1, 1);
  vl::nn::BatchNorm op(ctx(), eps);
  return op.forward(Y, M, X, G, B);
}

int mcnref_bnorm_forward_moment(int dtype, void* y, void const* moments, void const* x, void const* g,
                                void const* b, int H, int W, int C, int N, double eps)
{
  vl::Tensor Y = view(y, dtype, H, W, C, N), M = view(moments, dtype, C, 2, 1, 1), X = view(x, dtype, H, W, C, N);
  vl::Tensor G = view(g, dtype, C, 1, 1, 1), B = view(b, dtype, C, 1, 1, 1);
  vl::nn::BatchNorm op(ctx(), eps);
  return op.forwardWithMoment(Y, M, X, G, B);
}

int mcnref_bnorm_backward(int dtype, void* dx, void* dg, void* db, void* moments, void const* x,
                          void const* g, void const* b, void const* dy, int H, int W, int C, int N, double eps)
{
  vl::Tensor DX = view(dx, dtype, H, W, C, N), DG = view(dg, dtype, C, 1, 1, 1), DB = view(db, dtype, C, 1, 1, 1);
  vl::Tensor M = view(moments, dtype, C, 2, 1, 1), X = view(x, dtype, H, W, C, N);
  vl::Tensor G = view(g, dtype, C, 1, 1, 1), B = view(b, dtype, C, 1, 1, 1), DY = view(dy, dtype, H, W, C, N);
  vl::nn::BatchNorm op(ctx(), eps);
  return op.backward(DX, DG, DB, M, X, G, B, DY);
}

int mcnref_bnorm_backward_moment(int dtype, void* dx, void* dg, void* db, void const* moments, void const* x,
                                 void const* g, void const* b, void const* dy, int H, int W, int C, int N,
                                 double eps)
{
  vl::Tensor DX = view(dx, dtype, H, W, C, N), DG = view(dg, dtype, C, 1, 1, 1), DB = view(db, dtype, C, 1, 1, 1);
  vl::Tensor M = view(moments, dtype, C, 2, 1, 1), X = view(x, dtype, H, W, C, N);
  vl::Tensor G = view(g, dtype, C, 1, 1, 1), B = view(b, dtype, C, 1, 1, 1), DY = view(dy, dtype, H, W, C, N);
  vl::nn::BatchNorm op(ctx(), eps);
  return op.backwardWithMoment(DX, DG, DB, M, X, G, B, DY);
}

// prm = {poolH,poolW,strideY,strideX,padT,padB,padL,padR,method(0 max,1 avg)}
int mcnref_pool_forward(int dtype, void* y, void const* x, int H, int W, int C, int N, int const* prm)
{
  int Ho = (H + prm[4] + prm[5] - prm[0]) / prm[2] + 1, Wo = (W + prm[6] + prm[7] - prm[1]) / prm[3] + 1;
  vl::Tensor Y = view(y, dtype, Ho, Wo, C, N), X = view(x, dtype, H, W, C, N);
  vl::nn::Pooling op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5], prm[6], prm[7],
                     prm[8] ? vl::nn::Pooling::Average : vl::nn::Pooling::Max);
  return op.forward(Y, X);
}

// dx is zero-filled first, as the gateway does (vl_nnpool.cu:255-259).
int mcnref_pool_backward(int dtype, void* dx, void const* x, void const* dy, int H, int W, int C, int N,
                         int const* prm)
{
  int Ho = (H + prm[4] + prm[5] - prm[0]) / prm[2] + 1, Wo = (W + prm[6] + prm[7] - prm[1]) / prm[3] + 1;
  vl::Tensor DX = view(dx, dtype, H, W, C, N), X = view(x, dtype, H, W, C, N), DY = view(dy, dtype, Ho, Wo, C, N);
  memset(dx, 0, (size_t)H * W * C * N * (dtype ? 8 : 4));
  vl::nn::Pooling op(ctx(), prm[0], prm[1], prm[2], prm[3], prm[4], prm[5], prm[6], prm[7],
                     prm[8] ? vl::nn::Pooling::Average : vl::nn::Pooling::Max);
  return op.backward(DX, X, DY);
}

// rois: 5 x K values [image; u1; v1; u2; v2]; transform: 6 doubles, column-major 2x3.
int mcnref_roipool_forward(int dtype, void* y, void const* x, void const* rois, int H, int W, int C, int N,
                           int numROIs, int S0, int S1, double const* transform, int method)
{
  vl::Tensor Y = view(y, dtype, S0, S1, C, numROIs), X = view(x, dtype, H, W, C, N);
  vl::Tensor R = view(rois, dtype, 5, numROIs, 1, 1);
  std::array<int, 2> sub = {{S0, S1}};
  std::array<double, 6> tf;
  for (int i = 0; i < 6; ++i) tf[i] = transform[i];
  vl::nn::ROIPooling op(ctx(), sub, tf, method ? vl::nn::ROIPooling::Average : vl::nn::ROIPooling::Max);
  return op.forward(Y, X, R);
}

int mcnref_roipool_backward(int dtype, void* dx, void const* x, void const* rois, void const* dy, int H, int W,
                            int C, int N, int numROIs, int S0, int S1, double const* transform, int method)
{
  vl::Tensor DX = view(dx, dtype, H, W, C, N), X = view(x, dtype, H, W, C, N);
  vl::Tensor R = view(rois, dtype, 5, numROIs, 1, 1), DY = view(dy, dtype, S0, S1, C, numROIs);
  memset(dx, 0, (size_t)H * W * C * N * (dtype ? 8 : 4));
  std::array<int, 2> sub = {{S0, S1}};
  std::array<double, 6> tf;
  for (int i = 0; i < 6; ++i) tf[i] = transform[i];
  vl::nn::ROIPooling op(ctx(), sub, tf, method ? vl::nn::ROIPooling::Average : vl::nn::ROIPooling::Max);
  return op.backward(DX, X, R, DY);
}

// x: H x W x C x N; grid: 2 x Ho x Wo x Ng; y, dy: Ho x Wo x C x Ng.
int mcnref_sampler_forward(int dtype, void* y, void const* x, void const* grid, int H, int W, int C, int N,
                           int Ho, int Wo, int Ng)
{
  vl::Tensor Y = view(y, dtype, Ho, Wo, C, Ng), X = view(x, dtype, H, W, C, N);
  size_t gd[4] = {2, (size_t)Ho, (size_t)Wo, (size_t)Ng};
  vl::TensorShape gs;
  gs.setDimensions(gd, 4);  // the (dims, n) constructor is declared but never defined
  vl::DataType dt = dtype ? vl::VLDT_Double : vl::VLDT_Float;
  vl::Tensor G(gs, dt, vl::VLDT_CPU, const_cast<void*>(grid), gs.getNumElements() * vl::getDataTypeSizeInBytes(dt));
  vl::nn::BilinearSampler op(ctx());
  return op.forward(Y, X, G);
}

// dx and dgrid are zero-filled first, as the gateway does (vl_nnbilinearsampler.cu:176-181).
int mcnref_sampler_backward(int dtype, void* dx, void* dgrid, void const* x, void const* grid, void const* dy,
                            int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  size_t es = dtype ? 8 : 4;
  vl::Tensor DX = view(dx, dtype, H, W, C, N), X = view(x, dtype, H, W, C, N), DY = view(dy, dtype, Ho, Wo, C, Ng);
  size_t gd[4] = {2, (size_t)Ho, (size_t)Wo, (size_t)Ng};
  vl::TensorShape gs;
  gs.setDimensions(gd, 4);  // the (dims, n) constructor is declared but never defined
  vl::DataType dt = dtype ? vl::VLDT_Double : vl::VLDT_Float;
  vl::Tensor G(gs, dt, vl::VLDT_CPU, const_cast<void*>(grid), gs.getNumElements() * es);
  vl::Tensor DG = dgrid ? vl::Tensor(gs, dt, vl::VLDT_CPU, dgrid, gs.getNumElements() * es) : vl::Tensor();
  if (dx) memset(dx, 0, (size_t)H * W * C * N * es);
  if (dgrid) memset(dgrid, 0, gs.getNumElements() * es);
  vl::nn::BilinearSampler op(ctx());
  return op.backward(DX, DG, X, G, DY);
}

// vl::nn::LRN (bits/nnnormalize.hpp:20-44); prm = {normDepth, kappa, alpha, beta}
int mcnref_lrn_forward(int dtype, void* y, void const* x, int H, int W, int C, int N, double const* prm)
{
  vl::Tensor Y = view(y, dtype, H, W, C, N), X = view(x, dtype, H, W, C, N);
  vl::nn::LRN op(ctx(), (int)prm[0], prm[1], prm[2], prm[3]);
  return op.forward(Y, X);
}

int mcnref_lrn_backward(int dtype, void* dx, void const* x, void const* dy, int H, int W, int C, int N, double const* prm)
{
  vl::Tensor DX = view(dx, dtype, H, W, C, N), X = view(x, dtype, H, W, C, N), DY = view(dy, dtype, H, W, C, N);
  vl::nn::LRN op(ctx(), (int)prm[0], prm[1], prm[2], prm[3]);
  return op.backward(DX, X, DY);
}

}  // extern "C"
