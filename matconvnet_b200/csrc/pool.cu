// Max / average pooling, forward and backward (vl::nn::Pooling,
// reference bits/nnpooling.hpp:21-49; CPU definition bits/nnpooling.cu:102-214).
//
// HBM-bound.  Two families:
//  * non-overlapping 2x2 / stride 2 / no pad on even H and W (every pooling layer of
//    VGG-16): each thread owns whole windows, so the backward pass REPLAYS the argmax
//    scan and overwrites dx with 64/128-bit stores -- no atomics, no zero fill, no
//    scratch; algorithmic traffic 4*(2*in + out) bytes is also the real traffic.
//  * everything else: forward = one thread per output; backward = one thread per
//    INPUT element gathering from the windows that cover it, visited in the
//    reference's order (wo outer, ho inner), so sums are formed in the same order as
//    on the CPU and the result is bit-identical and run-to-run deterministic.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 256;

struct PoolParams {
  int H, W, Ho, Wo;
  int poolH, poolW, strideY, strideX, padTop, padLeft;
  size_t planes;   // C * N
};

// ------------------------------------------------------------------ generic forward
template <bool kMax>
__global__ void pool_fwd_generic(float* __restrict__ y, float const* __restrict__ x, PoolParams p)
{
  size_t total = p.planes * (size_t)p.Ho * p.Wo;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int ho = (int)(i % p.Ho);
    size_t t = i / p.Ho;
    int wo = (int)(t % p.Wo);
    size_t z = t / p.Wo;
    int x1 = wo * p.strideX - p.padLeft, y1 = ho * p.strideY - p.padTop;
    int x2 = min(x1 + p.poolW, p.W), y2 = min(y1 + p.poolH, p.H);
    x1 = max(x1, 0); y1 = max(y1, 0);
    float const* xz = x + z * (size_t)p.H * p.W;
    if (kMax) {
      float best = -INFINITY;
      for (int u = x1; u < x2; ++u)
        for (int v = y1; v < y2; ++v) { float a = xz[(size_t)u * p.H + v]; best = (best < a) ? a : best; }
      y[i] = best;
    } else {
      float s = 0.f;
      for (int u = x1; u < x2; ++u)
        for (int v = y1; v < y2; ++v) s = __fadd_rn(s, xz[(size_t)u * p.H + v]);
      float scale = __fdiv_rn(1.f, (float)((y2 - y1) * (x2 - x1)));
      y[i] = __fmul_rn(s, scale);
    }
  }
}

// ------------------------------------------------------------------ generic backward (gather)
// Thread per input element (v = row, u = column, plane z).  Windows covering it:
// ho in [ceil((v + padTop - poolH + 1)/strideY), floor((v + padTop)/strideY)], likewise wo.
__device__ __forceinline__ int floor_div(int a, int b) { int q = a / b; return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q; }
__device__ __forceinline__ int ceil_div_i(int a, int b) { return -floor_div(-a, b); }

// relu: x is the output of a ReLU and dx the derivative with respect to that ReLU's input: zero where x is not positive.
template <bool kMax>
__global__ void pool_bwd_generic(float* __restrict__ dx, float const* __restrict__ x,
                                 float const* __restrict__ dy, PoolParams p, bool relu)
{
  size_t total = p.planes * (size_t)p.H * p.W;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int v = (int)(i % p.H);
    size_t t = i / p.H;
    int u = (int)(t % p.W);
    size_t z = t / p.W;
    int ho0 = max(ceil_div_i(v + p.padTop - p.poolH + 1, p.strideY), 0);
    int ho1 = min(floor_div(v + p.padTop, p.strideY), p.Ho - 1);
    int wo0 = max(ceil_div_i(u + p.padLeft - p.poolW + 1, p.strideX), 0);
    int wo1 = min(floor_div(u + p.padLeft, p.strideX), p.Wo - 1);
    float const* xz = x + z * (size_t)p.H * p.W;
    float const* dyz = dy + z * (size_t)p.Ho * p.Wo;
    float acc = 0.f;
    for (int wo = wo0; wo <= wo1; ++wo)
      for (int ho = ho0; ho <= ho1; ++ho) {
        int x1 = wo * p.strideX - p.padLeft, y1 = ho * p.strideY - p.padTop;
        int x2 = min(x1 + p.poolW, p.W), y2 = min(y1 + p.poolH, p.H);
        x1 = max(x1, 0); y1 = max(y1, 0);
        float d = dyz[(size_t)wo * p.Ho + ho];
        if (kMax) {
          // Replay the reference scan: column-outer, row-inner, first strictly greater wins.
          float best = -INFINITY;
          int bu = -1, bv = -1;
          for (int uu = x1; uu < x2; ++uu)
            for (int vv = y1; vv < y2; ++vv) {
              float a = xz[(size_t)uu * p.H + vv];
              if (a > best) { best = a; bu = uu; bv = vv; }
            }
          if (bu == u && bv == v) acc = __fadd_rn(acc, d);
        } else {
          float scale = __fdiv_rn(1.f, (float)((y2 - y1) * (x2 - x1)));
          acc = __fadd_rn(acc, __fmul_rn(d, scale));
        }
      }
    if (relu) acc = xz[(size_t)u * p.H + v] > 0.f ? acc : 0.f;
    dx[i] = acc;
  }
}

// ------------------------------------------------------------------ 2x2 / stride 2 fast path
// kV outputs (consecutive ho) per thread; loads 2*kV floats from each of the two columns.
template <int kV> struct VecT;
template <> struct VecT<1> { typedef float2 in_t; typedef float out_t; };
template <> struct VecT<2> { typedef float4 in_t; typedef float2 out_t; };

__device__ __forceinline__ void unpack(float2 v, float* o) { o[0] = v.x; o[1] = v.y; }
__device__ __forceinline__ void unpack(float4 v, float* o) { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
__device__ __forceinline__ void pack(float2& v, float const* o) { v.x = o[0]; v.y = o[1]; }
__device__ __forceinline__ void pack(float4& v, float const* o) { v.x = o[0]; v.y = o[1]; v.z = o[2]; v.w = o[3]; }
__device__ __forceinline__ void unpack(float v, float* o) { o[0] = v; }
__device__ __forceinline__ void pack(float& v, float const* o) { v = o[0]; }

template <int kV, bool kMax>
__global__ void pool2x2_fwd(float* __restrict__ y, float const* __restrict__ x, int H, int W, size_t planes)
{
  typedef typename VecT<kV>::in_t in_t;
  typedef typename VecT<kV>::out_t out_t;
  int Ho = H >> 1, Wo = W >> 1, Hv = Ho / kV;
  size_t total = planes * (size_t)Wo * Hv;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int hv = (int)(i % Hv);
    size_t col = i / Hv;                       // = wo + Wo * z
    size_t z = col / Wo;
    int wo = (int)(col - z * Wo);
    float const* base = x + (z * W + 2 * (size_t)wo) * H + 2 * kV * (size_t)hv;
    float a[2 * kV], b[2 * kV], o[kV];
    unpack(*reinterpret_cast<in_t const*>(base), a);
    unpack(*reinterpret_cast<in_t const*>(base + H), b);
#pragma unroll
    for (int j = 0; j < kV; ++j) {
      if (kMax) {
        float best = -INFINITY;
        best = (best < a[2 * j]) ? a[2 * j] : best;
        best = (best < a[2 * j + 1]) ? a[2 * j + 1] : best;
        best = (best < b[2 * j]) ? b[2 * j] : best;
        best = (best < b[2 * j + 1]) ? b[2 * j + 1] : best;
        o[j] = best;
      } else {
        float s = __fadd_rn(__fadd_rn(__fadd_rn(a[2 * j], a[2 * j + 1]), b[2 * j]), b[2 * j + 1]);
        o[j] = __fmul_rn(s, 0.25f);
      }
    }
    out_t ov;
    pack(ov, o);
    *reinterpret_cast<out_t*>(y + col * Ho + kV * (size_t)hv) = ov;
  }
}

template <int kV, bool kMax, bool kRelu>
__global__ void pool2x2_bwd(float* __restrict__ dx, float const* __restrict__ x, float const* __restrict__ dy,
                            int H, int W, size_t planes)
{
  typedef typename VecT<kV>::in_t in_t;
  typedef typename VecT<kV>::out_t out_t;
  int Ho = H >> 1, Wo = W >> 1, Hv = Ho / kV;
  size_t total = planes * (size_t)Wo * Hv;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int hv = (int)(i % Hv);
    size_t col = i / Hv;
    size_t z = col / Wo;
    int wo = (int)(col - z * Wo);
    size_t off = (z * W + 2 * (size_t)wo) * H + 2 * kV * (size_t)hv;
    float d[kV], ra[2 * kV], rb[2 * kV];
    unpack(*reinterpret_cast<out_t const*>(dy + col * Ho + kV * (size_t)hv), d);
    float a[2 * kV], b[2 * kV];
    if (kMax || kRelu) {
      unpack(*reinterpret_cast<in_t const*>(x + off), a);
      unpack(*reinterpret_cast<in_t const*>(x + off + H), b);
    }
    if (kMax) {
#pragma unroll
      for (int j = 0; j < kV; ++j) {
        // scan order of the reference: column 0 rows 0,1 then column 1 rows 0,1; strict '>'
        float best = -INFINITY;
        int w = -1;
        if (a[2 * j] > best) { best = a[2 * j]; w = 0; }
        if (a[2 * j + 1] > best) { best = a[2 * j + 1]; w = 1; }
        if (b[2 * j] > best) { best = b[2 * j]; w = 2; }
        if (b[2 * j + 1] > best) { best = b[2 * j + 1]; w = 3; }
        float g = __fadd_rn(0.f, d[j]);   // the reference adds dy to a zero-filled dx: -0 becomes +0
        ra[2 * j] = (w == 0) ? g : 0.f;
        ra[2 * j + 1] = (w == 1) ? g : 0.f;
        rb[2 * j] = (w == 2) ? g : 0.f;
        rb[2 * j + 1] = (w == 3) ? g : 0.f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kV; ++j) {
        float g = __fadd_rn(0.f, __fmul_rn(d[j], 0.25f));
        ra[2 * j] = g; ra[2 * j + 1] = g; rb[2 * j] = g; rb[2 * j + 1] = g;
      }
    }
    if (kRelu) {
#pragma unroll
      for (int j = 0; j < 2 * kV; ++j) { ra[j] = a[j] > 0.f ? ra[j] : 0.f; rb[j] = b[j] > 0.f ? rb[j] : 0.f; }
    }
    in_t va, vb;
    pack(va, ra);
    pack(vb, rb);
    *reinterpret_cast<in_t*>(dx + off) = va;
    *reinterpret_cast<in_t*>(dx + off + H) = vb;
  }
}

bool fast2x2(vlb_pool_desc const* d, void const* a, void const* b, void const* c)
{
  bool shape = d->poolH == 2 && d->poolW == 2 && d->strideY == 2 && d->strideX == 2 && d->padTop == 0 &&
               d->padBottom == 0 && d->padLeft == 0 && d->padRight == 0 && (d->H % 2 == 0) && (d->W % 2 == 0);
  uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c;
  return shape && (bits & 15) == 0;
}

int validate(vlb_ctx* ctx, vlb_pool_desc const* d, int* Ho, int* Wo)
{
  VLB_REQUIRE(ctx, d, "pooling: null descriptor");
  VLB_REQUIRE(ctx, d->H > 0 && d->W > 0 && d->C > 0 && d->N > 0, "pooling: empty input");
  VLB_REQUIRE(ctx, d->poolH >= 1 && d->poolW >= 1, "pooling: POOL has a dimension smaller than 1");
  VLB_REQUIRE(ctx, d->strideY >= 1 && d->strideX >= 1, "pooling: STRIDE smaller than 1");
  VLB_REQUIRE(ctx, d->padTop >= 0 && d->padBottom >= 0 && d->padLeft >= 0 && d->padRight >= 0, "pooling: negative PAD");
  VLB_REQUIRE(ctx, d->H + d->padTop + d->padBottom >= d->poolH && d->W + d->padLeft + d->padRight >= d->poolW,
              "pooling: pooling window larger than the padded input");
  // The gateway rejects a padding as large as the window (matlab/src/vl_nnpool.cu:232-237).
  VLB_REQUIRE(ctx, d->padTop < d->poolH && d->padBottom < d->poolH && d->padLeft < d->poolW && d->padRight < d->poolW,
              "pooling: padding larger or equal than the pooling window");
  VLB_REQUIRE(ctx, d->method == VLB_POOL_MAX || d->method == VLB_POOL_AVG, "pooling: unknown method");
  vlb_pool_output_shape(d, Ho, Wo);
  return VLB_Success;
}

}  // namespace

namespace {

template <int kV, bool kMax>
void launch2x2_bwd(vlb_ctx* ctx, unsigned grid, float* dX, float const* X, float const* dY, int H, int W, size_t planes, bool relu)
{
  if (relu) pool2x2_bwd<kV, kMax, true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, dY, H, W, planes);
  else      pool2x2_bwd<kV, kMax, false><<<grid, kThreads, 0, ctx->stream>>>(dX, X, dY, H, W, planes);
}

int pool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, vlb_pool_desc const* d, bool relu, char const* where)
{
  if (!ctx) return VLB_IllegalArgument;
  int Ho, Wo;
  int rc = validate(ctx, d, &Ho, &Wo);
  if (rc) return vlb::pass_error(ctx, rc, where);
  VLB_REQUIRE(ctx, dX && X && dY, "pool_backward: null tensor");
  size_t planes = (size_t)d->C * d->N;
  bool isMax = d->method == VLB_POOL_MAX;
  if (fast2x2(d, dX, X, dY)) {
    bool v2 = (d->H % 4 == 0);
    size_t total = planes * (size_t)Wo * (v2 ? Ho / 2 : Ho);
    unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
    if (v2) { if (isMax) launch2x2_bwd<2, true>(ctx, grid, dX, X, dY, d->H, d->W, planes, relu);
              else       launch2x2_bwd<2, false>(ctx, grid, dX, X, dY, d->H, d->W, planes, relu); }
    else    { if (isMax) launch2x2_bwd<1, true>(ctx, grid, dX, X, dY, d->H, d->W, planes, relu);
              else       launch2x2_bwd<1, false>(ctx, grid, dX, X, dY, d->H, d->W, planes, relu); }
  } else {
    PoolParams p = {d->H, d->W, Ho, Wo, d->poolH, d->poolW, d->strideY, d->strideX, d->padTop, d->padLeft, planes};
    unsigned grid = vlb::grid_for(planes * (size_t)d->H * d->W, kThreads, ctx->smCount * 16);
    if (isMax) pool_bwd_generic<true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, dY, p, relu);
    else       pool_bwd_generic<false><<<grid, kThreads, 0, ctx->stream>>>(dX, X, dY, p, relu);
  }
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, where);
}

}  // namespace

extern "C" {

int vlb_pool_output_shape(vlb_pool_desc const* d, int* Ho, int* Wo)
{
  if (!d) return VLB_IllegalArgument;
  if (Ho) *Ho = (d->H + d->padTop + d->padBottom - d->poolH) / d->strideY + 1;
  if (Wo) *Wo = (d->W + d->padLeft + d->padRight - d->poolW) / d->strideX + 1;
  return VLB_Success;
}

int vlb_pool_forward(vlb_ctx* ctx, float* Y, float const* X, vlb_pool_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  int Ho, Wo;
  int rc = validate(ctx, d, &Ho, &Wo);
  if (rc) return vlb::pass_error(ctx, rc, "vlb_pool_forward");
  VLB_REQUIRE(ctx, Y && X, "pool_forward: null tensor");
  size_t planes = (size_t)d->C * d->N;
  bool isMax = d->method == VLB_POOL_MAX;
  if (fast2x2(d, Y, X, X)) {
    bool v2 = (d->H % 4 == 0);
    size_t total = planes * (size_t)Wo * (v2 ? Ho / 2 : Ho);
    unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
    if (v2) { if (isMax) pool2x2_fwd<2, true><<<grid, kThreads, 0, ctx->stream>>>(Y, X, d->H, d->W, planes);
              else       pool2x2_fwd<2, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, d->H, d->W, planes); }
    else    { if (isMax) pool2x2_fwd<1, true><<<grid, kThreads, 0, ctx->stream>>>(Y, X, d->H, d->W, planes);
              else       pool2x2_fwd<1, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, d->H, d->W, planes); }
  } else {
    PoolParams p = {d->H, d->W, Ho, Wo, d->poolH, d->poolW, d->strideY, d->strideX, d->padTop, d->padLeft, planes};
    unsigned grid = vlb::grid_for(planes * (size_t)Ho * Wo, kThreads, ctx->smCount * 16);
    if (isMax) pool_fwd_generic<true><<<grid, kThreads, 0, ctx->stream>>>(Y, X, p);
    else       pool_fwd_generic<false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, p);
  }
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_pool_forward");
}

int vlb_pool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, vlb_pool_desc const* d)
{
  return pool_backward(ctx, dX, X, dY, d, false, "vlb_pool_backward");
}

int vlb_relu_pool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, vlb_pool_desc const* d)
{
  return pool_backward(ctx, dX, X, dY, d, true, "vlb_relu_pool_backward");
}

}  // extern "C"
