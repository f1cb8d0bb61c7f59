// ROI pooling (vl::nn::ROIPooling, reference bits/nnroipooling.hpp:23-45; CPU definition
// bits/nnroipooling.cu:102-189 forward, :217-305 backward).
//
// The bin geometry follows the CPU reference's arithmetic exactly -- affine map in
// double rounded to float, round-half-away, bin size as a double quotient rounded to
// float, float products with floor/ceil (bits/nnroipooling.cu:129-165) -- using the
// _rn intrinsics so that no multiply-add is contracted; the reference's own GPU code
// does the same maths in float throughout and can differ in the last place.
// One thread per output bin; adjacent threads take adjacent ph, so reads of a bin
// column are contiguous.  Backward scatters with atomics because ROIs overlap; the
// scan order for the arg-max is the CPU's (w outer, h inner, first strictly greater).
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 256;

struct RoiParams {
  int H, W, C, N, numROIs, S0, S1;
  double tf[6];
};

struct RoiGeom { int image, start_h, start_w; float bin_h, bin_w; };

__device__ __forceinline__ RoiGeom roi_geom(float const* r, RoiParams const& p)
{
  RoiGeom g;
  double u1_ = (double)r[1], v1_ = (double)r[2], u2_ = (double)r[3], v2_ = (double)r[4];
  // (tf0*u + tf2*v) + tf4, each step rounded to double: no fused multiply-add
  float u1 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[0], u1_), __dmul_rn(p.tf[2], v1_)), p.tf[4]);
  float v1 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[1], u1_), __dmul_rn(p.tf[3], v1_)), p.tf[5]);
  float u2 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[0], u2_), __dmul_rn(p.tf[2], v2_)), p.tf[4]);
  float v2 = (float)__dadd_rn(__dadd_rn(__dmul_rn(p.tf[1], u2_), __dmul_rn(p.tf[3], v2_)), p.tf[5]);
  int image = (int)r[0];
  // ::round on the float promoted to double (bits/nnroipooling.cu:137-140)
  g.start_h = (int)round((double)v1) - 1;
  g.start_w = (int)round((double)u1) - 1;
  int end_h = (int)round((double)v2) - 1, end_w = (int)round((double)u2) - 1;
  int rh = max(end_h - g.start_h + 1, 1), rw = max(end_w - g.start_w + 1, 1);
  g.image = min(max(image - 1, 0), p.N - 1);
  g.bin_h = (float)((double)rh / (double)p.S0);
  g.bin_w = (float)((double)rw / (double)p.S1);
  return g;
}

__device__ __forceinline__ void roi_bin(int q, float bin, int start, int extent, int& lo, int& hi)
{
  int a = (int)floorf(__fmul_rn((float)q, bin));
  int b = (int)ceilf(__fmul_rn((float)(q + 1), bin));
  lo = min(max(a + start, 0), extent);
  hi = min(max(b + start, 0), extent);
}

__global__ void roipool_bounds_kernel(int* __restrict__ bounds, int* __restrict__ images,
                                      float const* __restrict__ rois, RoiParams p)
{
  int total = p.S0 * p.S1 * p.numROIs;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    int ph = i % p.S0, pw = (i / p.S0) % p.S1, r = i / (p.S0 * p.S1);
    RoiGeom g = roi_geom(rois + 5 * (size_t)r, p);
    int hs, he, ws, we;
    roi_bin(ph, g.bin_h, g.start_h, p.H, hs, he);
    roi_bin(pw, g.bin_w, g.start_w, p.W, ws, we);
    bounds[4 * (size_t)i + 0] = hs; bounds[4 * (size_t)i + 1] = he;
    bounds[4 * (size_t)i + 2] = ws; bounds[4 * (size_t)i + 3] = we;
    if (images && ph == 0 && pw == 0) images[r] = g.image;
  }
}

// kBackward = false: y[bin] = max / mean.  kBackward = true: dx += routed dy.
template <bool kMax, bool kBackward>
__global__ void roipool_kernel(float* __restrict__ out, float const* __restrict__ x,
                               float const* __restrict__ rois, float const* __restrict__ dy, RoiParams p)
{
  size_t total = (size_t)p.S0 * p.S1 * p.C * p.numROIs;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int ph = (int)(i % p.S0);
    size_t t = i / p.S0;
    int pw = (int)(t % p.S1); t /= p.S1;
    int c = (int)(t % p.C);
    int r = (int)(t / p.C);
    RoiGeom g = roi_geom(rois + 5 * (size_t)r, p);
    int hs, he, ws, we;
    roi_bin(ph, g.bin_h, g.start_h, p.H, hs, he);
    roi_bin(pw, g.bin_w, g.start_w, p.W, ws, we);
    size_t off = (size_t)p.H * p.W * ((size_t)c + (size_t)p.C * g.image);
    float const* xz = x + off;
    bool empty = (he <= hs) || (we <= ws);
    if (!kBackward) {
      float o = 0.f;
      if (!empty) {
        if (kMax) {
          float best = -INFINITY;
          for (int w = ws; w < we; ++w)
            for (int h = hs; h < he; ++h) { float a = xz[(size_t)w * p.H + h]; best = (best < a) ? a : best; }
          o = best;
        } else {
          float s = 0.f;
          for (int w = ws; w < we; ++w)
            for (int h = hs; h < he; ++h) s = __fadd_rn(s, xz[(size_t)w * p.H + h]);
          o = __fmul_rn(s, __fdiv_rn(1.f, (float)((he - hs) * (we - ws))));
        }
      }
      out[i] = o;
    } else {
      if (empty) continue;
      float d = dy[i];
      float* dxz = out + off;
      if (kMax) {
        float best = -INFINITY;
        long where = -1;
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) {
            float a = xz[(size_t)w * p.H + h];
            if (a > best) { best = a; where = (long)w * p.H + h; }
          }
        if (where >= 0) atomicAdd(dxz + where, d);
      } else {
        float g2 = __fmul_rn(d, __fdiv_rn(1.f, (float)((he - hs) * (we - ws))));
        for (int w = ws; w < we; ++w)
          for (int h = hs; h < he; ++h) atomicAdd(dxz + (size_t)w * p.H + h, g2);
      }
    }
  }
}

int make_params(vlb_ctx* ctx, RoiParams* p, int H, int W, int C, int N, int numROIs, int S0, int S1,
                double const* tf, int method)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0, "roipool: empty input");
  VLB_REQUIRE(ctx, numROIs >= 0, "roipool: negative ROI count");
  VLB_REQUIRE(ctx, S0 >= 1 && S1 >= 1, "roipool: SUBDIVISIONS has a dimension smaller than 1");
  VLB_REQUIRE(ctx, tf != nullptr, "roipool: null transform");
  VLB_REQUIRE(ctx, method == VLB_POOL_MAX || method == VLB_POOL_AVG, "roipool: unknown method");
  p->H = H; p->W = W; p->C = C; p->N = N; p->numROIs = numROIs; p->S0 = S0; p->S1 = S1;
  for (int i = 0; i < 6; ++i) p->tf[i] = tf[i];
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_roipool_bounds(vlb_ctx* ctx, int* bounds, int* images, float const* rois, int H, int W, int N,
                       int numROIs, int S0, int S1, double const* transform)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, 1, N, numROIs, S0, S1, transform, VLB_POOL_MAX);
  if (rc) return rc;
  VLB_REQUIRE(ctx, bounds && rois, "roipool_bounds: null tensor");
  if (numROIs == 0) return VLB_Success;
  roipool_bounds_kernel<<<vlb::grid_for((size_t)S0 * S1 * numROIs, kThreads), kThreads, 0, ctx->stream>>>(bounds, images, rois, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_bounds");
}

int vlb_roipool_forward(vlb_ctx* ctx, float* Y, float const* X, float const* rois, int H, int W, int C, int N,
                        int numROIs, int S0, int S1, double const* transform, int method)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, C, N, numROIs, S0, S1, transform, method);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X && rois, "roipool_forward: null tensor");
  if (numROIs == 0) return VLB_Success;
  size_t total = (size_t)S0 * S1 * C * numROIs;
  unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
  if (method == VLB_POOL_MAX) roipool_kernel<true, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, rois, nullptr, p);
  else                        roipool_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, rois, nullptr, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_forward");
}

int vlb_roipool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* rois, float const* dY, int H, int W,
                         int C, int N, int numROIs, int S0, int S1, double const* transform, int method)
{
  if (!ctx) return VLB_IllegalArgument;
  RoiParams p;
  int rc = make_params(ctx, &p, H, W, C, N, numROIs, S0, S1, transform, method);
  if (rc) return rc;
  VLB_REQUIRE(ctx, dX && X && rois && dY, "roipool_backward: null tensor");
  cudaError_t e = cudaMemsetAsync(dX, 0, sizeof(float) * (size_t)H * W * C * N, ctx->stream);
  if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  if (numROIs == 0) return VLB_Success;
  size_t total = (size_t)S0 * S1 * C * numROIs;
  unsigned grid = vlb::grid_for(total, kThreads, ctx->smCount * 16);
  if (method == VLB_POOL_MAX) roipool_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, rois, dY, p);
  else                        roipool_kernel<false, true><<<grid, kThreads, 0, ctx->stream>>>(dX, X, rois, dY, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_roipool_backward");
}

}  // extern "C"
