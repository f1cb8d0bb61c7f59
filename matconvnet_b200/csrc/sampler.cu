// Bilinear sampler (vl::nn::BilinearSampler, reference bits/nnbilinearsampler.hpp:21-36;
// CPU definition bits/nnbilinearsampler.cu:32-149).
//
// One thread per output pixel (q = ho + Ho*wo, grid n) walks the C channels: the grid
// entry and the four tap weights are computed once and reused for every channel; reads
// of dy and writes of y are contiguous across the warp; x taps of neighbouring output
// pixels fall in the same or adjacent 32-byte sectors.  Backward-to-data scatters with
// atomicAdd (footprints of different outputs overlap); backward-to-grid accumulates
// the channels in ascending order in a register, the order of the CPU loop, and writes
// each grid entry once.  dx and dgrid are overwritten: dx is cleared first, dgrid is
// written whole.
//
// Boundary rule of the CPU reference, kept as it is: the taps are guarded by
// `-1 <= sy && sy < inHeight` with inHeight a size_t (bits/nnbilinearsampler.cu:92), so
// sy == -1 is compared as a huge unsigned number and fails: samples whose floor is -1
// in either coordinate contribute nothing.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 128;

struct Taps {
  int sx, sy;
  float wx, wy;
  bool inside;
};

__device__ __forceinline__ Taps make_taps(float gy, float gx, int H, int W)
{
  Taps t;
  float py = __fmul_rn(__fmul_rn(0.5f, __fadd_rn(gy, 1.f)), (float)(H - 1));
  float px = __fmul_rn(__fmul_rn(0.5f, __fadd_rn(gx, 1.f)), (float)(W - 1));
  float fx = floorf(px), fy = floorf(py);
  // keep the int conversion defined for wild grid values
  fx = fminf(fmaxf(fx, -2.f), (float)W + 1.f);
  fy = fminf(fmaxf(fy, -2.f), (float)H + 1.f);
  t.sx = (int)fx; t.sy = (int)fy;
  t.inside = (t.sy >= 0 && t.sy < H && t.sx >= 0 && t.sx < W);
  t.wx = __fadd_rn(px, -(float)t.sx);
  t.wy = __fadd_rn(py, -(float)t.sy);
  return t;
}

// mode 0: forward.  mode 1: backward (dx and/or dgrid).
template <int kMode>
__global__ void sampler_kernel(float* __restrict__ y, float* __restrict__ dx, float* __restrict__ dgrid,
                               float const* __restrict__ x, float const* __restrict__ grid,
                               float const* __restrict__ dy, int H, int W, int C, int N, int Q, int Ng)
{
  int group = Ng / N;
  size_t total = (size_t)Q * Ng;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int q = (int)(i % Q);
    int n = (int)(i / Q);
    float2 gv = reinterpret_cast<float2 const*>(grid)[i];
    Taps t = make_taps(gv.x, gv.y, H, W);
    // tap (i = row offset, j = column offset); weights as in bits/nnbilinearsampler.cu:108-110
    float wwx[2] = {__fadd_rn(1.f, -t.wx), t.wx};
    float wwy[2] = {__fadd_rn(1.f, -t.wy), t.wy};
    bool ok[2][2];
    int idx[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        int ssy = t.sy + ii, ssx = t.sx + j;
        ok[j][ii] = t.inside && ssy >= 0 && ssy < H && ssx >= 0 && ssx < W;
        idx[j][ii] = ssy + ssx * H;
      }
    size_t imgOff = (size_t)H * W * C * (size_t)(n / group);
    float const* xz = x + imgOff;
    float* dxz = (kMode == 1 && dx) ? dx + imgOff : nullptr;
    size_t outOff = (size_t)q + (size_t)Q * C * (size_t)n;
    float accGy = 0.f, accGx = 0.f;
    for (int c = 0; c < C; ++c) {
      if (kMode == 0) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int ii = 0; ii < 2; ++ii)
            if (ok[j][ii]) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(wwx[j], wwy[ii]), xz[idx[j][ii]]));
        y[outOff] = acc;
      } else {
        float d = dy[outOff];
        float dgx = 0.f, dgy = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int ii = 0; ii < 2; ++ii)
            if (ok[j][ii]) {
              if (dxz) atomicAdd(dxz + idx[j][ii], __fmul_rn(__fmul_rn(wwx[j], wwy[ii]), d));
              if (dgrid) {
                float xv = xz[idx[j][ii]];
                float sj = j ? 1.f : -1.f, si = ii ? 1.f : -1.f;
                dgx = __fadd_rn(dgx, __fmul_rn(__fmul_rn(__fmul_rn(sj, wwy[ii]), d), xv));
                dgy = __fadd_rn(dgy, __fmul_rn(__fmul_rn(__fmul_rn(si, wwx[j]), d), xv));
              }
            }
        if (dgrid) {
          accGy = __fadd_rn(accGy, __fmul_rn(__fmul_rn(0.5f, (float)(H - 1)), dgy));
          accGx = __fadd_rn(accGx, __fmul_rn(__fmul_rn(0.5f, (float)(W - 1)), dgx));
        }
      }
      xz += (size_t)H * W;
      if (dxz) dxz += (size_t)H * W;
      outOff += Q;
    }
    if (kMode == 1 && dgrid) reinterpret_cast<float2*>(dgrid)[i] = make_float2(accGy, accGx);
  }
}

int validate(vlb_ctx* ctx, int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && Ho > 0 && Wo > 0 && Ng > 0, "bilinearsampler: empty tensor");
  // GRID must hold a whole number of grids per image (matlab/src/vl_nnbilinearsampler.cu:141-146)
  VLB_REQUIRE(ctx, Ng % N == 0, "bilinearsampler: the number of grids is not a multiple of the number of images");
  VLB_REQUIRE(ctx, (long long)H * W < (1LL << 31) && (long long)Ho * Wo < (1LL << 31), "bilinearsampler: plane too large");
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_sampler_forward(vlb_ctx* ctx, float* Y, float const* X, float const* grid, int H, int W, int C, int N,
                        int Ho, int Wo, int Ng)
{
  if (!ctx) return VLB_IllegalArgument;
  int rc = validate(ctx, H, W, C, N, Ho, Wo, Ng);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X && grid, "sampler_forward: null tensor");
  VLB_REQUIRE(ctx, (((uintptr_t)grid) & 7) == 0, "sampler_forward: grid must be 8-byte aligned");
  size_t total = (size_t)Ho * Wo * Ng;
  sampler_kernel<0><<<vlb::grid_for(total, kThreads, ctx->smCount * 32), kThreads, 0, ctx->stream>>>(
      Y, nullptr, nullptr, X, grid, nullptr, H, W, C, N, Ho * Wo, Ng);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sampler_forward");
}

int vlb_sampler_backward(vlb_ctx* ctx, float* dX, float* dGrid, float const* X, float const* grid, float const* dY,
                         int H, int W, int C, int N, int Ho, int Wo, int Ng)
{
  if (!ctx) return VLB_IllegalArgument;
  int rc = validate(ctx, H, W, C, N, Ho, Wo, Ng);
  if (rc) return rc;
  VLB_REQUIRE(ctx, grid && dY, "sampler_backward: null tensor");
  VLB_REQUIRE(ctx, !dGrid || X, "sampler_backward: the grid derivative needs the input");
  VLB_REQUIRE(ctx, ((((uintptr_t)grid) | ((uintptr_t)dGrid)) & 7) == 0, "sampler_backward: grid must be 8-byte aligned");
  if (!dX && !dGrid) return VLB_Success;
  if (dX) {
    cudaError_t e = cudaMemsetAsync(dX, 0, sizeof(float) * (size_t)H * W * C * N, ctx->stream);
    if (e != cudaSuccess) return vlb::set_error(ctx, VLB_Cuda, cudaGetErrorString(e));
  }
  size_t total = (size_t)Ho * Wo * Ng;
  sampler_kernel<1><<<vlb::grid_for(total, kThreads, ctx->smCount * 32), kThreads, 0, ctx->stream>>>(
      nullptr, dX, dGrid, X, grid, dY, H, W, C, N, Ho * Wo, Ng);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sampler_backward");
}

}  // extern "C"
