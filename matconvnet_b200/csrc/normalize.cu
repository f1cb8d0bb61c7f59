// Blocks of the reference's other ImageNet models (AlexNet, VGG-F/M/S: examples/imagenet/cnn_imagenet_init.m:148-154,
// 392-396): cross-channel local response normalisation (vl::nn::LRN, reference bits/nnnormalize.hpp:20-44, CPU definition
// bits/nnnormalize.cu:143-400), softmax (matlab/vl_nnsoftmax.m) and dropout (matlab/vl_nndropout.m).
//
// LRN: y_t = x_t * L_t^-beta with L_t = kappa + alpha * sum of x_q^2 over the channels q in [t - m1, t + m2] that exist,
// m1 = (normDepth - 1) / 2, m2 = normDepth - m1 - 1.  One thread per (pixel, image) walks the channels, a stride of one
// plane apart, so a warp reads and writes whole lines; the window sum slides as in the CPU loop (add the square that
// enters, subtract the one that leaves).  Backward follows the CPU's three sweeps (bits/nnnormalize.cu:296-383): the term
// dz_t * L_t^-beta and the running integral over the channels of x_t * 2*alpha*beta * dz_t * L_t^(-beta-1) -- kept in the
// context's scratch, written and read back by the same thread -- then the difference of the integral over the window.
// The reference's CPU code evaluates the power with a cubic approximation of log2 and exp2 (VL_NNNORMALIZE_FAST,
// bits/nnnormalize.cu:49-125); here it is powf, which the reference's own GPU kernels use (bits/nnnormalize_gpu.cu:27-66).
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 256;

struct LrnParams { int P, C, N, m1, m2; float kappa, alpha, beta; };

__global__ void lrn_forward_kernel(float* __restrict__ y, float const* __restrict__ x, LrnParams p)
{
  size_t const total = (size_t)p.P * p.N, step = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    size_t const n = i / p.P, pix = i - n * p.P;
    float const* xp = x + pix + (size_t)p.P * p.C * n;
    float* yp = y + pix + (size_t)p.P * p.C * n;
    float acc = 0.f;
    for (int t = -p.m2; t < p.C; ++t) {
      int const tm = t - p.m1 - 1, tp = t + p.m2;
      float const am = tm >= 0 ? xp[(size_t)p.P * tm] : 0.f, ap = tp < p.C ? xp[(size_t)p.P * tp] : 0.f;
      acc += ap * ap - am * am;
      if (t >= 0) yp[(size_t)p.P * t] = xp[(size_t)p.P * t] * powf(p.kappa + p.alpha * acc, -p.beta);
    }
  }
}

__global__ void lrn_backward_kernel(float* __restrict__ dx, float* __restrict__ integral, float const* __restrict__ x,
                                    float const* __restrict__ dz, LrnParams p)
{
  size_t const total = (size_t)p.P * p.N, step = (size_t)gridDim.x * blockDim.x;
  float const ab2 = 2.f * p.alpha * p.beta;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    size_t const n = i / p.P, pix = i - n * p.P, off = pix + (size_t)p.P * p.C * n;
    float const* xp = x + off;
    float const* zp = dz + off;
    float* dp = dx + off;
    float* ip = integral + off;
    float acc = 0.f, run = 0.f;
    for (int t = -p.m2; t < p.C; ++t) {
      int const tm = t - p.m1 - 1, tp = t + p.m2;
      float const am = tm >= 0 ? xp[(size_t)p.P * tm] : 0.f, ap = tp < p.C ? xp[(size_t)p.P * tp] : 0.f;
      acc += ap * ap - am * am;
      if (t >= 0) {
        float const L = p.kappa + p.alpha * acc;
        float const temp1 = zp[(size_t)p.P * t] * powf(L, -p.beta);
        float const temp2 = xp[(size_t)p.P * t] * ab2 * temp1 / L;
        dp[(size_t)p.P * t] = temp1;
        run += temp2;
        ip[(size_t)p.P * t] = run;
      }
    }
    // the sum of temp2 over the channels q whose window holds t: q in [t - m2, t + m1]
    for (int t = 0; t < p.C; ++t) {
      int const q1 = t - p.m2 - 1, q2 = min(t + p.m1, p.C - 1);
      float s = ip[(size_t)p.P * q2];
      if (q1 >= 0) s -= ip[(size_t)p.P * q1];
      dp[(size_t)p.P * t] -= s * xp[(size_t)p.P * t];
    }
  }
}

// ---- softmax over the channels: one block per (pixel, image)
__device__ float block_reduce(float v, bool isMax, float* red)
{
  for (int o = 16; o > 0; o >>= 1) {
    float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = isMax ? fmaxf(v, u) : v + u;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  int const nw = blockDim.x >> 5;
  v = (int)threadIdx.x < nw ? red[threadIdx.x] : (isMax ? -INFINITY : 0.f);
  if (threadIdx.x < 32) {
    for (int o = 16; o > 0; o >>= 1) {
      float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = isMax ? fmaxf(v, u) : v + u;
    }
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  v = red[0];
  __syncthreads();
  return v;
}

// forward: y = exp(x - max) / sum; backward (dz != nullptr): out = y .* (dz - sum(dz .* y))   (matlab/vl_nnsoftmax.m:24-29)
__global__ void softmax_kernel(float* __restrict__ out, float const* __restrict__ x, float const* __restrict__ dz, int P, int C)
{
  __shared__ float red[32];
  size_t const off = blockIdx.x + (size_t)P * C * blockIdx.y;
  float const* xp = x + off;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, xp[(size_t)P * c]);
  m = block_reduce(m, true, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) s += expf(xp[(size_t)P * c] - m);
  s = block_reduce(s, false, red);
  float dot = 0.f;
  if (dz) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) dot += dz[off + (size_t)P * c] * (expf(xp[(size_t)P * c] - m) / s);
    dot = block_reduce(dot, false, red);
  }
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float const yv = expf(xp[(size_t)P * c] - m) / s;
    out[off + (size_t)P * c] = dz ? yv * (dz[off + (size_t)P * c] - dot) : yv;
  }
}

// ---- dropout: mask = scale * (u >= rate), u uniform in [0, 1) from a counter-based generator: element i of a call with
// seed s always gets the same number, whatever the grid
__device__ __forceinline__ uint32_t mix(uint32_t a, uint32_t b, uint32_t c)
{
  // three rounds of a multiply-xorshift finaliser over (index, seed)
  uint32_t h = a * 0x9E3779B1u ^ b * 0x85EBCA77u ^ c * 0xC2B2AE3Du;
  h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
  h += a; h ^= h >> 16; h *= 0x7FEB352Du; h ^= h >> 15; h *= 0x846CA68Bu; h ^= h >> 16;
  return h;
}

__global__ void dropout_mask_kernel(float* __restrict__ mask, size_t n, float rate, float scale, uint32_t seedLo, uint32_t seedHi)
{
  size_t const step = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    uint32_t const h = mix((uint32_t)i, (uint32_t)(i >> 32) ^ seedLo, seedHi);
    float const u = (float)(h >> 8) * (1.f / 16777216.f);       // 24 bits: every value is representable
    mask[i] = u >= rate ? scale : 0.f;
  }
}

__global__ void mul_kernel(float* y, float const* a, float const* b, size_t n)
{
  size_t const step = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) y[i] = a[i] * b[i];
}

int lrn_params(vlb_ctx* ctx, LrnParams* p, int H, int W, int C, int N, int normDepth, double kappa, double alpha, double beta)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0, "normalize: empty tensor");
  VLB_REQUIRE(ctx, normDepth >= 1, "normalize: the normalisation depth is smaller than 1");       // matlab/src/vl_nnnormalize.cu:128-130
  p->P = H * W; p->C = C; p->N = N;
  p->m1 = (normDepth - 1) / 2; p->m2 = normDepth - p->m1 - 1;
  p->kappa = (float)kappa; p->alpha = (float)alpha; p->beta = (float)beta;
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_lrn_forward(vlb_ctx* ctx, float* Y, float const* X, int H, int W, int C, int N, int normDepth, double kappa,
                    double alpha, double beta)
{
  if (!ctx) return VLB_IllegalArgument;
  LrnParams p;
  int rc = lrn_params(ctx, &p, H, W, C, N, normDepth, kappa, alpha, beta);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X, "lrn_forward: null tensor");
  lrn_forward_kernel<<<vlb::grid_for((size_t)p.P * N, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(Y, X, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_lrn_forward");
}

int vlb_lrn_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, int H, int W, int C, int N, int normDepth,
                     double kappa, double alpha, double beta)
{
  if (!ctx) return VLB_IllegalArgument;
  LrnParams p;
  int rc = lrn_params(ctx, &p, H, W, C, N, normDepth, kappa, alpha, beta);
  if (rc) return rc;
  VLB_REQUIRE(ctx, dX && X && dY, "lrn_backward: null tensor");
  float* integral = (float*)vlb::workspace(ctx, sizeof(float) * (size_t)p.P * C * N);
  if (!integral) return vlb::pass_error(ctx, ctx->lastError, "vlb_lrn_backward");
  lrn_backward_kernel<<<vlb::grid_for((size_t)p.P * N, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(dX, integral, X, dY, p);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_lrn_backward");
}

int vlb_softmax_forward(vlb_ctx* ctx, float* Y, float const* X, int H, int W, int C, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y && X, "softmax_forward: null tensor");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && N <= 65535, "softmax_forward: bad shape");
  int const threads = C >= 256 ? 256 : (C >= 64 ? 64 : 32);
  softmax_kernel<<<dim3(H * W, N), threads, 0, ctx->stream>>>(Y, X, nullptr, H * W, C);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_softmax_forward");
}

int vlb_softmax_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, int H, int W, int C, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, dX && X && dY, "softmax_backward: null tensor");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && N <= 65535, "softmax_backward: bad shape");
  int const threads = C >= 256 ? 256 : (C >= 64 ? 64 : 32);
  softmax_kernel<<<dim3(H * W, N), threads, 0, ctx->stream>>>(dX, X, dY, H * W, C);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_softmax_backward");
}

int vlb_dropout_mask(vlb_ctx* ctx, float* mask, size_t n, double rate, unsigned long long seed)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, mask, "dropout_mask: null tensor");
  VLB_REQUIRE(ctx, rate >= 0.0 && rate < 1.0, "dropout_mask: RATE must be in [0, 1)");
  if (n == 0) return VLB_Success;
  float const scale = (float)(1.0 / (1.0 - rate));         // scale = 1 / (1 - rate), converted to single (matlab/vl_nndropout.m:44-56)
  dropout_mask_kernel<<<vlb::grid_for(n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(
      mask, n, (float)rate, scale, (uint32_t)seed, (uint32_t)(seed >> 32));
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_dropout_mask");
}

int vlb_mul(vlb_ctx* ctx, float* Y, float const* A, float const* B, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y && A && B, "mul: null tensor");
  if (n == 0) return VLB_Success;
  mul_kernel<<<vlb::grid_for(n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(Y, A, B, n);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_mul");
}

}  // extern "C"
