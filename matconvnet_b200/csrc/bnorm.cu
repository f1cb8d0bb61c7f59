// Batch normalisation (vl::nn::BatchNorm, reference bits/nnbnorm.hpp:22-59;
// CPU definition bits/nnbnorm.cu:46-164).
//
// HBM-bound.  The regular entry points run one fused launch (bnorm_fused_kernel below: reduce, derive the
// coefficients, apply, all by the cluster that owns the channel); forward with given moments and the
// allocation-free entry point use the separate passes:
//   1. reduce: per channel sum(x), sum(x^2) [, sum(dy*x), sum(dy)].  A channel is split
//      across a thread-block CLUSTER of kCluster CTAs (C alone would leave most of the
//      148 SMs idle: the reference launches exactly C blocks, bits/nnbnorm_gpu.cu:1113).
//      Each CTA sweeps its share with 128-bit loads, reduces with warp shuffles, and the
//      cluster's rank-0 CTA gathers the kCluster partials through distributed shared
//      memory in rank order and finishes the per-channel arithmetic in the reference's
//      order (bits/nnbnorm.cu:126-133).  No scratch memory, no atomics, deterministic.
//   2. apply: y or dx, element-wise with the per-channel coefficients.
// Algorithmic traffic of backward: 8*m*C bytes (pass 1) + 12*m*C bytes (pass 2), m = H*W*N.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>

namespace cg = cooperative_groups;

namespace {

constexpr int kCluster = 8;
constexpr int kThreads = 256;

// stats layout handed from pass 1 to pass 2 (device memory, 4*C floats):
// [0,C) mean, [C,2C) sigma, [2C,3C) dgamma, [3C,4C) dbeta

template <int kSums>
__device__ __forceinline__ void accumulate(float (&acc)[4], float x, float dy)
{
  acc[0] += x;
  acc[1] = fmaf(x, x, acc[1]);
  if (kSums == 4) { acc[2] = fmaf(dy, x, acc[2]); acc[3] += dy; }
}

// kMode 0: moments only (forward).  1: moments + ders (backward).  2: ders only, moments given.
template <int kMode, bool kVec>
__global__ void __cluster_dims__(1, kCluster, 1) __launch_bounds__(kThreads)
bnorm_reduce_kernel(float* __restrict__ momentsOut,   // 2*C or nullptr
                    float* __restrict__ dgOut, float* __restrict__ dbOut,
                    float const* __restrict__ momentsIn,  // mode 2
                    float const* __restrict__ x, float const* __restrict__ dy,
                    int WH, int C, int N, float eps)
{
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float part[4];
  __shared__ float warpRed[kThreads / 32][4];
  int c = blockIdx.x;
  int rank = (int)cluster.block_rank();   // the cluster spans grid y
  float acc[4] = {0.f, 0.f, 0.f, 0.f};

  // Work items: (image n, chunk of the plane).  Item i of this channel goes to CTA i % kCluster.
  if (kVec) {
    int WH4 = WH >> 2;
    long long items = (long long)N * WH4;
    for (long long i = (long long)rank * kThreads + threadIdx.x; i < items; i += (long long)kCluster * kThreads) {
      int n = (int)(i / WH4);
      int q = (int)(i - (long long)n * WH4);
      size_t off = ((size_t)n * C + c) * (size_t)WH + 4 * (size_t)q;
      float4 xv = *reinterpret_cast<float4 const*>(x + off);
      float4 dv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kMode != 0) dv = *reinterpret_cast<float4 const*>(dy + off);
      if (kMode == 2) {
        acc[2] = fmaf(dv.x, xv.x, acc[2]); acc[2] = fmaf(dv.y, xv.y, acc[2]);
        acc[2] = fmaf(dv.z, xv.z, acc[2]); acc[2] = fmaf(dv.w, xv.w, acc[2]);
        acc[3] += (dv.x + dv.y) + (dv.z + dv.w);
      } else {
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.x, dv.x);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.y, dv.y);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.z, dv.z);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.w, dv.w);
      }
    }
  } else {
    long long items = (long long)N * WH;
    for (long long i = (long long)rank * kThreads + threadIdx.x; i < items; i += (long long)kCluster * kThreads) {
      int n = (int)(i / WH);
      int q = (int)(i - (long long)n * WH);
      size_t off = ((size_t)n * C + c) * (size_t)WH + q;
      float xv = x[off];
      float dv = (kMode != 0) ? dy[off] : 0.f;
      if (kMode == 2) { acc[2] = fmaf(dv, xv, acc[2]); acc[3] += dv; }
      else accumulate<kMode == 0 ? 2 : 4>(acc, xv, dv);
    }
  }

#pragma unroll
  for (int j = 0; j < 4; ++j)
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { for (int j = 0; j < 4; ++j) warpRed[warp][j] = acc[j]; }
  __syncthreads();
  if (threadIdx.x < 4) {
    float s = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) s += warpRed[w][threadIdx.x];
    part[threadIdx.x] = s;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < kCluster; ++r) {
      float const* remote = cluster.map_shared_rank(part, r);
      for (int j = 0; j < 4; ++j) tot[j] += remote[j];
    }
    float mass = (float)((long long)WH * N);
    float mean, sigma;
    if (kMode == 2) { mean = momentsIn[c]; sigma = momentsIn[c + C]; }
    else {
      // reference bits/nnbnorm.cu:65-70
      mean = __fdiv_rn(tot[0], mass);
      float s2 = __fadd_rn(__fdiv_rn(tot[1], mass), -__fmul_rn(mean, mean));
      s2 = fmaxf(s2, 0.f);
      sigma = __fsqrt_rn(__fadd_rn(s2, eps));
      if (momentsOut) { momentsOut[c] = mean; momentsOut[c + C] = sigma; }
    }
    if (kMode != 0) {
      // reference bits/nnbnorm.cu:94-98
      dbOut[c] = tot[3];
      dgOut[c] = __fdiv_rn(__fadd_rn(tot[2], -__fmul_rn(mean, tot[3])), sigma);
    }
  }
  cluster.sync();   // keep every CTA's shared memory alive until rank 0 has read it
}

// One launch for the whole operator: the cluster that reduced a channel also applies it.
// After the reduction rank 0 derives the channel's coefficients into its shared memory, the other
// CTAs read them through distributed shared memory, and every CTA sweeps the same items again --
// they are still in L2 (a channel's x and dy, 8*m bytes, times the clusters in flight), so DRAM sees
// x and dy once and the result once: 12*m*C bytes backward, 8*m*C forward.
// kMode 0: forward, moments computed.  1: backward, moments computed.  2: backward, moments given.
template <int kMode, bool kVec>
__global__ void __cluster_dims__(1, kCluster, 1) __launch_bounds__(kThreads)
bnorm_fused_kernel(float* __restrict__ out,            // y or dx
                   float* __restrict__ momentsOut,     // 2*C or nullptr
                   float* __restrict__ dgOut, float* __restrict__ dbOut,
                   float const* __restrict__ momentsIn,  // mode 2
                   float const* __restrict__ x, float const* __restrict__ dy,
                   float const* __restrict__ g, float const* __restrict__ b,
                   int WH, int C, int N, float eps, int relu)      // relu (forward): the stored value is max(y, 0)
{
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float part[4];
  __shared__ float coef[4];
  __shared__ float warpRed[kThreads / 32][4];
  int const c = blockIdx.x;
  int const rank = (int)cluster.block_rank();   // the cluster spans grid y
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int const WH4 = WH >> 2;
  long long const items = kVec ? (long long)N * WH4 : (long long)N * WH;
  long long const first = (long long)rank * kThreads + threadIdx.x, step = (long long)kCluster * kThreads;

#pragma unroll 8
  for (long long i = first; i < items; i += step) {
    if (kVec) {
      int n = (int)(i / WH4);
      int q = (int)(i - (long long)n * WH4);
      size_t off = ((size_t)n * C + c) * (size_t)WH + 4 * (size_t)q;
      float4 xv = *reinterpret_cast<float4 const*>(x + off);
      float4 dv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kMode != 0) dv = *reinterpret_cast<float4 const*>(dy + off);
      if (kMode == 2) {
        acc[2] = fmaf(dv.x, xv.x, acc[2]); acc[2] = fmaf(dv.y, xv.y, acc[2]);
        acc[2] = fmaf(dv.z, xv.z, acc[2]); acc[2] = fmaf(dv.w, xv.w, acc[2]);
        acc[3] += (dv.x + dv.y) + (dv.z + dv.w);
      } else {
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.x, dv.x);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.y, dv.y);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.z, dv.z);
        accumulate<kMode == 0 ? 2 : 4>(acc, xv.w, dv.w);
      }
    } else {
      int n = (int)(i / WH);
      int q = (int)(i - (long long)n * WH);
      size_t off = ((size_t)n * C + c) * (size_t)WH + q;
      float xv = x[off];
      float dv = (kMode != 0) ? dy[off] : 0.f;
      if (kMode == 2) { acc[2] = fmaf(dv, xv, acc[2]); acc[3] += dv; }
      else accumulate<kMode == 0 ? 2 : 4>(acc, xv, dv);
    }
  }

#pragma unroll
  for (int j = 0; j < 4; ++j)
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
  int const warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { for (int j = 0; j < 4; ++j) warpRed[warp][j] = acc[j]; }
  __syncthreads();
  if (threadIdx.x < 4) {
    float s = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) s += warpRed[w][threadIdx.x];
    part[threadIdx.x] = s;
  }
  cluster.sync();
  // rank 0 gathers the partial sums of all ranks through distributed shared memory -- 32 threads fetch one value each, so that
  // the remote reads are one round trip instead of 32 -- and thread 0 adds them in rank order
  __shared__ float gath[kCluster][4];
  if (rank == 0 && threadIdx.x < kCluster * 4) {
    int const r = threadIdx.x >> 2, j = threadIdx.x & 3;
    gath[r][j] = cluster.map_shared_rank(part, r)[j];
  }
  if (rank == 0) __syncwarp();
  if (rank == 0 && threadIdx.x == 0) {
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < kCluster; ++r)
      for (int j = 0; j < 4; ++j) tot[j] += gath[r][j];
    float const mass = (float)((long long)WH * N);
    float mean, sigma;
    if (kMode == 2) { mean = momentsIn[c]; sigma = momentsIn[c + C]; }
    else {
      // reference bits/nnbnorm.cu:65-70
      mean = __fdiv_rn(tot[0], mass);
      float s2 = __fadd_rn(__fdiv_rn(tot[1], mass), -__fmul_rn(mean, mean));
      s2 = fmaxf(s2, 0.f);
      sigma = __fsqrt_rn(__fadd_rn(s2, eps));
      if (momentsOut) { momentsOut[c] = mean; momentsOut[c + C] = sigma; }
    }
    float const G1 = __fdiv_rn(g[c], sigma);
    if (kMode != 0) {
      // reference bits/nnbnorm.cu:94-98, 148-153
      float const dbv = tot[3];
      float const dgv = __fdiv_rn(__fadd_rn(tot[2], -__fmul_rn(mean, tot[3])), sigma);
      dbOut[c] = dbv;
      dgOut[c] = dgv;
      coef[0] = mean; coef[1] = __fdiv_rn(dbv, mass); coef[2] = G1;
      coef[3] = __fdiv_rn(__fmul_rn(G1, dgv), __fmul_rn(mass, sigma));
    } else {
      // reference bits/nnbnorm.cu:192-196
      coef[0] = mean; coef[1] = G1; coef[2] = b[c]; coef[3] = 0.f;
    }
  }
  cluster.sync();
  float k0, k1, k2, k3;
  {
    float const* rc = cluster.map_shared_rank(coef, 0);
    k0 = rc[0]; k1 = rc[1]; k2 = rc[2]; k3 = rc[3];
  }
  // (rank 0's shared memory has to outlive these reads: the cluster meets once more at the very end, where nobody waits long)

#pragma unroll 8
  for (long long i = first; i < items; i += step) {
    if (kVec) {
      int n = (int)(i / WH4);
      int q = (int)(i - (long long)n * WH4);
      size_t off = ((size_t)n * C + c) * (size_t)WH + 4 * (size_t)q;
      float4 xv = *reinterpret_cast<float4 const*>(x + off);
      float4 o;
      if (kMode == 0) {
        o.x = __fadd_rn(__fmul_rn(k1, __fadd_rn(xv.x, -k0)), k2);
        o.y = __fadd_rn(__fmul_rn(k1, __fadd_rn(xv.y, -k0)), k2);
        o.z = __fadd_rn(__fmul_rn(k1, __fadd_rn(xv.z, -k0)), k2);
        o.w = __fadd_rn(__fmul_rn(k1, __fadd_rn(xv.w, -k0)), k2);
        if (relu) { o.x = o.x > 0.f ? o.x : 0.f; o.y = o.y > 0.f ? o.y : 0.f; o.z = o.z > 0.f ? o.z : 0.f; o.w = o.w > 0.f ? o.w : 0.f; }
      } else {
        float4 dv = *reinterpret_cast<float4 const*>(dy + off);
        o.x = __fadd_rn(__fmul_rn(k2, __fadd_rn(dv.x, -k1)), -__fmul_rn(k3, __fadd_rn(xv.x, -k0)));
        o.y = __fadd_rn(__fmul_rn(k2, __fadd_rn(dv.y, -k1)), -__fmul_rn(k3, __fadd_rn(xv.y, -k0)));
        o.z = __fadd_rn(__fmul_rn(k2, __fadd_rn(dv.z, -k1)), -__fmul_rn(k3, __fadd_rn(xv.z, -k0)));
        o.w = __fadd_rn(__fmul_rn(k2, __fadd_rn(dv.w, -k1)), -__fmul_rn(k3, __fadd_rn(xv.w, -k0)));
      }
      *reinterpret_cast<float4*>(out + off) = o;
    } else {
      int n = (int)(i / WH);
      int q = (int)(i - (long long)n * WH);
      size_t off = ((size_t)n * C + c) * (size_t)WH + q;
      if (kMode == 0) { float o = __fadd_rn(__fmul_rn(k1, __fadd_rn(x[off], -k0)), k2); out[off] = (relu && !(o > 0.f)) ? 0.f : o; }
      else out[off] = __fadd_rn(__fmul_rn(k2, __fadd_rn(dy[off], -k1)), -__fmul_rn(k3, __fadd_rn(x[off], -k0)));
    }
  }
  cluster.sync();   // every CTA has read rank 0's coefficients long ago; rank 0 may exit
}

template <int kMode>
void launch_fused(vlb_ctx* ctx, bool vec, float* out, float* momOut, float* dg, float* db, float const* momIn,
                  float const* x, float const* dy, float const* g, float const* b, int WH, int C, int N, float eps, int relu = 0)
{
  dim3 grid(C, kCluster);
  if (vec) bnorm_fused_kernel<kMode, true><<<grid, kThreads, 0, ctx->stream>>>(out, momOut, dg, db, momIn, x, dy, g, b, WH, C, N, eps, relu);
  else     bnorm_fused_kernel<kMode, false><<<grid, kThreads, 0, ctx->stream>>>(out, momOut, dg, db, momIn, x, dy, g, b, WH, C, N, eps, relu);
  VLB_LAUNCHED(ctx, 1);
}

// Per-channel coefficients, computed once so that pass 2 is pure multiply/add.
// forward: cf = {mean, g/sigma, b, -}   (reference bits/nnbnorm.cu:192-196)
// backward: cf = {mean, db/m, G1 = g/sigma, G2 = G1*dg/(m*sigma)}   (bits/nnbnorm.cu:148-153)
__global__ void bnorm_coef_kernel(float4* __restrict__ cf, float const* __restrict__ moments,
                                  float const* __restrict__ g, float const* __restrict__ b,
                                  float const* __restrict__ dg, float const* __restrict__ db, int C, float mass)
{
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float mean = moments[c], sigma = moments[c + C];
  float G1 = __fdiv_rn(g[c], sigma);
  if (dg) {
    float muz = __fdiv_rn(db[c], mass);
    float G2 = __fdiv_rn(__fmul_rn(G1, dg[c]), __fmul_rn(mass, sigma));
    cf[c] = make_float4(mean, muz, G1, G2);
  } else {
    cf[c] = make_float4(mean, G1, b[c], 0.f);
  }
}

// y = g/sigma * (x - mean) + b (reference bits/nnbnorm.cu:192-203)
template <bool kVec>
__global__ void bnorm_fwd_apply_kernel(float* __restrict__ y, float const* __restrict__ x,
                                       float4 const* __restrict__ cf, int WH, int C, size_t total)
{
  size_t stride = (size_t)gridDim.x * blockDim.x;
  if (kVec) {
    size_t total4 = total >> 2;
    int WH4 = WH >> 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
      int c = (int)((i / WH4) % C);
      float4 k = __ldg(cf + c);
      float4 v = reinterpret_cast<float4 const*>(x)[i];
      v.x = __fadd_rn(__fmul_rn(k.y, __fadd_rn(v.x, -k.x)), k.z);
      v.y = __fadd_rn(__fmul_rn(k.y, __fadd_rn(v.y, -k.x)), k.z);
      v.z = __fadd_rn(__fmul_rn(k.y, __fadd_rn(v.z, -k.x)), k.z);
      v.w = __fadd_rn(__fmul_rn(k.y, __fadd_rn(v.w, -k.x)), k.z);
      reinterpret_cast<float4*>(y)[i] = v;
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      int c = (int)((i / WH) % C);
      float4 k = __ldg(cf + c);
      y[i] = __fadd_rn(__fmul_rn(k.y, __fadd_rn(x[i], -k.x)), k.z);
    }
  }
}

// dx = G1*(dy - db/m) - G2*(x - mean) (reference bits/nnbnorm.cu:136-164)
template <bool kVec>
__global__ void bnorm_bwd_apply_kernel(float* __restrict__ dx, float const* __restrict__ x,
                                       float const* __restrict__ dy, float4 const* __restrict__ cf,
                                       int WH, int C, size_t total)
{
  size_t stride = (size_t)gridDim.x * blockDim.x;
  if (kVec) {
    size_t total4 = total >> 2;
    int WH4 = WH >> 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
      int c = (int)((i / WH4) % C);
      float4 k = __ldg(cf + c);
      float4 xv = reinterpret_cast<float4 const*>(x)[i];
      float4 dv = reinterpret_cast<float4 const*>(dy)[i];
      float4 o;
      o.x = __fadd_rn(__fmul_rn(k.z, __fadd_rn(dv.x, -k.y)), -__fmul_rn(k.w, __fadd_rn(xv.x, -k.x)));
      o.y = __fadd_rn(__fmul_rn(k.z, __fadd_rn(dv.y, -k.y)), -__fmul_rn(k.w, __fadd_rn(xv.y, -k.x)));
      o.z = __fadd_rn(__fmul_rn(k.z, __fadd_rn(dv.z, -k.y)), -__fmul_rn(k.w, __fadd_rn(xv.z, -k.x)));
      o.w = __fadd_rn(__fmul_rn(k.z, __fadd_rn(dv.w, -k.y)), -__fmul_rn(k.w, __fadd_rn(xv.w, -k.x)));
      reinterpret_cast<float4*>(dx)[i] = o;
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      int c = (int)((i / WH) % C);
      float4 k = __ldg(cf + c);
      dx[i] = __fadd_rn(__fmul_rn(k.z, __fadd_rn(dy[i], -k.y)), -__fmul_rn(k.w, __fadd_rn(x[i], -k.x)));
    }
  }
}

bool vec_ok(int WH, void const* a, void const* b, void const* c)
{
  uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c;
  return (WH % 4 == 0) && (bits & 15) == 0;
}

int validate(vlb_ctx* ctx, int H, int W, int C, int N)
{
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0, "bnorm: empty input");
  VLB_REQUIRE(ctx, (long long)H * W * N < (1LL << 31), "bnorm: H*W*N too large");
  return VLB_Success;
}

template <int kMode>
void launch_reduce(vlb_ctx* ctx, bool vec, float* momOut, float* dg, float* db, float const* momIn,
                   float const* x, float const* dy, int WH, int C, int N, float eps)
{
  dim3 grid(C, kCluster);
  if (vec) bnorm_reduce_kernel<kMode, true><<<grid, kThreads, 0, ctx->stream>>>(momOut, dg, db, momIn, x, dy, WH, C, N, eps);
  else     bnorm_reduce_kernel<kMode, false><<<grid, kThreads, 0, ctx->stream>>>(momOut, dg, db, momIn, x, dy, WH, C, N, eps);
  VLB_LAUNCHED(ctx, 1);
}

// Scratch layout (context workspace): [0, 2C) moments when the caller passes none,
// then 4C floats of per-channel coefficients (16-byte aligned).
static float* scratch(vlb_ctx* ctx, int C, float4** cf)
{
  size_t momBytes = ((sizeof(float) * 2 * (size_t)C + 255) / 256) * 256;
  char* ws = (char*)vlb::workspace(ctx, momBytes + sizeof(float4) * (size_t)C);
  if (!ws) return nullptr;
  *cf = (float4*)(ws + momBytes);
  return (float*)ws;
}

static int forward_common(vlb_ctx* ctx, float* Y, float* momOut, float const* momIn, float const* X, float const* g,
                          float const* b, int H, int W, int C, int N, double eps, char const* where, int relu = 0)
{
  int rc = validate(ctx, H, W, C, N);
  if (rc) return rc;
  VLB_REQUIRE(ctx, Y && X && g && b, "bnorm_forward: null tensor");
  float4* cf = nullptr;
  float* ownMom = scratch(ctx, C, &cf);
  if (!ownMom) return vlb::pass_error(ctx, ctx->lastError, where);
  int WH = H * W;
  float const* mom = momIn;
  if (!momIn) {
    // moments computed and applied by the same clusters (the reference computes them into the context
    // workspace when the caller does not ask for them, bits/nnbnorm.cu:233-240)
    launch_fused<0>(ctx, vec_ok(WH, Y, X, X), Y, momOut, nullptr, nullptr, nullptr, X, nullptr, g, b, WH, C, N, (float)eps, relu);
    return vlb::check_launch(ctx, where);
  }
  bnorm_coef_kernel<<<vlb::ceil_div(C, 256), 256, 0, ctx->stream>>>(cf, mom, g, b, nullptr, nullptr, C, 0.f);
  size_t total = (size_t)WH * C * N;
  bool vec = vec_ok(WH, Y, X, X);
  unsigned grid = vlb::grid_for(vec ? total / 4 : total, kThreads, ctx->smCount * 16);
  if (vec) bnorm_fwd_apply_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(Y, X, cf, WH, C, total);
  else     bnorm_fwd_apply_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(Y, X, cf, WH, C, total);
  VLB_LAUNCHED(ctx, 2);
  return vlb::check_launch(ctx, where);
}

static int backward_common(vlb_ctx* ctx, float* dX, float* dG, float* dB, float* momOut, float const* momIn,
                           float const* X, float const* g, float const* dY, int H, int W, int C, int N,
                           double eps, char const* where)
{
  int rc = validate(ctx, H, W, C, N);
  if (rc) return rc;
  VLB_REQUIRE(ctx, dX && dG && dB && X && g && dY, "bnorm_backward: null tensor");
  int WH = H * W;
  bool vec = vec_ok(WH, X, dY, dX);
  if (!momIn) launch_fused<1>(ctx, vec, dX, momOut, dG, dB, nullptr, X, dY, g, nullptr, WH, C, N, (float)eps);
  else        launch_fused<2>(ctx, vec, dX, nullptr, dG, dB, momIn, X, dY, g, nullptr, WH, C, N, (float)eps);
  return vlb::check_launch(ctx, where);
}

}  // namespace

extern "C" {

int vlb_bnorm_forward_moment(vlb_ctx* ctx, float* Y, float const* moments, float const* X, float const* g,
                             float const* b, int H, int W, int C, int N, double eps)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, moments, "bnorm_forward_moment: null moments");
  return forward_common(ctx, Y, nullptr, moments, X, g, b, H, W, C, N, eps, "vlb_bnorm_forward_moment");
}

int vlb_bnorm_forward(vlb_ctx* ctx, float* Y, float* moments, float const* X, float const* g, float const* b,
                      int H, int W, int C, int N, double eps)
{
  if (!ctx) return VLB_IllegalArgument;
  return forward_common(ctx, Y, moments, nullptr, X, g, b, H, W, C, N, eps, "vlb_bnorm_forward");
}

int vlb_bnorm_relu_forward(vlb_ctx* ctx, float* Y, float* moments, float const* X, float const* g, float const* b,
                           int H, int W, int C, int N, double eps)
{
  if (!ctx) return VLB_IllegalArgument;
  return forward_common(ctx, Y, moments, nullptr, X, g, b, H, W, C, N, eps, "vlb_bnorm_relu_forward", 1);
}

int vlb_bnorm_backward(vlb_ctx* ctx, float* dX, float* dG, float* dB, float* moments, float const* X,
                       float const* g, float const* b, float const* dY, int H, int W, int C, int N, double eps)
{
  if (!ctx) return VLB_IllegalArgument;
  (void)b;
  return backward_common(ctx, dX, dG, dB, moments, nullptr, X, g, dY, H, W, C, N, eps, "vlb_bnorm_backward");
}

int vlb_bnorm_backward_moment(vlb_ctx* ctx, float* dX, float* dG, float* dB, float const* moments, float const* X,
                              float const* g, float const* b, float const* dY, int H, int W, int C, int N, double eps)
{
  if (!ctx) return VLB_IllegalArgument;
  (void)b;
  VLB_REQUIRE(ctx, moments, "bnorm_backward_moment: null moments");
  return backward_common(ctx, dX, dG, dB, nullptr, moments, X, g, dY, H, W, C, N, eps, "vlb_bnorm_backward_moment");
}

}  // extern "C"

// ====================================================================================
// Batch-norm backward for callers that must not allocate
// ====================================================================================
// Some hosts hand the whole device to an allocator of their own (MATLAB's gpuArray pool, a
// serving process with a fixed arena) or run inside a latency budget that a cudaMalloc --
// which synchronises the whole device -- would break.  Such callers cannot create a vlb_ctx
// (it allocates) nor let the scratch buffer grow.  For them the two per-channel scratch arrays
// of the backward pass live in a fixed array inside the library image: moments (2*C floats,
// used when the caller passes none) and the coefficients {mean, db/m, G1, G2} (4*C floats).
constexpr int kNoAllocMaxChannels = 4096;
static __device__ __align__(256) float g_bnormNoAllocScratch[6 * kNoAllocMaxChannels];   // 96 KB per GPU that loads the library

namespace {

// Device address of the array above, one per device.  The array's name is only a stand-in in
// host code; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device with that device current.
constexpr int kMaxDevices = 64;
float* g_noAllocPtr[kMaxDevices] = {};

void report(char* errbuf, size_t errlen, char const* msg)
{
  if (errbuf && errlen) snprintf(errbuf, errlen, "%s", msg);
}

}  // namespace

extern "C" int vlb_bnorm_backward_noalloc(void* cudaStream, float* dX, float* dG, float* dB, float* moments,
                                          float const* X, float const* g, float const* dY, int H, int W, int C,
                                          int N, double eps, char* errbuf, size_t errlen)
{
  if (!dX || !dG || !dB || !X || !g || !dY) { report(errbuf, errlen, "bnorm_backward_noalloc: null tensor"); return VLB_IllegalArgument; }
  if (H <= 0 || W <= 0 || C <= 0 || N <= 0 || (long long)H * W * N >= (1LL << 31)) {
    report(errbuf, errlen, "bnorm_backward_noalloc: empty or oversized input");
    return VLB_IllegalArgument;
  }
  if (C > kNoAllocMaxChannels) {
    report(errbuf, errlen, "bnorm_backward_noalloc: more than 4096 channels do not fit the built-in scratch array; "
                           "use vlb_bnorm_backward with a context");
    return VLB_IllegalArgument;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { report(errbuf, errlen, "bnorm_backward_noalloc: no usable current device"); return VLB_Cuda; }
  if (!g_noAllocPtr[dev]) {
    // first call on this device: the kernels are built for sm_100a only, so refuse anything else before a launch
    // could fail and leave its error pending for the host process; then resolve the array's device address (no
    // allocation takes place).  Two host threads making their first call on one device at the same time would both
    // do this and store the same address: harmless, but the entry point is meant for one calling thread per device.
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) { cudaGetLastError(); report(errbuf, errlen, cudaGetErrorString(e)); return VLB_Cuda; }
    if (major != 10) { report(errbuf, errlen, "bnorm_backward_noalloc: the kernels are built for sm_100a only"); return VLB_Unsupported; }
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_bnormNoAllocScratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      report(errbuf, errlen, cudaGetErrorString(e));
      return VLB_Cuda;
    }
    g_noAllocPtr[dev] = p;
  }
  cudaStream_t stream = (cudaStream_t)cudaStream;
  float* ownMom = g_noAllocPtr[dev];
  float4* cf = reinterpret_cast<float4*>(g_noAllocPtr[dev] + 2 * kNoAllocMaxChannels);
  float* mom = moments ? moments : ownMom;
  // Nothing in the scratch has to start from zero: pass 1 writes every moment and pass 1b every
  // coefficient of channels [0, C) before pass 2 reads them; entries beyond C keep an earlier call's
  // values and are never read.
  int WH = H * W;
  bool vec = vec_ok(WH, X, dY, dX);
  dim3 grid(C, kCluster);
  if (vec) bnorm_reduce_kernel<1, true><<<grid, kThreads, 0, stream>>>(mom, dG, dB, nullptr, X, dY, WH, C, N, (float)eps);
  else     bnorm_reduce_kernel<1, false><<<grid, kThreads, 0, stream>>>(mom, dG, dB, nullptr, X, dY, WH, C, N, (float)eps);
  float mass = (float)((long long)WH * N);
  bnorm_coef_kernel<<<vlb::ceil_div(C, 256), 256, 0, stream>>>(cf, mom, g, nullptr, dG, dB, C, mass);
  size_t total = (size_t)WH * C * N;
  unsigned blocks = vlb::grid_for(vec ? total / 4 : total, kThreads, 148 * 16);
  if (vec) bnorm_bwd_apply_kernel<true><<<blocks, kThreads, 0, stream>>>(dX, X, dY, cf, WH, C, total);
  else     bnorm_bwd_apply_kernel<false><<<blocks, kThreads, 0, stream>>>(dX, X, dY, cf, WH, C, total);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    report(errbuf, errlen, cudaGetErrorString(e));
    cudaGetLastError();      // reported once: cleared so that later calls are not blamed for it
    return VLB_Cuda;
  }
  return VLB_Success;
}
