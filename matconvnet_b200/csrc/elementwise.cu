// Element-wise and small reduction kernels: ReLU, Sum, scale, Bias, softmax-loss.
// All are HBM-bound: 128-bit accesses where alignment allows, grid-stride loops
// sized from the SM count.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int kThreads = 256;

inline bool aligned16(void const* p) { return (((uintptr_t)p) & 15) == 0; }

// ---------------------------------------------------------------- ReLU / sum / scale
// y = max(x, 0) (reference matlab/vl_nnrelu.m:45)
// y and x may be the same array (element i is read before it is written)
__global__ void relu_fwd_kernel(float* y, float const* x, size_t n, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 v = reinterpret_cast<float4 const*>(x)[i];
      v.x = v.x > 0.f ? v.x : 0.f; v.y = v.y > 0.f ? v.y : 0.f;
      v.z = v.z > 0.f ? v.z : 0.f; v.w = v.w > 0.f ? v.w : 0.f;
      reinterpret_cast<float4*>(y)[i] = v;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) y[i] = x[i] > 0.f ? x[i] : 0.f;
  } else {
    for (size_t i = i0; i < n; i += stride) y[i] = x[i] > 0.f ? x[i] : 0.f;
  }
}

// dx = dy .* (x > 0) (reference matlab/vl_nnrelu.m:47)
// dx may be dy (every element is read before it is written, by the same thread)
__global__ void relu_bwd_kernel(float* dx, float const* __restrict__ x, float const* dy, size_t n, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 v = reinterpret_cast<float4 const*>(x)[i];
      float4 d = reinterpret_cast<float4 const*>(dy)[i];
      d.x = v.x > 0.f ? d.x : 0.f; d.y = v.y > 0.f ? d.y : 0.f;
      d.z = v.z > 0.f ? d.z : 0.f; d.w = v.w > 0.f ? d.w : 0.f;
      reinterpret_cast<float4*>(dx)[i] = d;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) dx[i] = x[i] > 0.f ? dy[i] : 0.f;
  } else {
    for (size_t i = i0; i < n; i += stride) dx[i] = x[i] > 0.f ? dy[i] : 0.f;
  }
}

// y = alpha*a + beta*b as the reference computes it: a scaled by alpha, then an axpy of b (matlab/src/vl_taccummex.cu:50-76);
// y may be a.
__device__ __forceinline__ float taccum1(float alpha, float a, float beta, float b) { return __fmaf_rn(beta, b, __fmul_rn(alpha, a)); }

__global__ void taccum_kernel(float* y, float alpha, float const* a, float beta, float const* b, size_t n, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 u = reinterpret_cast<float4 const*>(a)[i], v = reinterpret_cast<float4 const*>(b)[i];
      u.x = taccum1(alpha, u.x, beta, v.x); u.y = taccum1(alpha, u.y, beta, v.y);
      u.z = taccum1(alpha, u.z, beta, v.z); u.w = taccum1(alpha, u.w, beta, v.w);
      reinterpret_cast<float4*>(y)[i] = u;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) y[i] = taccum1(alpha, a[i], beta, b[i]);
  } else {
    for (size_t i = i0; i < n; i += stride) y[i] = taccum1(alpha, a[i], beta, b[i]);
  }
}

// The trainer's update of one parameter tensor (reference examples/cnn_train.m:478-499), its four vl_taccum passes in one:
//   g = gradMult*G + decay*W;  M = momentum*M - g;  delta = nesterov ? momentum*M - g : M;  W = W + lr*delta
// with every intermediate rounded as in the separate passes.
struct SgdParams { float gradMult, decay, momentum, lr; int nesterov; };

__device__ __forceinline__ void sgd1(float& w, float& m, float g0, SgdParams const& p)
{
  float const g = taccum1(p.gradMult, g0, p.decay, w);
  m = taccum1(p.momentum, m, -1.f, g);
  float const delta = p.nesterov ? __fsub_rn(__fmul_rn(p.momentum, m), g) : m;
  w = taccum1(1.f, w, p.lr, delta);
}

__global__ void sgd_update_kernel(float* w, float* m, float const* __restrict__ g, size_t n, SgdParams p, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 W = reinterpret_cast<float4*>(w)[i], M = reinterpret_cast<float4*>(m)[i];
      float4 const G = reinterpret_cast<float4 const*>(g)[i];
      sgd1(W.x, M.x, G.x, p); sgd1(W.y, M.y, G.y, p); sgd1(W.z, M.z, G.z, p); sgd1(W.w, M.w, G.w, p);
      reinterpret_cast<float4*>(w)[i] = W;
      reinterpret_cast<float4*>(m)[i] = M;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) sgd1(w[i], m[i], g[i], p);
  } else {
    for (size_t i = i0; i < n; i += stride) sgd1(w[i], m[i], g[i], p);
  }
}

// The trainer's other solvers (reference examples/+solver/adagrad.m, adadelta.m, adam.m, rmsprop.m; call site
// examples/cnn_train.m:478-507): the normalisation + weight decay pass (vl_taccum) and the solver's element-wise MATLAB
// expression in one kernel.  Every MATLAB operation on single arrays rounds to single, so each is one _rn operation here
// and nothing is contracted into a fused multiply-add.
struct SolverParams { int solver; float gradMult, decay, lr, rho, eps, beta1, beta2, omb2; };

__device__ __forceinline__ void solver1(float& w, float& s1, float& s2, float g0, SolverParams const& p)
{
  float const g = taccum1(p.gradMult, g0, p.decay, w);
  float const gg = __fmul_rn(g, g);
  if (p.solver == VLB_SOLVER_ADAGRAD) {
    // g_sqr = g_sqr * rho + grad.^2 ;  w = w - lr * grad ./ (sqrt(g_sqr) + epsilon)
    s1 = __fadd_rn(__fmul_rn(s1, p.rho), gg);
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(p.lr, g), __fadd_rn(__fsqrt_rn(s1), p.eps)));
  } else if (p.solver == VLB_SOLVER_RMSPROP) {
    // g_sqr = g_sqr * rho + grad.^2 * (1 - rho) ;  w = w - lr * grad ./ (sqrt(g_sqr) + epsilon)
    s1 = __fadd_rn(__fmul_rn(s1, p.rho), __fmul_rn(gg, p.beta1));          // beta1 carries single(1 - rho)
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(p.lr, g), __fadd_rn(__fsqrt_rn(s1), p.eps)));
  } else if (p.solver == VLB_SOLVER_ADADELTA) {
    // g_sqr = g_sqr * rho + grad.^2 * (1 - rho) ;  new_delta = -sqrt((delta_sqr + eps) ./ (g_sqr + eps)) .* grad ;
    // delta_sqr = delta_sqr * rho + new_delta.^2 * (1 - rho) ;  w = w + new_delta
    s1 = __fadd_rn(__fmul_rn(s1, p.rho), __fmul_rn(gg, p.beta1));
    float const nd = __fmul_rn(-__fsqrt_rn(__fdiv_rn(__fadd_rn(s2, p.eps), __fadd_rn(s1, p.eps))), g);
    s2 = __fadd_rn(__fmul_rn(s2, p.rho), __fmul_rn(__fmul_rn(nd, nd), p.beta1));
    w = __fadd_rn(w, nd);
  } else {
    // m = beta1 * m + (1 - beta1) * grad ;  v = beta2 * v + (1 - beta2) * grad.^2 ;  w = w - lr_t * m ./ (v.^0.5 + eps)
    // (lr carries lr_t, rho carries single(1 - beta1), omb2 single(1 - beta2): see vlb_solver_update)
    s1 = __fadd_rn(__fmul_rn(p.beta1, s1), __fmul_rn(p.rho, g));
    s2 = __fadd_rn(__fmul_rn(p.beta2, s2), __fmul_rn(p.omb2, gg));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(p.lr, s1), __fadd_rn(__fsqrt_rn(s2), p.eps)));
  }
}

__global__ void solver_update_kernel(float* w, float* s1, float* s2, float const* __restrict__ g, size_t n, SolverParams p, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool const two = s2 != nullptr;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 W = reinterpret_cast<float4*>(w)[i], A = reinterpret_cast<float4*>(s1)[i];
      float4 B = two ? reinterpret_cast<float4*>(s2)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 const G = reinterpret_cast<float4 const*>(g)[i];
      solver1(W.x, A.x, B.x, G.x, p); solver1(W.y, A.y, B.y, G.y, p); solver1(W.z, A.z, B.z, G.z, p); solver1(W.w, A.w, B.w, G.w, p);
      reinterpret_cast<float4*>(w)[i] = W;
      reinterpret_cast<float4*>(s1)[i] = A;
      if (two) reinterpret_cast<float4*>(s2)[i] = B;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) {
      float b = two ? s2[i] : 0.f;
      solver1(w[i], s1[i], b, g[i], p);
      if (two) s2[i] = b;
    }
  } else {
    for (size_t i = i0; i < n; i += stride) {
      float b = two ? s2[i] : 0.f;
      solver1(w[i], s1[i], b, g[i], p);
      if (two) s2[i] = b;
    }
  }
}

__global__ void sum_kernel(float* y, float const* a, float const* b, size_t n, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 u = reinterpret_cast<float4 const*>(a)[i], v = reinterpret_cast<float4 const*>(b)[i];
      u.x += v.x; u.y += v.y; u.z += v.z; u.w += v.w;
      reinterpret_cast<float4*>(y)[i] = u;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) y[i] = a[i] + b[i];
  } else {
    for (size_t i = i0; i < n; i += stride) y[i] = a[i] + b[i];
  }
}

__global__ void scale_kernel(float* x, float alpha, size_t n, bool vec)
{
  size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    size_t n4 = n >> 2;
    for (size_t i = i0; i < n4; i += stride) {
      float4 u = reinterpret_cast<float4*>(x)[i];
      u.x *= alpha; u.y *= alpha; u.z *= alpha; u.w *= alpha;
      reinterpret_cast<float4*>(x)[i] = u;
    }
    for (size_t i = (n4 << 2) + i0; i < n; i += stride) x[i] *= alpha;
  } else {
    for (size_t i = i0; i < n; i += stride) x[i] *= alpha;
  }
}

// ---------------------------------------------------------------- Bias
// One block row per (k, n) plane of P = H*W elements.
// mode 0: y = bv (+ xm*x); mode 1: y = bv + ym*y (+ xm*x); mode 2: y = 0 (+ xm*x)
__global__ void bias_fwd_kernel(float* __restrict__ y, float ym, float const* __restrict__ x, float xm,
                                float const* __restrict__ b, float bm, int P, int K, size_t planes, int mode)
{
  for (size_t plane = blockIdx.y; plane < planes; plane += gridDim.y) {
    int k = (int)(plane % K);
    float bv = (mode == 2) ? 0.f : __fmul_rn(bm, b[k]);
    float* yp = y + plane * (size_t)P;
    float const* xp = x ? x + plane * (size_t)P : nullptr;
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < P; p += gridDim.x * blockDim.x) {
      float v = bv;
      if (mode == 1) v = __fadd_rn(bv, __fmul_rn(ym, yp[p]));
      if (xp) v = __fadd_rn(v, __fmul_rn(xm, xp[p]));
      yp[p] = v;
    }
  }
}

// The same for small planes (P < 64, e.g. the 1x1 outputs of a fully connected layer): one thread per element.
__global__ void bias_fwd_flat_kernel(float* __restrict__ y, float ym, float const* __restrict__ x, float xm,
                                     float const* __restrict__ b, float bm, int P, int K, size_t total, int mode)
{
  size_t const step = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += step) {
    int const k = (int)((e / P) % K);
    float v = (mode == 2) ? 0.f : __fmul_rn(bm, b[k]);
    if (mode == 1) v = __fadd_rn(v, __fmul_rn(ym, y[e]));
    if (x) v = __fadd_rn(v, __fmul_rn(xm, x[e]));
    y[e] = v;
  }
}

// db[k] = beta*db[k] + bm * sum over (p, n) of dy; one block per k, fixed-order tree.
__global__ void bias_bwd_db_kernel(float* __restrict__ db, float beta, float bm, float const* __restrict__ dy,
                                   int P, int K, int N)
{
  __shared__ float red[32];
  int k = blockIdx.x;
  float s = 0.f;
  size_t total = (size_t)P * N;
  for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
    size_t n = i / P, p = i - n * P;
    s += dy[p + (size_t)P * (k + (size_t)K * n)];
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) db[k] = (beta == 0.f) ? bm * s : bm * s + beta * db[k];
  }
}

// dx = dxm*dx + xm*dy ; dxm == 0 means overwrite
__global__ void axpby_kernel(float* dx, float dxm, float xm, float const* dy, size_t n)
{
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = __fmul_rn(xm, dy[i]);
    if (dxm != 0.f) v = __fadd_rn(__fmul_rn(dxm, dx[i]), v);
    dx[i] = v;
  }
}

// ---------------------------------------------------------------- softmax loss
// One block per (pixel, image): max-shifted log-sum-exp over C channels
// (reference matlab/vl_nnsoftmaxloss.m:72-84).  `terms` gets one loss term per block
// (forward) or dx gets (softmax - onehot) * scale (backward).
__device__ float block_reduce(float v, bool isMax, float* red)
{
  for (int o = 16; o > 0; o >>= 1) {
    float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = isMax ? fmaxf(v, u) : v + u;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  int nw = blockDim.x >> 5;
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

__global__ void softmaxloss_kernel(float* __restrict__ terms, float* __restrict__ dx, float const* __restrict__ x,
                                   float const* __restrict__ labels, float scale, int P, int C, int* __restrict__ status)
{
  __shared__ float red[32];
  int p = blockIdx.x, n = blockIdx.y;
  float const* xp = x + p + (size_t)P * C * n;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, xp[(size_t)P * c]);
  m = block_reduce(m, true, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) s += expf(xp[(size_t)P * c] - m);
  s = block_reduce(s, false, red);
  // class 0 skips the location: mass = (c > 0), index max(c - 1, 0) (matlab/vl_nnsoftmaxloss.m:55-67).  A class above C
  // is an indexing error in the reference; here it is reported through the context's status word and skipped likewise.
  float const labf = labels[n];
  bool const tooBig = labf > (float)C;
  if (tooBig && threadIdx.x == 0) atomicExch(status, kStatusBadLabel);
  float const mass = (labf > 0.f && !tooBig) ? 1.f : 0.f;
  int const lab = min(max((int)labf - 1, 0), C - 1);
  if (dx) {
    float* dp = dx + p + (size_t)P * C * n;
    float const ms = mass * scale;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float v = expf(xp[(size_t)P * c] - m) / s;
      if (c == lab) v -= 1.f;
      dp[(size_t)P * c] = v * ms;
    }
  } else if (threadIdx.x == 0) {
    terms[p + (size_t)P * n] = mass * (m + logf(s) - xp[(size_t)P * lab]);
  }
}

// loss = (sum of terms) / N, one block, fixed order.
__global__ void loss_finish_kernel(float* loss, float const* terms, int count, float invN)
{
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) s += terms[i];
  s = block_reduce(s, false, red);
  if (threadIdx.x == 0) *loss = s * invN;
}

}  // namespace

extern "C" {

int vlb_relu_forward(vlb_ctx* ctx, float* Y, float const* X, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y && X, "relu_forward: null tensor");
  if (n == 0) return VLB_Success;
  bool vec = aligned16(Y) && aligned16(X);
  relu_fwd_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(Y, X, n, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_relu_forward");
}

int vlb_relu_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, dX && X && dY, "relu_backward: null tensor");
  if (n == 0) return VLB_Success;
  bool vec = aligned16(dX) && aligned16(X) && aligned16(dY);
  relu_bwd_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(dX, X, dY, n, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_relu_backward");
}

int vlb_sum(vlb_ctx* ctx, float* Y, float const* A, float const* B, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y && A && B, "sum: null tensor");
  if (n == 0) return VLB_Success;
  bool vec = aligned16(Y) && aligned16(A) && aligned16(B);
  sum_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(Y, A, B, n, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sum");
}

int vlb_scale(vlb_ctx* ctx, float* x, double alpha, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, x, "scale: null tensor");
  if (n == 0) return VLB_Success;
  bool vec = aligned16(x);
  scale_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(x, (float)alpha, n, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_scale");
}

int vlb_taccum(vlb_ctx* ctx, float* Y, double alpha, float const* A, double beta, float const* B, size_t n)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y && A && B, "taccum: null tensor");
  if (n == 0) return VLB_Success;
  bool vec = aligned16(Y) && aligned16(A) && aligned16(B);
  taccum_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(
      Y, (float)alpha, A, (float)beta, B, n, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_taccum");
}

int vlb_sgd_update(vlb_ctx* ctx, float* W, float* M, float const* G, size_t n, double gradMult, double decay,
                   double momentum, double lr, int nesterov)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, W && M && G, "sgd_update: null tensor");
  if (n == 0) return VLB_Success;
  SgdParams p = {(float)gradMult, (float)decay, (float)momentum, (float)lr, nesterov ? 1 : 0};
  bool vec = aligned16(W) && aligned16(M) && aligned16(G);
  sgd_update_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(W, M, G, n, p, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_sgd_update");
}

int vlb_solver_update(vlb_ctx* ctx, int solver, float* W, float* S1, float* S2, float const* G, size_t n, double gradMult,
                      double decay, double lr, vlb_solver_opts const* opts, long long t)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, solver >= VLB_SOLVER_ADAGRAD && solver <= VLB_SOLVER_RMSPROP, "solver_update: unknown solver");
  bool const two = solver == VLB_SOLVER_ADADELTA || solver == VLB_SOLVER_ADAM;
  VLB_REQUIRE(ctx, W && S1 && G && opts && (!two || S2), "solver_update: null tensor");
  VLB_REQUIRE(ctx, solver != VLB_SOLVER_ADAM || t >= 1, "solver_update: adam needs the step count t >= 1");
  if (n == 0) return VLB_Success;
  SolverParams p = {};
  p.solver = solver; p.gradMult = (float)gradMult; p.decay = (float)decay; p.lr = (float)lr;
  p.rho = (float)opts->rho; p.eps = (float)opts->epsilon;
  // MATLAB evaluates scalar expressions such as (1 - rho) in double and converts the result to single when it meets the array
  p.beta1 = (float)(1.0 - opts->rho);
  if (solver == VLB_SOLVER_ADAM) {
    p.beta1 = (float)opts->beta1; p.beta2 = (float)opts->beta2;
    p.rho = (float)(1.0 - opts->beta1); p.omb2 = (float)(1.0 - opts->beta2);
    // lr_t = lr * (((1 - beta2^t)^0.5) / (1 - beta1^t))   (examples/+solver/adam.m)
    p.lr = (float)(lr * (sqrt(1.0 - pow(opts->beta2, (double)t)) / (1.0 - pow(opts->beta1, (double)t))));
  }
  bool vec = aligned16(W) && aligned16(S1) && aligned16(G) && (!two || aligned16(S2));
  solver_update_kernel<<<vlb::grid_for(vec ? n / 4 + 1 : n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(
      W, S1, two ? S2 : nullptr, G, n, p, vec);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_solver_update");
}

int vlb_bias_forward(vlb_ctx* ctx, float* Y, double yMult, float const* X, double xMult, float const* b,
                     double bMult, int H, int W, int K, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, Y, "bias_forward: null output");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && K > 0 && N > 0, "bias_forward: empty tensor");
  int P = H * W;
  int mode = (b && bMult != 0) ? ((float)yMult == 0.f ? 0 : 1) : 2;
  float const* xin = (X && xMult != 0) ? X : nullptr;
  size_t planes = (size_t)K * N;
  if (P < 64) {
    size_t total = planes * (size_t)P;
    bias_fwd_flat_kernel<<<vlb::grid_for(total, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(
        Y, (float)yMult, xin, (float)xMult, b, (float)bMult, P, K, total, mode);
    VLB_LAUNCHED(ctx, 1);
    return vlb::check_launch(ctx, "vlb_bias_forward");
  }
  dim3 grid(vlb::ceil_div(P, kThreads) > 64 ? 64 : vlb::ceil_div(P, kThreads), (unsigned)(planes > 32768 ? 32768 : planes));
  bias_fwd_kernel<<<grid, kThreads, 0, ctx->stream>>>(Y, (float)yMult, xin, (float)xMult, b, (float)bMult, P, K, planes, mode);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_bias_forward");
}

int vlb_bias_backward(vlb_ctx* ctx, float* dX, double dXMult, float* db, double dbMult, double xMult,
                      double bMult, float const* dY, int H, int W, int K, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, dY, "bias_backward: null derOutput");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && K > 0 && N > 0, "bias_backward: empty tensor");
  int P = H * W;
  if (db) {
    bias_bwd_db_kernel<<<K, 256, 0, ctx->stream>>>(db, (float)dbMult, (float)bMult, dY, P, K, N);
    VLB_LAUNCHED(ctx, 1);
  }
  if (dX) {
    size_t n = (size_t)P * K * N;
    axpby_kernel<<<vlb::grid_for(n, kThreads, ctx->smCount * 8), kThreads, 0, ctx->stream>>>(dX, (float)dXMult, (float)xMult, dY, n);
    VLB_LAUNCHED(ctx, 1);
  }
  return vlb::check_launch(ctx, "vlb_bias_backward");
}

int vlb_softmaxloss_forward(vlb_ctx* ctx, float* loss, float const* X, float const* labels, int H, int W, int C, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, loss && X && labels, "softmaxloss_forward: null tensor");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && N <= 65535, "softmaxloss_forward: bad shape");
  int P = H * W;
  float* terms = (float*)vlb::workspace(ctx, sizeof(float) * (size_t)P * N);
  if (!terms) return vlb::pass_error(ctx, ctx->lastError, "vlb_softmaxloss_forward");
  int threads = C >= 256 ? 256 : (C >= 64 ? 64 : 32);
  softmaxloss_kernel<<<dim3(P, N), threads, 0, ctx->stream>>>(terms, nullptr, X, labels, 0.f, P, C, ctx->deviceStatus);
  loss_finish_kernel<<<1, 256, 0, ctx->stream>>>(loss, terms, P * N, 1.f / (float)N);
  VLB_LAUNCHED(ctx, 2);
  return vlb::check_launch(ctx, "vlb_softmaxloss_forward");
}

int vlb_softmaxloss_backward(vlb_ctx* ctx, float* dX, float const* X, float const* labels, double dzdy,
                             int H, int W, int C, int N)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, dX && X && labels, "softmaxloss_backward: null tensor");
  VLB_REQUIRE(ctx, H > 0 && W > 0 && C > 0 && N > 0 && N <= 65535, "softmaxloss_backward: bad shape");
  int P = H * W;
  int threads = C >= 256 ? 256 : (C >= 64 ? 64 : 32);
  softmaxloss_kernel<<<dim3(P, N), threads, 0, ctx->stream>>>(nullptr, dX, X, labels, (float)dzdy / (float)N, P, C, ctx->deviceStatus);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "vlb_softmaxloss_backward");
}

}  // extern "C"
