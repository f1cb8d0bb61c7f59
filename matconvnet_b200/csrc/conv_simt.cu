// CUDA-core implicit-GEMM convolution: the exact-fp32 path (VLB_PRECISION_FP32) and the path
// for every stride / dilation / padding / group configuration of vl::nn::Convolution
// (reference bits/nnconv.cu:71-317) that the tensor-core kernels do not cover.
//
// No patch matrix is ever written (the reference builds one per image, bits/nnconv.cu:
// 109-117,283-291): operands are gathered straight from the tensors with the index algebra
//   h = ho*strideY + fh*dilateY - padTop,  w = wo*strideX + fw*dilateX - padLeft
// (bits/impl/im2row_cpu.cpp:97-106), one kernel per direction for the whole batch.
// All three directions are instances of  D[i][j] = sum_r A(i,r) * B(j,r):
//   fprop  i = output pixel (ho,wo,n)   j = filter in group   r = (fh,fw,fc)
//   dgrad  i = input pixel (h,w,n)      j = channel in group  r = (fh,fw,filter in group)
//   wgrad  i = (fh,fw,fc)               j = filter in group   r = output pixel (ho,wo,n)
// Tile 64x64x16, 256 threads, 4x4 accumulators per thread.  wgrad splits r across CTAs and
// reduces the partial filters from scratch in a fixed order (deterministic, no atomics).
#include "common.cuh"
#include "conv_internal.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, kThreads = 256;

using vlb::ConvGeom;

// ---------------------------------------------------------------- operand accessors
struct FpropOp {
  static constexpr bool kIFast = true;
  ConvGeom g;
  float const* x; float const* f; float const* b; float* y;
  float outMult, inMult;
  int M, Nn, R, splits;
  struct ICtx { int h0, w0; long long base; bool valid; };
  struct RCtx { int dh, dw; long long off; int r; bool valid; };
  __device__ ICtx decodeI(int i, int grp) const {
    ICtx c; c.valid = i < M;
    int ho = i % g.Ho, t = i / g.Ho, wo = t % g.Wo, n = t / g.Wo;
    c.h0 = ho * g.sy - g.pt; c.w0 = wo * g.sx - g.pl;
    c.base = (long long)g.H * g.W * ((long long)grp * g.FC + (long long)g.C * n);
    return c;
  }
  __device__ RCtx decodeR(int r, int) const {
    RCtx c; c.valid = r < R; c.r = r;
    int fh = r % g.FH, t = r / g.FH, fw = t % g.FW, fc = t / g.FW;
    c.dh = fh * g.dy; c.dw = fw * g.dx; c.off = (long long)g.H * g.W * fc;
    return c;
  }
  __device__ float A(ICtx const& i, RCtx const& r) const {
    int h = i.h0 + r.dh, w = i.w0 + r.dw;
    if (!i.valid || !r.valid || h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[i.base + r.off + (long long)w * g.H + h];
  }
  __device__ float B(int j, RCtx const& r, int grp) const {
    if (j >= Nn || !r.valid) return 0.f;
    return f[(long long)R * ((long long)grp * g.Kg + j) + r.r];
  }
  __device__ void store(int i, int j, int grp, int, float v) const {
    if (i >= M || j >= Nn) return;
    int P = g.Ho * g.Wo, pix = i % P, n = i / P, k = grp * g.Kg + j;
    long long o = pix + (long long)P * (k + (long long)g.K * n);
    float r = inMult * v;
    if (b) r += b[k];
    if (outMult != 0.f) r += outMult * y[o];
    y[o] = r;
  }
};

struct DgradOp {
  static constexpr bool kIFast = true;
  ConvGeom g;
  float const* dy; float const* f; float* dx;
  int M, Nn, R, splits;
  struct ICtx { int hp, wp; long long base; bool valid; };
  struct RCtx { int dh, dw, fh, fw, kk; bool valid; };
  __device__ ICtx decodeI(int i, int grp) const {
    ICtx c; c.valid = i < M;
    int h = i % g.H, t = i / g.H, w = t % g.W, n = t / g.W;
    c.hp = h + g.pt; c.wp = w + g.pl;
    c.base = (long long)g.Ho * g.Wo * ((long long)grp * g.Kg + (long long)g.K * n);
    return c;
  }
  __device__ RCtx decodeR(int r, int) const {
    RCtx c; c.valid = r < R;
    c.fh = r % g.FH; int t = r / g.FH; c.fw = t % g.FW; c.kk = t / g.FW;
    c.dh = c.fh * g.dy; c.dw = c.fw * g.dx;
    return c;
  }
  __device__ float A(ICtx const& i, RCtx const& r) const {
    if (!i.valid || !r.valid) return 0.f;
    int hn = i.hp - r.dh, wn = i.wp - r.dw;
    if (hn < 0 || wn < 0) return 0.f;
    int ho = hn / g.sy, wo = wn / g.sx;
    if (ho * g.sy != hn || wo * g.sx != wn || ho >= g.Ho || wo >= g.Wo) return 0.f;
    return dy[i.base + (long long)g.Ho * g.Wo * r.kk + (long long)wo * g.Ho + ho];
  }
  __device__ float B(int j, RCtx const& r, int grp) const {
    if (j >= Nn || !r.valid) return 0.f;
    return f[r.fh + (long long)g.FH * (r.fw + (long long)g.FW * (j + (long long)g.FC * ((long long)grp * g.Kg + r.kk)))];
  }
  __device__ void store(int i, int j, int grp, int, float v) const {
    if (i >= M || j >= Nn) return;
    int P = g.H * g.W, pix = i % P, n = i / P;
    dx[pix + (long long)P * ((long long)grp * g.FC + j + (long long)g.C * n)] = v;
  }
};

struct WgradOp {
  static constexpr bool kIFast = false;
  ConvGeom g;
  float const* x; float const* dy; float* out;   // out: dF, or split partials [split][K*V]
  int M, Nn, R, splits;
  struct ICtx { int dh, dw; long long off; bool valid; };
  struct RCtx { int h0, w0; long long xbase, ybase; bool valid; };
  __device__ ICtx decodeI(int i, int grp) const {
    ICtx c; c.valid = i < M;
    int fh = i % g.FH, t = i / g.FH, fw = t % g.FW, fc = t / g.FW;
    c.dh = fh * g.dy; c.dw = fw * g.dx;
    c.off = (long long)g.H * g.W * ((long long)grp * g.FC + fc);
    return c;
  }
  __device__ RCtx decodeR(int r, int grp) const {
    RCtx c; c.valid = r < R;
    int ho = r % g.Ho, t = r / g.Ho, wo = t % g.Wo, n = t / g.Wo;
    c.h0 = ho * g.sy - g.pt; c.w0 = wo * g.sx - g.pl;
    c.xbase = (long long)g.H * g.W * g.C * n;
    c.ybase = (long long)wo * g.Ho + ho + (long long)g.Ho * g.Wo * ((long long)grp * g.Kg + (long long)g.K * n);
    return c;
  }
  __device__ float A(ICtx const& i, RCtx const& r) const {
    int h = r.h0 + i.dh, w = r.w0 + i.dw;
    if (!i.valid || !r.valid || h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[r.xbase + i.off + (long long)w * g.H + h];
  }
  __device__ float B(int j, RCtx const& r, int) const {
    if (j >= Nn || !r.valid) return 0.f;
    return dy[r.ybase + (long long)g.Ho * g.Wo * j];
  }
  __device__ void store(int i, int j, int grp, int split, float v) const {
    if (i >= M || j >= Nn) return;
    long long V = M;
    out[(long long)split * V * g.K + V * ((long long)grp * g.Kg + j) + i] = v;
  }
};

// ---------------------------------------------------------------- the kernel
template <class Op>
__global__ void __launch_bounds__(kThreads) igemm_simt_kernel(Op op)
{
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  int grp = blockIdx.z / op.splits, split = blockIdx.z % op.splits;
  int i0 = blockIdx.x * BM, j0 = blockIdx.y * BN;
  int chunk = ((op.R + op.splits - 1) / op.splits + BK - 1) / BK * BK;
  int rBeg = split * chunk, rEnd = min(op.R, rBeg + chunk);

  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

  typename Op::ICtx ictx[4];
  if (Op::kIFast) ictx[0] = op.decodeI(i0 + (tid & 63), grp);
  else
#pragma unroll
    for (int t = 0; t < 4; ++t) ictx[t] = op.decodeI(i0 + (tid >> 4) + 16 * t, grp);

  for (int r0 = rBeg; r0 < rEnd; r0 += BK) {
    if (Op::kIFast) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        int rl = (tid >> 6) + 4 * t;
        int r = r0 + rl;
        typename Op::RCtx rc = op.decodeR(r < rEnd ? r : op.R, grp);
        As[rl][tid & 63] = op.A(ictx[0], rc);
      }
    } else {
      int r = r0 + (tid & 15);
      typename Op::RCtx rc = op.decodeR(r < rEnd ? r : op.R, grp);
#pragma unroll
      for (int t = 0; t < 4; ++t) As[tid & 15][(tid >> 4) + 16 * t] = op.A(ictx[t], rc);
    }
    {
      int r = r0 + (tid & 15);
      typename Op::RCtx rc = op.decodeR(r < rEnd ? r : op.R, grp);
#pragma unroll
      for (int t = 0; t < 4; ++t) Bs[tid & 15][(tid >> 4) + 16 * t] = op.B(j0 + (tid >> 4) + 16 * t, rc, grp);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) { a[t] = As[kk][tx + 16 * t]; b[t] = Bs[kk][ty + 16 * t]; }
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(a[p], b[q], acc[p][q]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int p = 0; p < 4; ++p)
#pragma unroll
    for (int q = 0; q < 4; ++q) op.store(i0 + tx + 16 * p, j0 + ty + 16 * q, grp, split, acc[p][q]);
}

// dF[e] = sum over splits (ascending) of partial[s][e]
__global__ void splitk_reduce_kernel(float* __restrict__ out, float const* __restrict__ part, size_t n, int splits)
{
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    float s = part[e];
    for (int k = 1; k < splits; ++k) s += part[(size_t)k * n + e];
    out[e] = s;
  }
}

}  // namespace

namespace vlb {

int conv_fprop_simt(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                    float const* F, float const* b)
{
  FpropOp op;
  op.g = g; op.x = X; op.f = F; op.b = b; op.y = Y; op.outMult = outMult; op.inMult = inMult;
  long long M = (long long)g.Ho * g.Wo * g.N;
  VLB_REQUIRE(ctx, M < (1LL << 31) - BM, "conv: output too large for 32-bit pixel index");
  op.M = (int)M; op.Nn = g.Kg; op.R = g.FH * g.FW * g.FC; op.splits = 1;
  dim3 grid(ceil_div(op.M, BM), ceil_div(op.Nn, BN), g.G);
  VLB_REQUIRE(ctx, grid.y <= 65535 && grid.z <= 65535, "conv: too many filters or groups");
  igemm_simt_kernel<FpropOp><<<grid, kThreads, 0, ctx->stream>>>(op);
  VLB_LAUNCHED(ctx, 1);
  return check_launch(ctx, "conv_fprop_simt");
}

int conv_dgrad_simt(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY)
{
  DgradOp op;
  op.g = g; op.dy = dY; op.f = F; op.dx = dX;
  long long M = (long long)g.H * g.W * g.N;
  VLB_REQUIRE(ctx, M < (1LL << 31) - BM, "conv: input too large for 32-bit pixel index");
  op.M = (int)M; op.Nn = g.FC; op.R = g.FH * g.FW * g.Kg; op.splits = 1;
  dim3 grid(ceil_div(op.M, BM), ceil_div(op.Nn, BN), g.G);
  VLB_REQUIRE(ctx, grid.y <= 65535 && grid.z <= 65535, "conv: too many channels or groups");
  igemm_simt_kernel<DgradOp><<<grid, kThreads, 0, ctx->stream>>>(op);
  VLB_LAUNCHED(ctx, 1);
  return check_launch(ctx, "conv_dgrad_simt");
}

int conv_wgrad_simt(vlb_ctx* ctx, ConvGeom const& g, float* dF, float const* X, float const* dY)
{
  WgradOp op;
  op.g = g; op.x = X; op.dy = dY;
  long long R = (long long)g.Ho * g.Wo * g.N;
  VLB_REQUIRE(ctx, R < (1LL << 31) - BK, "conv: output too large for 32-bit pixel index");
  op.M = g.FH * g.FW * g.FC; op.Nn = g.Kg; op.R = (int)R;
  int tiles = ceil_div(op.M, BM) * ceil_div(op.Nn, BN) * g.G;
  int splits = 1;
  if (tiles < 2 * ctx->smCount) {
    splits = (2 * ctx->smCount + tiles - 1) / tiles;
    int maxSplits = ceil_div(op.R, 4 * BK);
    if (splits > maxSplits) splits = maxSplits;
    if (splits < 1) splits = 1;
    if ((long long)g.G * splits > 65535) splits = 65535 / g.G;
  }
  op.splits = splits;
  size_t nF = (size_t)op.M * g.K;
  if (splits > 1) {
    float* part = (float*)workspace(ctx, sizeof(float) * nF * splits);
    if (!part) return pass_error(ctx, ctx->lastError, "conv_wgrad_simt");
    op.out = part;
  } else {
    op.out = dF;
  }
  dim3 grid(ceil_div(op.M, BM), ceil_div(op.Nn, BN), g.G * splits);
  VLB_REQUIRE(ctx, grid.y <= 65535 && grid.z <= 65535, "conv: too many filters or groups");
  igemm_simt_kernel<WgradOp><<<grid, kThreads, 0, ctx->stream>>>(op);
  VLB_LAUNCHED(ctx, 1);
  if (splits > 1) {
    splitk_reduce_kernel<<<grid_for(nF, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(dF, op.out, nF, splits);
    VLB_LAUNCHED(ctx, 1);
  }
  return check_launch(ctx, "conv_wgrad_simt");
}

}  // namespace vlb
