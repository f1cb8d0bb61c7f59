// Entry points of vl::nn::Convolution and vl::nn::FullyConnected (reference
// bits/nnconv.cu:444-468, bits/nnfullyconnected.cu:190-216): validation as the MEX
// gateway does it (matlab/src/vl_nnconv.cu:281-342), then dispatch to the tensor-core
// kernels or, for what they do not cover and for VLB_PRECISION_FP32, the CUDA-core ones.
#include "conv_internal.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {

using vlb::ConvGeom;

constexpr int kCluster = 8;
constexpr int kThreads = 256;

// db[k] = sum over pixels and images of dy (reference bits/nnconv.cu:229-244).  One
// cluster of kCluster CTAs per filter; partials meet in rank 0 through distributed shared
// memory in rank order: deterministic, no scratch.
template <bool kVec>
__global__ void __cluster_dims__(1, kCluster, 1) __launch_bounds__(kThreads)
conv_dbias_kernel(float* __restrict__ db, float const* __restrict__ dy, int P, int K, int N)
{
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float part;
  __shared__ float warpRed[kThreads / 32];
  int k = blockIdx.x, rank = (int)cluster.block_rank();
  float acc = 0.f;
  if (kVec) {
    int P4 = P >> 2;
    long long items = (long long)N * P4;
    for (long long i = (long long)rank * kThreads + threadIdx.x; i < items; i += (long long)kCluster * kThreads) {
      int n = (int)(i / P4), q = (int)(i - (long long)n * P4);
      float4 v = *reinterpret_cast<float4 const*>(dy + ((size_t)n * K + k) * (size_t)P + 4 * (size_t)q);
      acc += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    long long items = (long long)N * P;
    for (long long i = (long long)rank * kThreads + threadIdx.x; i < items; i += (long long)kCluster * kThreads) {
      int n = (int)(i / P), q = (int)(i - (long long)n * P);
      acc += dy[((size_t)n * K + k) * (size_t)P + q];
    }
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warpRed[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) s += warpRed[w];
    part = s;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    float s = 0.f;
    for (int r = 0; r < kCluster; ++r) s += *cluster.map_shared_rank(&part, r);
    db[k] = s;
  }
  cluster.sync();
}

// The same for 1x1 outputs (fully connected layers): db[k] = sum over images of dy[k + K*n]; one thread per
// filter, reads coalesced across the filters, images added in order.
__global__ void conv_dbias_p1_kernel(float* __restrict__ db, float const* __restrict__ dy, int K, int N)
{
  int const k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float s = 0.f;
  for (int n = 0; n < N; ++n) s += dy[(size_t)n * K + k];
  db[k] = s;
}

int launch_dbias(vlb_ctx* ctx, float* db, float const* dY, int P, int K, int N)
{
  if (P == 1) {
    conv_dbias_p1_kernel<<<vlb::ceil_div(K, 128), 128, 0, ctx->stream>>>(db, dY, K, N);
    VLB_LAUNCHED(ctx, 1);
    return vlb::check_launch(ctx, "conv_dbias");
  }
  bool vec = (P % 4 == 0) && ((((uintptr_t)dY) & 15) == 0);
  dim3 grid(K, kCluster);
  if (vec) conv_dbias_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(db, dY, P, K, N);
  else     conv_dbias_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(db, dY, P, K, N);
  VLB_LAUNCHED(ctx, 1);
  return vlb::check_launch(ctx, "conv_dbias");
}

__global__ void copy_kernel(float* dst, float const* src, size_t n)
{
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

int make_geom(vlb_ctx* ctx, vlb_conv_desc const* d, ConvGeom* g)
{
  VLB_REQUIRE(ctx, d, "conv: null descriptor");
  VLB_REQUIRE(ctx, d->H > 0 && d->W > 0 && d->C > 0 && d->N > 0, "conv: empty input");
  VLB_REQUIRE(ctx, d->FH > 0 && d->FW > 0 && d->FC > 0 && d->K > 0, "conv: empty filter bank");
  VLB_REQUIRE(ctx, d->strideY >= 1 && d->strideX >= 1, "conv: at least one element of STRIDE is smaller than one");
  VLB_REQUIRE(ctx, d->dilateY >= 1 && d->dilateX >= 1, "conv: at least one element of DILATE is smaller than one");
  VLB_REQUIRE(ctx, d->padTop >= 0 && d->padBottom >= 0 && d->padLeft >= 0 && d->padRight >= 0,
              "conv: an element of PAD is negative");
  // matlab/src/vl_nnconv.cu:301-322
  VLB_REQUIRE(ctx, d->C % d->FC == 0, "conv: the FILTERS depth does not divide the DATA depth");
  int G = d->C / d->FC;
  VLB_REQUIRE(ctx, d->K % G == 0, "conv: the number of filter groups does not divide the number of filters");
  int extY = (d->FH - 1) * d->dilateY + 1, extX = (d->FW - 1) * d->dilateX + 1;
  VLB_REQUIRE(ctx, d->H + d->padTop + d->padBottom >= extY && d->W + d->padLeft + d->padRight >= extX,
              "conv: FILTERS are larger than the DATA (including padding)");
  g->H = d->H; g->W = d->W; g->C = d->C; g->N = d->N;
  g->FH = d->FH; g->FW = d->FW; g->FC = d->FC; g->K = d->K;
  g->sy = d->strideY; g->sx = d->strideX;
  g->pt = d->padTop; g->pb = d->padBottom; g->pl = d->padLeft; g->pr = d->padRight;
  g->dy = d->dilateY; g->dx = d->dilateX;
  g->Ho = (d->H + d->padTop + d->padBottom - extY) / d->strideY + 1;
  g->Wo = (d->W + d->padLeft + d->padRight - extX) / d->strideX + 1;
  g->G = G; g->Kg = d->K / G;
  VLB_REQUIRE(ctx, (long long)d->H * d->W * d->C * d->N < (1LL << 40), "conv: input too large");
  return VLB_Success;
}

int check_fc(vlb_ctx* ctx, vlb_conv_desc const* d)
{
  VLB_REQUIRE(ctx, d, "fc: null descriptor");
  // the conditions under which the gateway takes the fully-connected route (matlab/src/vl_nnconv.cu:351-361)
  VLB_REQUIRE(ctx, d->FH == d->H && d->FW == d->W && d->FC == d->C, "fc: the filters must cover the whole input");
  VLB_REQUIRE(ctx, d->strideY == 1 && d->strideX == 1 && d->dilateY == 1 && d->dilateX == 1 && d->padTop == 0 &&
                   d->padBottom == 0 && d->padLeft == 0 && d->padRight == 0, "fc: stride/pad/dilate must be trivial");
  return VLB_Success;
}

}  // namespace

extern "C" {

int vlb_conv_output_shape(vlb_conv_desc const* d, int* Ho, int* Wo)
{
  if (!d || d->strideY < 1 || d->strideX < 1) return VLB_IllegalArgument;
  if (Ho) *Ho = (d->H + d->padTop + d->padBottom - ((d->FH - 1) * d->dilateY + 1)) / d->strideY + 1;
  if (Wo) *Wo = (d->W + d->padLeft + d->padRight - ((d->FW - 1) * d->dilateX + 1)) / d->strideX + 1;
  return VLB_Success;
}

int vlb_conv_forward(vlb_ctx* ctx, float* Y, double outMult, float const* X, double inMult, float const* F,
                     float const* b, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  ConvGeom g;
  int rc = make_geom(ctx, d, &g);
  if (rc) return vlb::pass_error(ctx, rc, "vlb_conv_forward");
  VLB_REQUIRE(ctx, Y && X && F, "conv_forward: null tensor");
  rc = vlb::conv_fprop_small(ctx, g, Y, (float)outMult, X, (float)inMult, F, b);
  if (rc != VLB_Unsupported) return rc ? vlb::pass_error(ctx, rc, "vlb_conv_forward") : rc;
  if (ctx->precision != VLB_PRECISION_FP32) {
    rc = vlb::conv_fprop_tc(ctx, g, Y, (float)outMult, X, (float)inMult, F, b);
    if (rc != VLB_Unsupported) return rc ? vlb::pass_error(ctx, rc, "vlb_conv_forward") : rc;
    ctx->reluDone = false;      // the CUDA-core kernel below has no fused ReLU
  }
  rc = vlb::conv_fprop_simt(ctx, g, Y, (float)outMult, X, (float)inMult, F, b);
  return rc ? vlb::pass_error(ctx, rc, "vlb_conv_forward") : rc;
}

int vlb_conv_relu_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  ctx->fuseRelu = true; ctx->reluDone = false;
  int rc = vlb_conv_forward(ctx, Y, 0.0, X, 1.0, F, b, d);
  bool const done = ctx->reluDone;
  ctx->fuseRelu = false; ctx->reluDone = false;
  if (rc || done) return rc;
  int Ho = 0, Wo = 0;
  vlb_conv_output_shape(d, &Ho, &Wo);
  return vlb_relu_forward(ctx, Y, Y, (size_t)Ho * Wo * d->K * d->N);
}

int vlb_conv_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                      float const* dY, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  ConvGeom g;
  int rc = make_geom(ctx, d, &g);
  if (rc) return vlb::pass_error(ctx, rc, "vlb_conv_backward");
  VLB_REQUIRE(ctx, dY, "conv_backward: null derOutput");
  VLB_REQUIRE(ctx, !dX || F, "conv_backward: the data derivative needs the filters");
  VLB_REQUIRE(ctx, !dF || X, "conv_backward: the filter derivative needs the data");
  bool tc = ctx->precision != VLB_PRECISION_FP32;
  bool dbDone = false;
  if (dF) {
    rc = vlb::conv_wgrad_small(ctx, g, dF, db, X, dY, &dbDone);
    if (rc == VLB_Unsupported) rc = tc ? vlb::conv_wgrad_tc(ctx, g, dF, db, X, dY, &dbDone) : VLB_Unsupported;
    if (rc == VLB_Unsupported) rc = vlb::conv_wgrad_simt(ctx, g, dF, X, dY);
    if (rc) return vlb::pass_error(ctx, rc, "vlb_conv_backward");
  }
  if (db && !dbDone) {
    rc = launch_dbias(ctx, db, dY, g.Ho * g.Wo, g.K, g.N);
    if (rc) return vlb::pass_error(ctx, rc, "vlb_conv_backward");
  }
  if (dX) {
    rc = vlb::conv_dgrad_small(ctx, g, dX, F, dY);
    if (rc == VLB_Unsupported) rc = tc ? vlb::conv_dgrad_tc(ctx, g, dX, F, dY) : VLB_Unsupported;
    if (rc == VLB_Unsupported) rc = vlb::conv_dgrad_simt(ctx, g, dX, F, dY);
    if (rc) return vlb::pass_error(ctx, rc, "vlb_conv_backward");
  }
  return VLB_Success;
}

int vlb_relu_conv_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                           float const* dY, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  VLB_REQUIRE(ctx, !dX || X, "relu_conv_backward: the data derivative needs the data (the ReLU's output)");
  ctx->reluMask = dX ? X : nullptr; ctx->maskDone = false;
  int rc = vlb_conv_backward(ctx, dX, dF, db, X, F, dY, d);
  bool const done = ctx->maskDone;
  ctx->reluMask = nullptr; ctx->maskDone = false;
  if (rc || done || !dX) return rc;
  return vlb_relu_backward(ctx, dX, X, dX, (size_t)d->H * d->W * d->C * d->N);
}

// ---- convolution transpose: the convolution whose data gradient / forward pass it re-uses ------------------
// The transposed convolution of X (H x W x C x N) with F (FH x FW x FD x C) is the data gradient of a convolution
// with stride = upsample and pad = crop whose input is the transposed convolution's output (reference
// bits/nnconv.cu:323-374); c receives that convolution's descriptor.
static int convt_geom(vlb_ctx* ctx, vlb_convt_desc const* d, vlb_conv_desc* c)
{
  VLB_REQUIRE(ctx, d, "convt: null descriptor");
  VLB_REQUIRE(ctx, d->H > 0 && d->W > 0 && d->C > 0 && d->N > 0, "convt: empty input");
  // matlab/src/vl_nnconvt.cu:262-290
  VLB_REQUIRE(ctx, d->upsampleY >= 1 && d->upsampleX >= 1, "convt: at least one element of UPSAMPLE is smaller than one");
  VLB_REQUIRE(ctx, d->cropTop >= 0 && d->cropBottom >= 0 && d->cropLeft >= 0 && d->cropRight >= 0,
              "convt: an element of CROP is negative");
  VLB_REQUIRE(ctx, d->FH > 0 && d->FW > 0 && d->FD > 0, "convt: a dimension of FILTERS is void");
  VLB_REQUIRE(ctx, d->numGroups >= 1, "convt: NUMGROUPS is less than 1");
  VLB_REQUIRE(ctx, d->FN % d->numGroups == 0, "convt: the number of filter groups does not divide the filter bank depth");
  VLB_REQUIRE(ctx, d->FN == d->C, "convt: the filter bank depth is not the same as the data depth");
  int Ho = 0, Wo = 0;
  vlb_convt_output_shape(d, &Ho, &Wo);
  VLB_REQUIRE(ctx, Ho >= 1 && Wo >= 1, "convt: the output array is empty due to CROP being too large");   // :299-301
  c->H = Ho; c->W = Wo; c->C = d->FD * d->numGroups; c->N = d->N;
  c->FH = d->FH; c->FW = d->FW; c->FC = d->FD; c->K = d->C;
  c->strideY = d->upsampleY; c->strideX = d->upsampleX;
  c->padTop = d->cropTop; c->padBottom = d->cropBottom; c->padLeft = d->cropLeft; c->padRight = d->cropRight;
  c->dilateY = 1; c->dilateX = 1;
  return VLB_Success;
}

int vlb_convt_output_shape(vlb_convt_desc const* d, int* Ho, int* Wo)
{
  if (!d) return VLB_IllegalArgument;
  if (Ho) *Ho = (d->H - 1) * d->upsampleY - (d->cropTop + d->cropBottom) + d->FH;
  if (Wo) *Wo = (d->W - 1) * d->upsampleX - (d->cropLeft + d->cropRight) + d->FW;
  return VLB_Success;
}

int vlb_convt_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b, vlb_convt_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  vlb_conv_desc c;
  int rc = convt_geom(ctx, d, &c);
  if (rc) return vlb::pass_error(ctx, rc, "vlb_convt_forward");
  VLB_REQUIRE(ctx, Y && X && F, "convt_forward: null tensor");
  // the whole batch in one call: this engine's data gradient writes every image's own slice (the reference loops over
  // the images because its row2im accumulates, bits/nnconv.cu:338-367)
  rc = vlb_conv_backward(ctx, Y, nullptr, nullptr, nullptr, F, X, &c);
  if (rc || !b) return rc;
  return vlb_bias_forward(ctx, Y, 1.0, nullptr, 0.0, b, 1.0, c.H, c.W, c.C, c.N);       // bits/nnconv.cu:368-370
}

int vlb_convt_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                       float const* dY, vlb_convt_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  vlb_conv_desc c;
  int rc = convt_geom(ctx, d, &c);
  if (rc) return vlb::pass_error(ctx, rc, "vlb_convt_backward");
  VLB_REQUIRE(ctx, dY, "convt_backward: null derOutput");
  VLB_REQUIRE(ctx, !dX || F, "convt_backward: the data derivative needs the filters");
  VLB_REQUIRE(ctx, !dF || X, "convt_backward: the filter derivative needs the data");
  if (dX) {                                             // bits/nnconv.cu:398-403
    rc = vlb_conv_forward(ctx, dX, 0.0, dY, 1.0, F, nullptr, &c);
    if (rc) return rc;
  }
  if (dF) {                                             // :405-409: the roles of data and output derivative exchanged
    rc = vlb_conv_backward(ctx, nullptr, dF, nullptr, dY, nullptr, X, &c);
    if (rc) return rc;
  }
  if (db) return vlb_bias_backward(ctx, nullptr, 0.0, db, 0.0, 0.0, 1.0, dY, c.H, c.W, c.C, c.N);      // :411-414
  return VLB_Success;
}

int vlb_fc_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  if (!F) {
    // null filters: copy (reference bits/nnfullyconnected.cu:71-76), then the bias
    VLB_REQUIRE(ctx, d && Y && X, "fc_forward: null tensor");
    size_t n = (size_t)d->H * d->W * d->C * d->N;
    copy_kernel<<<vlb::grid_for(n, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(Y, X, n);
    VLB_LAUNCHED(ctx, 1);
    if (b) return vlb_bias_forward(ctx, Y, 1.0, nullptr, 0.0, b, 1.0, 1, 1, d->H * d->W * d->C, d->N);
    return vlb::check_launch(ctx, "vlb_fc_forward");
  }
  int rc = check_fc(ctx, d);
  if (rc) return rc;
  return vlb_conv_forward(ctx, Y, 0.0, X, 1.0, F, b, d);
}

int vlb_fc_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                    float const* dY, vlb_conv_desc const* d)
{
  if (!ctx) return VLB_IllegalArgument;
  if (!F) {
    // null filters: dX = dY (reference bits/nnfullyconnected.cu:152-157)
    VLB_REQUIRE(ctx, d && dY, "fc_backward: null tensor");
    size_t n = (size_t)d->H * d->W * d->C * d->N;
    if (dX) {
      copy_kernel<<<vlb::grid_for(n, 256, ctx->smCount * 8), 256, 0, ctx->stream>>>(dX, dY, n);
      VLB_LAUNCHED(ctx, 1);
    }
    if (db) return launch_dbias(ctx, db, dY, 1, d->H * d->W * d->C, d->N);
    return vlb::check_launch(ctx, "vlb_fc_backward");
  }
  int rc = check_fc(ctx, d);
  if (rc) return rc;
  return vlb_conv_backward(ctx, dX, dF, db, X, F, dY, d);
}

}  // extern "C"
