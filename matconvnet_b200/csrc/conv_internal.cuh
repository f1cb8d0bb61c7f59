// Internal interfaces between the convolution translation units.
#pragma once
#include "common.cuh"

namespace vlb {

// Geometry of one convolution call, derived from vlb_conv_desc.
struct ConvGeom {
  int H, W, C, N;
  int FH, FW, FC, K;
  int Ho, Wo;
  int sy, sx, pt, pb, pl, pr, dy, dx;
  int G, Kg;        // groups = C / FC, filters per group = K / G
};

// CUDA-core implicit GEMM (conv_simt.cu): every configuration, exact fp32 products.
int conv_fprop_simt(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                    float const* F, float const* b);
int conv_dgrad_simt(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY);
int conv_wgrad_simt(vlb_ctx* ctx, ConvGeom const& g, float* dF, float const* X, float const* dY);

// Direct CUDA-core kernels for the image end of a network (conv_small.cu): forward with at most 64 input values
// per output pixel, data gradient onto at most 4 channels; at least 4096 output pixels.  VLB_Unsupported otherwise.
int conv_fprop_small(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                     float const* F, float const* b);
int conv_dgrad_small(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY);
int conv_wgrad_small(vlb_ctx* ctx, ConvGeom const& g, float* dF, float* db, float const* X, float const* dY, bool* dbDone);

// tcgen05 implicit GEMM (conv_tc.cu).  Each returns VLB_Unsupported -- without touching
// the context's error state -- when the configuration is outside what the tensor-core
// kernels cover, and the caller then takes the CUDA-core path.
int conv_fprop_tc(vlb_ctx* ctx, ConvGeom const& g, float* Y, float outMult, float const* X, float inMult,
                  float const* F, float const* b);
int conv_dgrad_tc(vlb_ctx* ctx, ConvGeom const& g, float* dX, float const* F, float const* dY);
int conv_wgrad_tc(vlb_ctx* ctx, ConvGeom const& g, float* dF, float* db, float const* X, float const* dY,
                  bool* dbDone);

}  // namespace vlb
