// tcgen05 implicit-GEMM convolution (placeholder until the tensor-core kernels land).
#include "conv_internal.cuh"

namespace vlb {

int conv_fprop_tc(vlb_ctx*, ConvGeom const&, float*, float, float const*, float, float const*, float const*)
{ return VLB_Unsupported; }
int conv_dgrad_tc(vlb_ctx*, ConvGeom const&, float*, float const*, float const*) { return VLB_Unsupported; }
int conv_wgrad_tc(vlb_ctx*, ConvGeom const&, float*, float*, float const*, float const*, bool*) { return VLB_Unsupported; }

}  // namespace vlb
