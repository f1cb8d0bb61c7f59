// vl::nn::BilinearSampler with the reference's interface (reference matlab/src/bits/nnbilinearsampler.hpp:21-36).
#ifndef VLB_NNBILINEARSAMPLER_HPP
#define VLB_NNBILINEARSAMPLER_HPP
#include "data.hpp"
namespace vl { namespace nn {

class BilinearSampler {
public:
  BilinearSampler(Context& context) : context(context) {}
  ErrorCode forward(Tensor& output, Tensor const& input, Tensor const& grid)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_sampler_forward(c, impl::f(output), impl::f(input), impl::f(grid), (int)input.getHeight(), (int)input.getWidth(),
                                             (int)input.getDepth(), (int)input.getSize(), (int)output.getHeight(), (int)output.getWidth(),
                                             (int)output.getSize()), "BilinearSampler::forward");
  }
  // derInput and derGrid are overwritten (either may be a null tensor)
  ErrorCode backward(Tensor& derInput, Tensor& derGrid, Tensor const& input, Tensor const& grid, Tensor const& derOutput)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    Tensor const& x = input ? input : static_cast<Tensor const&>(derInput);
    return context.check(vlb_sampler_backward(c, impl::f(derInput), impl::f(derGrid), impl::f(input), impl::f(grid), impl::f(derOutput),
                                              (int)x.getHeight(), (int)x.getWidth(), (int)x.getDepth(), (int)x.getSize(),
                                              (int)derOutput.getHeight(), (int)derOutput.getWidth(), (int)derOutput.getSize()),
                         "BilinearSampler::backward");
  }
  Context& context;
};

} }
#endif
