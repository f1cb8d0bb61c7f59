// vl::nn::BatchNorm with the reference's interface (reference matlab/src/bits/nnbnorm.hpp:22-59).
// moment = [mean(C); sigma(C)], sigma = sqrt(variance + epsilon); a null moment tensor means
// "compute it and keep it in scratch" (nnbnorm.cu:233-240,336-344).
#ifndef VLB_NNBNORM_HPP
#define VLB_NNBNORM_HPP
#include "data.hpp"
namespace vl { namespace nn {

class BatchNorm {
public:
  BatchNorm(Context& context, double epsilon) : context(context), epsilon(epsilon) {}
  ErrorCode forward(Tensor& output, Tensor& moment, Tensor const& input, Tensor const& multiplier, Tensor const& bias)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bnorm_forward(c, impl::f(output), impl::f(moment), impl::f(input), impl::f(multiplier), impl::f(bias),
                                           (int)input.getHeight(), (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), epsilon),
                         "BatchNorm::forward");
  }
  ErrorCode forwardWithMoment(Tensor& output, Tensor const& moment, Tensor const& input, Tensor const& multiplier, Tensor const& bias)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bnorm_forward_moment(c, impl::f(output), impl::f(moment), impl::f(input), impl::f(multiplier), impl::f(bias),
                                                  (int)input.getHeight(), (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), epsilon),
                         "BatchNorm::forwardWithMoment");
  }
  ErrorCode backward(Tensor& derInput, Tensor& derMultiplier, Tensor& derBias, Tensor& moment, Tensor const& input,
                     Tensor const& multiplier, Tensor const& bias, Tensor const& derOutput)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bnorm_backward(c, impl::f(derInput), impl::f(derMultiplier), impl::f(derBias), impl::f(moment), impl::f(input),
                                            impl::f(multiplier), impl::f(bias), impl::f(derOutput), (int)input.getHeight(), (int)input.getWidth(),
                                            (int)input.getDepth(), (int)input.getSize(), epsilon), "BatchNorm::backward");
  }
  ErrorCode backwardWithMoment(Tensor& derInput, Tensor& derMultiplier, Tensor& derBias, Tensor const& moment, Tensor const& input,
                               Tensor const& multiplier, Tensor const& bias, Tensor const& derOutput)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bnorm_backward_moment(c, impl::f(derInput), impl::f(derMultiplier), impl::f(derBias), impl::f(moment),
                                                   impl::f(input), impl::f(multiplier), impl::f(bias), impl::f(derOutput), (int)input.getHeight(),
                                                   (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), epsilon),
                         "BatchNorm::backwardWithMoment");
  }
  Context& context;
  double epsilon;
};

} }
#endif
