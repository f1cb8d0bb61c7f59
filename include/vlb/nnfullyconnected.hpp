// vl::nn::FullyConnected with the reference's interface (reference matlab/src/bits/nnfullyconnected.hpp:20-37).
#ifndef VLB_NNFULLYCONNECTED_HPP
#define VLB_NNFULLYCONNECTED_HPP
#include "data.hpp"
namespace vl { namespace nn {

class FullyConnected {
public:
  FullyConnected(Context& context) : context(context) {}
  ErrorCode forward(Tensor& output, Tensor const& input, Tensor const& filter, Tensor const& bias)
  {
    vlb_conv_desc d = desc(input, filter);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_fc_forward(c, impl::f(output), impl::f(input), impl::f(filter), impl::f(bias), &d), "FullyConnected::forward");
  }
  ErrorCode backward(Tensor& derInput, Tensor& derFilter, Tensor& derBias, Tensor const& input, Tensor const& filter,
                     Tensor const& derOutput)
  {
    vlb_conv_desc d = desc(input ? input : static_cast<Tensor const&>(derInput), filter ? filter : static_cast<Tensor const&>(derFilter));
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_fc_backward(c, impl::f(derInput), impl::f(derFilter), impl::f(derBias), impl::f(input), impl::f(filter),
                                         impl::f(derOutput), &d), "FullyConnected::backward");
  }
  Context& context;
private:
  static vlb_conv_desc desc(Tensor const& x, Tensor const& w)
  {
    int H = (int)x.getHeight(), W = (int)x.getWidth(), C = (int)x.getDepth(), N = (int)x.getSize();
    vlb_conv_desc d = {H, W, C, N, w ? (int)w.getHeight() : H, w ? (int)w.getWidth() : W, w ? (int)w.getDepth() : C,
                       w ? (int)w.getSize() : H * W * C, 1, 1, 0, 0, 0, 0, 1, 1};
    return d;
  }
};

} }
#endif
