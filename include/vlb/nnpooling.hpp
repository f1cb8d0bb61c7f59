// vl::nn::Pooling with the reference's interface (reference matlab/src/bits/nnpooling.hpp:21-49).
#ifndef VLB_NNPOOLING_HPP
#define VLB_NNPOOLING_HPP
#include "data.hpp"
namespace vl { namespace nn {

class Pooling {
public:
  enum Method { Max, Average };
  Pooling(Context& context, int poolHeight, int poolWidth, int strideY, int strideX, int padTop, int padBottom, int padLeft,
          int padRight, Method method)
  : context(context), poolHeight(poolHeight), poolWidth(poolWidth), strideY(strideY), strideX(strideX), padTop(padTop),
    padBottom(padBottom), padLeft(padLeft), padRight(padRight), method(method) {}
  ErrorCode forward(Tensor& output, Tensor const& input)
  {
    vlb_pool_desc d = desc(input);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_pool_forward(c, impl::f(output), impl::f(input), &d), "Pooling::forward");
  }
  // derInput is overwritten with the sum of the contributions (the reference accumulates into a zero-filled array)
  ErrorCode backward(Tensor& derInput, Tensor const& input, Tensor const& derOutput)
  {
    vlb_pool_desc d = desc(input);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_pool_backward(c, impl::f(derInput), impl::f(input), impl::f(derOutput), &d), "Pooling::backward");
  }
  Context& context;
  int poolHeight, poolWidth, strideY, strideX, padTop, padBottom, padLeft, padRight;
  Method method;
private:
  vlb_pool_desc desc(Tensor const& x) const
  {
    vlb_pool_desc d = {(int)x.getHeight(), (int)x.getWidth(), (int)x.getDepth(), (int)x.getSize(), poolHeight, poolWidth, strideY,
                       strideX, padTop, padBottom, padLeft, padRight, method == Max ? VLB_POOL_MAX : VLB_POOL_AVG};
    return d;
  }
};

} }
#endif
