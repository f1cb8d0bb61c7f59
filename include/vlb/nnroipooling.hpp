// vl::nn::ROIPooling with the reference's interface (reference matlab/src/bits/nnroipooling.hpp:23-45).
#ifndef VLB_NNROIPOOLING_HPP
#define VLB_NNROIPOOLING_HPP
#include <array>
#include "data.hpp"
namespace vl { namespace nn {

class ROIPooling {
public:
  enum Method { Max, Average };
  ROIPooling(Context& context, std::array<int, 2> subdivisions, std::array<double, 6> transform, Method method)
  : context(context), subdivisions(subdivisions), transform(transform), method(method) {}
  ErrorCode forward(Tensor& output, Tensor const& input, Tensor const& rois)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_roipool_forward(c, impl::f(output), impl::f(input), impl::f(rois), (int)input.getHeight(), (int)input.getWidth(),
                                             (int)input.getDepth(), (int)input.getSize(), (int)(rois.getNumElements() / 5), subdivisions[0],
                                             subdivisions[1], transform.data(), method == Max ? VLB_POOL_MAX : VLB_POOL_AVG),
                         "ROIPooling::forward");
  }
  ErrorCode backward(Tensor& derInput, Tensor const& input, Tensor const& rois, Tensor const& derOutput)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_roipool_backward(c, impl::f(derInput), impl::f(input), impl::f(rois), impl::f(derOutput), (int)input.getHeight(),
                                              (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), (int)(rois.getNumElements() / 5),
                                              subdivisions[0], subdivisions[1], transform.data(), method == Max ? VLB_POOL_MAX : VLB_POOL_AVG),
                         "ROIPooling::backward");
  }
  Context& context;
  std::array<int, 2> subdivisions;
  std::array<double, 6> transform;
  Method method;
};

} }
#endif
