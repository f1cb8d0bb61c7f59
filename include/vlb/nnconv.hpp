// vl::nn::Convolution with the reference's interface (reference matlab/src/bits/nnconv.hpp:23-52).
#ifndef VLB_NNCONV_HPP
#define VLB_NNCONV_HPP
#include "data.hpp"
namespace vl { namespace nn {

class Convolution {
public:
  Convolution(Context& context, int strideY, int strideX, int padTop, int padBottom, int padLeft, int padRight,
              int dilateY, int dilateX)
  : context(context), strideY(strideY), strideX(strideX), padTop(padTop), padBottom(padBottom), padLeft(padLeft),
    padRight(padRight), dilateY(dilateY), dilateX(dilateX) {}

  // output <- outputMult * output + inputMult * conv(input, filter) + bias   (nnconv.cu:71-157)
  ErrorCode forward(Tensor& output, double outputMult, Tensor const& input, double inputMult, Tensor const& filter,
                    Tensor const& bias)
  {
    if (!impl::gpuFloat(input) || !impl::gpuFloat(filter) || !impl::gpuFloat(output)) return context.setError(VLE_Unsupported, "GPU single precision only");
    vlb_conv_desc d = desc(input, filter);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_conv_forward(c, impl::f(output), outputMult, impl::f(input), inputMult, impl::f(filter), impl::f(bias), &d),
                         "Convolution::forward");
  }

  // any of derInput / derFilter / derBias may be a null tensor and is then skipped (nnconv.cu:163-317)
  ErrorCode backward(Tensor& derInput, Tensor& derFilter, Tensor& derBias, Tensor const& input, Tensor const& filter,
                     Tensor const& derOutput)
  {
    if (!impl::gpuFloat(derOutput) || !impl::gpuFloat(input) || !impl::gpuFloat(filter)) return context.setError(VLE_Unsupported, "GPU single precision only");
    Tensor const& x = input ? input : static_cast<Tensor const&>(derInput);
    Tensor const& w = filter ? filter : static_cast<Tensor const&>(derFilter);
    vlb_conv_desc d = desc(x, w);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_conv_backward(c, impl::f(derInput), impl::f(derFilter), impl::f(derBias), impl::f(input), impl::f(filter),
                                           impl::f(derOutput), &d), "Convolution::backward");
  }

  Context& context;
  int strideY, strideX, padTop, padBottom, padLeft, padRight, dilateY, dilateX;

private:
  vlb_conv_desc desc(Tensor const& x, Tensor const& w) const
  {
    vlb_conv_desc d = {(int)x.getHeight(), (int)x.getWidth(), (int)x.getDepth(), (int)x.getSize(),
                       (int)w.getHeight(), (int)w.getWidth(), (int)w.getDepth(), (int)w.getSize(),
                       strideY, strideX, padTop, padBottom, padLeft, padRight, dilateY, dilateX};
    return d;
  }
};

// vl::nn::ConvolutionTranspose (bits/nnconv.hpp:54-80)
class ConvolutionTranspose {
public:
  ConvolutionTranspose(Context& context, int upsampleY, int upsampleX, int cropTop, int cropBottom, int cropLeft, int cropRight)
    : context(context), upsampleY(upsampleY), upsampleX(upsampleX), cropTop(cropTop), cropBottom(cropBottom),
      cropLeft(cropLeft), cropRight(cropRight) {}

  // output <- the data gradient of the convolution with stride = upsample, pad = crop, plus bias   (nnconv.cu:323-374)
  ErrorCode forward(Tensor& output, Tensor const& input, Tensor const& filter, Tensor const& bias)
  {
    if (!impl::gpuFloat(input) || !impl::gpuFloat(filter) || !impl::gpuFloat(output)) return context.setError(VLE_Unsupported, "GPU single precision only");
    vlb_convt_desc d = desc(input, filter, output);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_convt_forward(c, impl::f(output), impl::f(input), impl::f(filter), impl::f(bias), &d),
                         "ConvolutionTranspose::forward");
  }

  // any of derData / derFilter / derBias may be a null tensor and is then skipped (nnconv.cu:380-421)
  ErrorCode backward(Tensor& derData, Tensor& derFilter, Tensor& derBias, Tensor const& input, Tensor const& filter,
                     Tensor const& derOutput)
  {
    if (!impl::gpuFloat(derOutput) || !impl::gpuFloat(input) || !impl::gpuFloat(filter)) return context.setError(VLE_Unsupported, "GPU single precision only");
    Tensor const& x = input ? input : static_cast<Tensor const&>(derData);
    Tensor const& w = filter ? filter : static_cast<Tensor const&>(derFilter);
    vlb_convt_desc d = desc(x, w, derOutput);
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_convt_backward(c, impl::f(derData), impl::f(derFilter), impl::f(derBias), impl::f(input),
                                            impl::f(filter), impl::f(derOutput), &d), "ConvolutionTranspose::backward");
  }

  Context& context;
  int upsampleY, upsampleX, cropTop, cropBottom, cropLeft, cropRight;

private:
  // the number of filter groups follows from the output depth (matlab/src/vl_nnconvt.cu:293-296)
  vlb_convt_desc desc(Tensor const& x, Tensor const& w, Tensor const& y) const
  {
    int const fd = (int)w.getDepth();
    vlb_convt_desc d = {(int)x.getHeight(), (int)x.getWidth(), (int)x.getDepth(), (int)x.getSize(),
                        (int)w.getHeight(), (int)w.getWidth(), fd, (int)w.getSize(),
                        upsampleY, upsampleX, cropTop, cropBottom, cropLeft, cropRight,
                        fd > 0 ? (int)y.getDepth() / fd : 1};
    return d;
  }
};

} }
#endif
