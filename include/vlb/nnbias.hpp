// vl::nn::Bias with the reference's interface (reference matlab/src/bits/nnbias.hpp:20-35).
#ifndef VLB_NNBIAS_HPP
#define VLB_NNBIAS_HPP
#include "data.hpp"
namespace vl { namespace nn {

class Bias {
public:
  Bias(Context& context) : context(context) {}
  // output <- outputMult * output + inputMult * input + biasMult * bias
  ErrorCode forward(Tensor& output, double outputMult, Tensor const& input, double inputMult, Tensor const& bias, double biasMult)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bias_forward(c, impl::f(output), outputMult, impl::f(input), inputMult, impl::f(bias), biasMult,
                                          (int)output.getHeight(), (int)output.getWidth(), (int)output.getDepth(), (int)output.getSize()),
                         "Bias::forward");
  }
  ErrorCode backward(Tensor& derInput, double derInputMult, Tensor& derBias, double derBiasMult, double inputMult, double biasMult,
                     Tensor const& derOutput)
  {
    vlb_ctx* c = context.get();
    if (!c) return context.getLastError();
    return context.check(vlb_bias_backward(c, impl::f(derInput), derInputMult, impl::f(derBias), derBiasMult, inputMult, biasMult,
                                           impl::f(derOutput), (int)derOutput.getHeight(), (int)derOutput.getWidth(),
                                           (int)derOutput.getDepth(), (int)derOutput.getSize()), "Bias::backward");
  }
  Context& context;
};

} }
#endif
