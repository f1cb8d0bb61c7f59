// The reference's operator classes (declared by its own headers matlab/src/bits/nnconv.hpp, nnfullyconnected.hpp,
// nnsubsample.hpp, nnbnorm.hpp, nnpooling.hpp, nnroipooling.hpp, nnbilinearsampler.hpp) DEFINED over the vlb C ABI.
// This is the binding a MatConvNet maintainer would add in place of bits/nn*.cu: the MEX gateways (vl_nnconv.cu, ...)
// compile unchanged against the same declarations and every device operation lands in libvlb.so.  Here it is linked
// with the unmodified gateways and a stand-in for the MEX API so that the gateways' own option parsing, shape checks
// and output allocation can be driven from a test without MATLAB.
//
// Single precision on the GPU only, like the engine: any other tensor gives VLE_Unsupported with a message.
#include "bits/data.hpp"
#include "bits/datacu.hpp"
#include "bits/nnconv.hpp"
#include "bits/nnfullyconnected.hpp"
#include "bits/nnsubsample.hpp"
#include "bits/nnbnorm.hpp"
#include "bits/nnpooling.hpp"
#include "bits/nnroipooling.hpp"
#include "bits/nnbilinearsampler.hpp"

#include "vlb.h"

#include <map>
#include <mutex>

namespace {

std::mutex g_lock;
std::map<vl::Context*, vlb_ctx*> g_engines;

// One engine context per vl::Context, created on first use and bound to the stream the reference's CudaHelper holds
// (CudaHelper::getStream, bits/datacu.hpp:69).
vlb_ctx* engine(vl::Context& context)
{
  std::lock_guard<std::mutex> guard(g_lock);
  vlb_ctx*& c = g_engines[&context];
  if (!c && vlb_ctx_create(&c) != VLB_Success) { c = nullptr; return nullptr; }
  vlb_ctx_set_stream(c, (void*)context.getCudaHelper().getStream());
  return c;
}

bool usable(vl::Tensor const& t)
{
  return t.isNull() || t.isEmpty() || (t.getDeviceType() == vl::VLDT_GPU && t.getDataType() == vl::VLDT_Float);
}

float* mem(vl::Tensor& t) { return t ? (float*)t.getMemory() : nullptr; }
float const* mem(vl::Tensor const& t) { return t ? (float const*)t.getMemory() : nullptr; }

vl::ErrorCode unsupported(vl::Context& context, char const* who)
{
  return context.setError(vl::VLE_Unsupported, (std::string(who) + ": the B200 engine takes single-precision gpuArrays only").c_str());
}

// Engine status -> the reference's error chain (Context::setError, bits/data.cu:332-352).
vl::ErrorCode done(vl::Context& context, vlb_ctx* c, int status, char const* who)
{
  if (status == VLB_Success) return vl::VLE_Success;
  std::string msg = std::string(who) + ": " + (c ? vlb_ctx_last_error(c) : "no engine context");
  if (c) vlb_ctx_reset_error(c);
  return context.setError((vl::ErrorCode)status, msg.c_str());
}

#define VLB_ENGINE(who)                                                                        \
  vlb_ctx* c = engine(context);                                                                \
  if (!c) return context.setError(vl::VLE_Cuda, who ": could not create the engine context")

vlb_conv_desc conv_desc(vl::Tensor const& x, vl::Tensor const& f, int sy, int sx, int pt, int pb, int pl, int pr, int dy, int dx)
{
  vlb_conv_desc d;
  d.H = (int)x.getHeight(); d.W = (int)x.getWidth(); d.C = (int)x.getDepth(); d.N = (int)x.getSize();
  d.FH = (int)f.getHeight(); d.FW = (int)f.getWidth(); d.FC = (int)f.getDepth(); d.K = (int)f.getSize();
  d.strideY = sy; d.strideX = sx;
  d.padTop = pt; d.padBottom = pb; d.padLeft = pl; d.padRight = pr;
  d.dilateY = dy; d.dilateX = dx;
  return d;
}

}  // namespace

// Releases every engine context (the test driver calls it after the gateways' own at-exit handlers).
extern "C" void vlb_functors_release(void)
{
  std::lock_guard<std::mutex> guard(g_lock);
  for (auto& kv : g_engines) if (kv.second) vlb_ctx_destroy(kv.second);
  g_engines.clear();
}

// Sets the arithmetic of every engine context created so far and of none created later (tests only).
extern "C" void vlb_functors_set_precision(int precision)
{
  std::lock_guard<std::mutex> guard(g_lock);
  for (auto& kv : g_engines) if (kv.second) vlb_ctx_set_precision(kv.second, precision);
}

extern "C" long long vlb_functors_launch_count(void)
{
  std::lock_guard<std::mutex> guard(g_lock);
  long long n = 0;
  for (auto& kv : g_engines) if (kv.second) n += vlb_ctx_launch_count(kv.second);
  return n;
}

namespace vl { namespace nn {

// ---------------------------------------------------------------- Convolution (bits/nnconv.cu:55-317)
Convolution::Convolution(Context& context, int strideY, int strideX, int padTop, int padBottom, int padLeft, int padRight,
                         int dilateY, int dilateX)
  : context(context), strideY(strideY), strideX(strideX), padTop(padTop), padBottom(padBottom), padLeft(padLeft),
    padRight(padRight), dilateY(dilateY), dilateX(dilateX)
{ }

vl::ErrorCode Convolution::forward(vl::Tensor& output, double outputMult, vl::Tensor const& input, double inputMult,
                                   vl::Tensor const& filter, vl::Tensor const& bias)
{
  if (!usable(output) || !usable(input) || !usable(filter) || !usable(bias)) return unsupported(context, "Convolution::forward");
  VLB_ENGINE("Convolution::forward");
  vlb_conv_desc d = conv_desc(input, filter, strideY, strideX, padTop, padBottom, padLeft, padRight, dilateY, dilateX);
  return done(context, c, vlb_conv_forward(c, mem(output), outputMult, mem(input), inputMult, mem(filter), mem(bias), &d),
              "Convolution::forward");
}

vl::ErrorCode Convolution::backward(vl::Tensor& derInput, vl::Tensor& derFilter, vl::Tensor& derBias, vl::Tensor const& input,
                                    vl::Tensor const& filter, vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(derFilter) || !usable(derBias) || !usable(input) || !usable(filter) || !usable(derOutput))
    return unsupported(context, "Convolution::backward");
  VLB_ENGINE("Convolution::backward");
  vlb_conv_desc d = conv_desc(input, filter, strideY, strideX, padTop, padBottom, padLeft, padRight, dilateY, dilateX);
  return done(context, c, vlb_conv_backward(c, mem(derInput), mem(derFilter), mem(derBias), mem(input), mem(filter), mem(derOutput), &d),
              "Convolution::backward");
}

// ---------------------------------------------------------------- FullyConnected (bits/nnfullyconnected.cu:40-262)
FullyConnected::FullyConnected(vl::Context& context) : context(context) { }

vl::ErrorCode FullyConnected::forward(vl::Tensor& output, vl::Tensor const& input, vl::Tensor const& filter, vl::Tensor const& bias)
{
  if (!usable(output) || !usable(input) || !usable(filter) || !usable(bias)) return unsupported(context, "FullyConnected::forward");
  VLB_ENGINE("FullyConnected::forward");
  // without filters the block is a copy plus bias; the descriptor then takes the input's own extent
  vlb_conv_desc d = conv_desc(input, filter ? filter : input, 1, 1, 0, 0, 0, 0, 1, 1);
  if (!filter) d.K = (int)input.getDepth() * (int)input.getHeight() * (int)input.getWidth();
  return done(context, c, vlb_fc_forward(c, mem(output), mem(input), mem(filter), mem(bias), &d), "FullyConnected::forward");
}

vl::ErrorCode FullyConnected::backward(vl::Tensor& derInput, vl::Tensor& derFilter, vl::Tensor& derBias, vl::Tensor const& input,
                                       vl::Tensor const& filter, vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(derFilter) || !usable(derBias) || !usable(input) || !usable(filter) || !usable(derOutput))
    return unsupported(context, "FullyConnected::backward");
  VLB_ENGINE("FullyConnected::backward");
  vlb_conv_desc d = conv_desc(input, filter ? filter : input, 1, 1, 0, 0, 0, 0, 1, 1);
  if (!filter) d.K = (int)input.getDepth() * (int)input.getHeight() * (int)input.getWidth();
  return done(context, c, vlb_fc_backward(c, mem(derInput), mem(derFilter), mem(derBias), mem(input), mem(filter), mem(derOutput), &d),
              "FullyConnected::backward");
}

// ---------------------------------------------------------------- Subsample (bits/nnsubsample.cu): the gateway's
// filter-less branch (vl_nnconv.cu:388-398, 437-447).  Not on the accelerated path.
Subsample::Subsample(vl::Context& context, int strideY, int strideX, int padTop, int padBottom, int padLeft, int padRight)
  : context(context), strideY(strideY), strideX(strideX), padTop(padTop), padBottom(padBottom), padLeft(padLeft), padRight(padRight)
{ }

vl::ErrorCode Subsample::forwardWithBias(vl::Tensor&, vl::Tensor const&, vl::Tensor const&)
{
  return context.setError(vl::VLE_Unsupported, "Subsample::forwardWithBias: convolution without filters is not covered by the B200 engine");
}

vl::ErrorCode Subsample::backwardWithBias(vl::Tensor&, vl::Tensor&, vl::Tensor const&)
{
  return context.setError(vl::VLE_Unsupported, "Subsample::backwardWithBias: convolution without filters is not covered by the B200 engine");
}

// ---------------------------------------------------------------- BatchNorm (bits/nnbnorm.cu:40-268)
BatchNorm::BatchNorm(vl::Context& context, double epsilon) : context(context), epsilon(epsilon) { }

vl::ErrorCode BatchNorm::forward(vl::Tensor& output, vl::Tensor& moment, vl::Tensor const& input, vl::Tensor const& multiplier,
                                 vl::Tensor const& bias)
{
  if (!usable(output) || !usable(moment) || !usable(input) || !usable(multiplier) || !usable(bias)) return unsupported(context, "BatchNorm::forward");
  VLB_ENGINE("BatchNorm::forward");
  return done(context, c, vlb_bnorm_forward(c, mem(output), mem(moment), mem(input), mem(multiplier), mem(bias), (int)input.getHeight(),
                                            (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), epsilon),
              "BatchNorm::forward");
}

vl::ErrorCode BatchNorm::forwardWithMoment(vl::Tensor& output, vl::Tensor const& moment, vl::Tensor const& input,
                                           vl::Tensor const& multiplier, vl::Tensor const& bias)
{
  if (!usable(output) || !usable(moment) || !usable(input) || !usable(multiplier) || !usable(bias))
    return unsupported(context, "BatchNorm::forwardWithMoment");
  VLB_ENGINE("BatchNorm::forwardWithMoment");
  return done(context, c, vlb_bnorm_forward_moment(c, mem(output), mem(moment), mem(input), mem(multiplier), mem(bias),
                                                   (int)input.getHeight(), (int)input.getWidth(), (int)input.getDepth(),
                                                   (int)input.getSize(), epsilon),
              "BatchNorm::forwardWithMoment");
}

vl::ErrorCode BatchNorm::backward(vl::Tensor& derInput, vl::Tensor& derMultiplier, vl::Tensor& derBias, vl::Tensor& moment,
                                  vl::Tensor const& input, vl::Tensor const& multiplier, vl::Tensor const& bias,
                                  vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(derMultiplier) || !usable(derBias) || !usable(moment) || !usable(input) || !usable(multiplier) ||
      !usable(bias) || !usable(derOutput))
    return unsupported(context, "BatchNorm::backward");
  VLB_ENGINE("BatchNorm::backward");
  return done(context, c, vlb_bnorm_backward(c, mem(derInput), mem(derMultiplier), mem(derBias), mem(moment), mem(input), mem(multiplier),
                                             mem(bias), mem(derOutput), (int)input.getHeight(), (int)input.getWidth(),
                                             (int)input.getDepth(), (int)input.getSize(), epsilon),
              "BatchNorm::backward");
}

vl::ErrorCode BatchNorm::backwardWithMoment(vl::Tensor& derInput, vl::Tensor& derMultiplier, vl::Tensor& derBias,
                                            vl::Tensor const& moment, vl::Tensor const& input, vl::Tensor const& multiplier,
                                            vl::Tensor const& bias, vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(derMultiplier) || !usable(derBias) || !usable(moment) || !usable(input) || !usable(multiplier) ||
      !usable(bias) || !usable(derOutput))
    return unsupported(context, "BatchNorm::backwardWithMoment");
  VLB_ENGINE("BatchNorm::backwardWithMoment");
  return done(context, c, vlb_bnorm_backward_moment(c, mem(derInput), mem(derMultiplier), mem(derBias), mem(moment), mem(input),
                                                    mem(multiplier), mem(bias), mem(derOutput), (int)input.getHeight(),
                                                    (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), epsilon),
              "BatchNorm::backwardWithMoment");
}

// ---------------------------------------------------------------- Pooling (bits/nnpooling.cu:40-206)
Pooling::Pooling(vl::Context& context, int poolHeight, int poolWidth, int strideY, int strideX, int padTop, int padBottom,
                 int padLeft, int padRight, Method method)
  : context(context), poolHeight(poolHeight), poolWidth(poolWidth), strideY(strideY), strideX(strideX), padTop(padTop),
    padBottom(padBottom), padLeft(padLeft), padRight(padRight), method(method)
{ }

static vlb_pool_desc pool_desc(Pooling const& op, vl::Tensor const& x)
{
  vlb_pool_desc d;
  d.H = (int)x.getHeight(); d.W = (int)x.getWidth(); d.C = (int)x.getDepth(); d.N = (int)x.getSize();
  d.poolH = op.poolHeight; d.poolW = op.poolWidth; d.strideY = op.strideY; d.strideX = op.strideX;
  d.padTop = op.padTop; d.padBottom = op.padBottom; d.padLeft = op.padLeft; d.padRight = op.padRight;
  d.method = op.method == Pooling::Max ? VLB_POOL_MAX : VLB_POOL_AVG;
  return d;
}

vl::ErrorCode Pooling::forward(vl::Tensor& output, vl::Tensor const& input)
{
  if (!usable(output) || !usable(input)) return unsupported(context, "Pooling::forward");
  VLB_ENGINE("Pooling::forward");
  vlb_pool_desc d = pool_desc(*this, input);
  return done(context, c, vlb_pool_forward(c, mem(output), mem(input), &d), "Pooling::forward");
}

vl::ErrorCode Pooling::backward(vl::Tensor& derInput, vl::Tensor const& input, vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(input) || !usable(derOutput)) return unsupported(context, "Pooling::backward");
  VLB_ENGINE("Pooling::backward");
  vlb_pool_desc d = pool_desc(*this, input);
  return done(context, c, vlb_pool_backward(c, mem(derInput), mem(input), mem(derOutput), &d), "Pooling::backward");
}

// ---------------------------------------------------------------- ROIPooling (bits/nnroipooling.cu:40-330)
ROIPooling::ROIPooling(vl::Context& context, std::array<int, 2> subdivisions, std::array<double, 6> transform, Method method)
  : context(context), subdivisions(subdivisions), transform(transform), method(method)
{ }

vl::ErrorCode ROIPooling::forward(vl::Tensor& output, vl::Tensor const& input, vl::Tensor const& rois)
{
  if (!usable(output) || !usable(input) || !usable(rois)) return unsupported(context, "ROIPooling::forward");
  VLB_ENGINE("ROIPooling::forward");
  int numROIs = (int)(rois.getNumElements() / 5);
  return done(context, c, vlb_roipool_forward(c, mem(output), mem(input), mem(rois), (int)input.getHeight(), (int)input.getWidth(),
                                              (int)input.getDepth(), (int)input.getSize(), numROIs, subdivisions[0], subdivisions[1],
                                              transform.data(), method == Max ? VLB_POOL_MAX : VLB_POOL_AVG),
              "ROIPooling::forward");
}

vl::ErrorCode ROIPooling::backward(vl::Tensor& derInput, vl::Tensor const& input, vl::Tensor const& rois, vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(input) || !usable(rois) || !usable(derOutput)) return unsupported(context, "ROIPooling::backward");
  VLB_ENGINE("ROIPooling::backward");
  int numROIs = (int)(rois.getNumElements() / 5);
  return done(context, c, vlb_roipool_backward(c, mem(derInput), mem(input), mem(rois), mem(derOutput), (int)input.getHeight(),
                                               (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), numROIs,
                                               subdivisions[0], subdivisions[1], transform.data(),
                                               method == Max ? VLB_POOL_MAX : VLB_POOL_AVG),
              "ROIPooling::backward");
}

// ---------------------------------------------------------------- BilinearSampler (bits/nnbilinearsampler.cu:36-120)
BilinearSampler::BilinearSampler(Context& context) : context(context) { }

vl::ErrorCode BilinearSampler::forward(vl::Tensor& output, vl::Tensor const& input, vl::Tensor const& grid)
{
  if (!usable(output) || !usable(input) || !usable(grid)) return unsupported(context, "BilinearSampler::forward");
  VLB_ENGINE("BilinearSampler::forward");
  // grid: 2 x Ho x Wo x Ng
  return done(context, c, vlb_sampler_forward(c, mem(output), mem(input), mem(grid), (int)input.getHeight(), (int)input.getWidth(),
                                              (int)input.getDepth(), (int)input.getSize(), (int)grid.getWidth(), (int)grid.getDepth(),
                                              (int)grid.getSize()),
              "BilinearSampler::forward");
}

vl::ErrorCode BilinearSampler::backward(vl::Tensor& derInput, vl::Tensor& derGrid, vl::Tensor const& input, vl::Tensor const& grid,
                                        vl::Tensor const& derOutput)
{
  if (!usable(derInput) || !usable(derGrid) || !usable(input) || !usable(grid) || !usable(derOutput))
    return unsupported(context, "BilinearSampler::backward");
  VLB_ENGINE("BilinearSampler::backward");
  return done(context, c, vlb_sampler_backward(c, mem(derInput), mem(derGrid), mem(input), mem(grid), mem(derOutput), (int)input.getHeight(),
                                               (int)input.getWidth(), (int)input.getDepth(), (int)input.getSize(), (int)grid.getWidth(),
                                               (int)grid.getDepth(), (int)grid.getSize()),
              "BilinearSampler::backward");
}

} }  // namespace vl::nn
