// Drives the engine through the reference's C++ operator interface (vl::nn::Convolution,
// BatchNorm, Pooling, ROIPooling, BilinearSampler, Bias, FullyConnected on vl::Tensor views, as the
// MEX gateways do, reference matlab/src/vl_nnconv.cu:449-464) and checks every result against the
// CPU checker (oracle/libmcn_oracle.so, loaded at run time) on identical seeded inputs.
// Build and run: see tests/test_cpp_classes.py.
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "vlb/nnbias.hpp"
#include "vlb/nnbilinearsampler.hpp"
#include "vlb/nnbnorm.hpp"
#include "vlb/nnconv.hpp"
#include "vlb/nnfullyconnected.hpp"
#include "vlb/nnpooling.hpp"
#include "vlb/nnroipooling.hpp"

static unsigned long long g_state = 88172645463325252ULL;
static double urand() { g_state ^= g_state << 13; g_state ^= g_state >> 7; g_state ^= g_state << 17; return (g_state >> 11) * (1.0 / 9007199254740992.0); }
static float nrand() { double u = urand() + 1e-12, v = urand(); return (float)(std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v)); }

struct Buf {
  std::vector<float> h;
  float* d;
  vl::TensorShape shape;
  Buf(size_t a, size_t b, size_t c, size_t n, int fill = 1) : h(a * b * c * n), d(NULL), shape(a, b, c, n)
  {
    for (size_t i = 0; i < h.size(); ++i) h[i] = fill == 1 ? nrand() : 0.f;
    cudaMalloc((void**)&d, sizeof(float) * (h.size() ? h.size() : 1));
    up();
  }
  ~Buf() { cudaFree(d); }
  void up() { cudaMemcpy(d, h.data(), sizeof(float) * h.size(), cudaMemcpyHostToDevice); }
  std::vector<float> down() const { std::vector<float> o(h.size()); cudaMemcpy(o.data(), d, sizeof(float) * o.size(), cudaMemcpyDeviceToHost); return o; }
  vl::Tensor t() { return vl::Tensor(shape, vl::VLDT_Float, vl::VLDT_GPU, d, sizeof(float) * h.size()); }
};

static double relL2(std::vector<float> const& a, std::vector<float> const& b)
{
  double num = 0, den = 0;
  for (size_t i = 0; i < a.size(); ++i) { double d = (double)a[i] - b[i]; num += d * d; den += (double)b[i] * b[i]; }
  return std::sqrt(num / (den > 1e-60 ? den : 1e-60));
}
static bool same(std::vector<float> const& a, std::vector<float> const& b)
{
  for (size_t i = 0; i < a.size(); ++i) if (!(a[i] == b[i])) return false;
  return true;
}

static int g_fail = 0;
static void report(char const* what, bool ok, double err)
{
  std::printf("%-34s %s  (%.3g)\n", what, ok ? "ok" : "FAILED", err);
  if (!ok) ++g_fail;
}

template <typename F> static F sym(void* lib, char const* name)
{
  F f = (F)dlsym(lib, name);
  if (!f) { std::fprintf(stderr, "missing symbol %s\n", name); std::exit(2); }
  return f;
}

int main(int argc, char** argv)
{
  if (argc < 2) { std::fprintf(stderr, "usage: %s path/to/libmcn_oracle.so\n", argv[0]); return 2; }
  void* lib = dlopen(argv[1], RTLD_NOW);
  if (!lib) { std::fprintf(stderr, "cannot load %s: %s\n", argv[1], dlerror()); return 2; }
  typedef int (*conv_bwd_t)(int, void*, void*, void*, void const*, void const*, void const*, int const*, int const*);
  typedef int (*conv_fwd_t)(int, void*, void const*, void const*, void const*, int const*, int const*);
  typedef int (*bn_bwd_t)(int, void*, void*, void*, void*, void const*, void const*, void const*, void const*, int, int, int, int, double);
  typedef int (*pool_t)(int, void*, void const*, void const*, int, int, int, int, int const*);
  typedef int (*poolf_t)(int, void*, void const*, int, int, int, int, int const*);
  typedef int (*roi_bwd_t)(int, void*, void const*, void const*, void const*, int, int, int, int, int, int, int, double const*, int);
  typedef int (*smp_bwd_t)(int, void*, void*, void const*, void const*, void const*, int, int, int, int, int, int, int);
  conv_fwd_t ref_conv_fwd = sym<conv_fwd_t>(lib, "mcno_conv_forward");
  conv_bwd_t ref_conv_bwd = sym<conv_bwd_t>(lib, "mcno_conv_backward");
  bn_bwd_t ref_bn_bwd = sym<bn_bwd_t>(lib, "mcno_bnorm_backward");
  poolf_t ref_pool_fwd = sym<poolf_t>(lib, "mcno_pool_forward");
  pool_t ref_pool_bwd = sym<pool_t>(lib, "mcno_pool_backward");
  roi_bwd_t ref_roi_bwd = sym<roi_bwd_t>(lib, "mcno_roipool_backward");
  smp_bwd_t ref_smp_bwd = sym<smp_bwd_t>(lib, "mcno_sampler_backward");

  vl::Context context;                       // one per process, like the MEX-file global (vl_nnconv.cu:64)
  if (!context.get()) { std::fprintf(stderr, "no engine context: %s\n", context.getLastErrorMessage().c_str()); return 3; }

  {  // ---- convolution 3x3 pad 1 with bias, forward and backward
    int H = 16, W = 12, C = 8, N = 3, K = 16;
    Buf x(H, W, C, N), f(3, 3, C, K), b(1, 1, 1, K), y(H, W, K, N, 0), dy(H, W, K, N), dx(H, W, C, N, 0), df(3, 3, C, K, 0), db(1, 1, 1, K, 0);
    vl::nn::Convolution op(context, 1, 1, 1, 1, 1, 1, 1, 1);
    vl::Tensor ty = y.t(), tdx = dx.t(), tdf = df.t(), tdb = db.t();
    vl::ErrorCode e1 = op.forward(ty, 0, x.t(), 1, f.t(), b.t());
    vl::ErrorCode e2 = op.backward(tdx, tdf, tdb, x.t(), f.t(), dy.t());
    int shape[8] = {H, W, C, N, 3, 3, C, K}, prm[8] = {1, 1, 1, 1, 1, 1, 1, 1};
    std::vector<float> ry(y.h.size()), rdx(dx.h.size()), rdf(df.h.size()), rdb(K);
    ref_conv_fwd(0, ry.data(), x.h.data(), f.h.data(), b.h.data(), shape, prm);
    ref_conv_bwd(0, rdx.data(), rdf.data(), rdb.data(), x.h.data(), f.h.data(), dy.h.data(), shape, prm);
    report("Convolution::forward", e1 == vl::VLE_Success && relL2(y.down(), ry) < 1e-5, relL2(y.down(), ry));
    report("Convolution::backward derInput", e2 == vl::VLE_Success && relL2(dx.down(), rdx) < 1e-5, relL2(dx.down(), rdx));
    report("Convolution::backward derFilter", relL2(df.down(), rdf) < 1e-5, relL2(df.down(), rdf));
    report("Convolution::backward derBias", relL2(db.down(), rdb) < 1e-5, relL2(db.down(), rdb));
    // a null derInput is skipped, the others are unchanged (nnconv.cu:190-212)
    vl::Tensor none;
    Buf df2(3, 3, C, K, 0);
    vl::Tensor tdf2 = df2.t();
    vl::ErrorCode e3 = op.backward(none, tdf2, none, x.t(), f.t(), dy.t());
    report("Convolution::backward null outputs", e3 == vl::VLE_Success && same(df2.down(), df.down()), 0);
    // CPU tensors are refused, not computed
    vl::Tensor cpu(x.shape, vl::VLDT_Float, vl::VLDT_CPU, x.h.data(), 0);
    report("Convolution refuses CPU tensors", op.forward(ty, 0, cpu, 1, f.t(), b.t()) == vl::VLE_Unsupported, 0);
    context.resetLastError();
  }
  {  // ---- fully connected (output 1x1)
    int H = 4, W = 4, C = 6, N = 5, K = 9;
    Buf x(H, W, C, N), f(H, W, C, K), b(1, 1, 1, K), y(1, 1, K, N, 0);
    vl::nn::FullyConnected op(context);
    vl::Tensor ty = y.t();
    vl::ErrorCode e = op.forward(ty, x.t(), f.t(), b.t());
    int shape[8] = {H, W, C, N, H, W, C, K}, prm[8] = {1, 1, 0, 0, 0, 0, 1, 1};
    std::vector<float> ry(y.h.size());
    ref_conv_fwd(0, ry.data(), x.h.data(), f.h.data(), b.h.data(), shape, prm);
    report("FullyConnected::forward", e == vl::VLE_Success && relL2(y.down(), ry) < 1e-5, relL2(y.down(), ry));
  }
  {  // ---- batch normalisation backward, moments returned
    int H = 8, W = 4, C = 5, N = 3;
    Buf x(H, W, C, N), g(C, 1, 1, 1), b(C, 1, 1, 1), dy(H, W, C, N), dx(H, W, C, N, 0), dg(C, 1, 1, 1, 0), db(C, 1, 1, 1, 0), mom(C, 2, 1, 1, 0);
    vl::nn::BatchNorm op(context, 1e-4);
    vl::Tensor tdx = dx.t(), tdg = dg.t(), tdb = db.t(), tm = mom.t();
    vl::ErrorCode e = op.backward(tdx, tdg, tdb, tm, x.t(), g.t(), b.t(), dy.t());
    std::vector<float> rdx(dx.h.size()), rdg(C), rdb(C), rm(2 * C);
    ref_bn_bwd(0, rdx.data(), rdg.data(), rdb.data(), rm.data(), x.h.data(), g.h.data(), b.h.data(), dy.h.data(), H, W, C, N, 1e-4);
    report("BatchNorm::backward derInput", e == vl::VLE_Success && relL2(dx.down(), rdx) < 1e-5, relL2(dx.down(), rdx));
    report("BatchNorm::backward derMultiplier", relL2(dg.down(), rdg) < 1e-5, relL2(dg.down(), rdg));
    report("BatchNorm::backward moment", relL2(mom.down(), rm) < 1e-5, relL2(mom.down(), rm));
  }
  {  // ---- pooling, bit-exact
    int H = 12, W = 10, C = 3, N = 2;
    Buf x(H, W, C, N);
    int prm[9] = {3, 3, 2, 2, 0, 1, 0, 1, 0};
    int Ho = (H + 1 - 3) / 2 + 1, Wo = (W + 1 - 3) / 2 + 1;
    Buf y(Ho, Wo, C, N, 0), dy(Ho, Wo, C, N), dx(H, W, C, N, 0);
    vl::nn::Pooling op(context, 3, 3, 2, 2, 0, 1, 0, 1, vl::nn::Pooling::Max);
    vl::Tensor ty = y.t(), tdx = dx.t();
    vl::ErrorCode e1 = op.forward(ty, x.t()), e2 = op.backward(tdx, x.t(), dy.t());
    std::vector<float> ry(y.h.size()), rdx(dx.h.size());
    ref_pool_fwd(0, ry.data(), x.h.data(), H, W, C, N, prm);
    ref_pool_bwd(0, rdx.data(), x.h.data(), dy.h.data(), H, W, C, N, prm);
    report("Pooling::forward (bit-exact)", e1 == vl::VLE_Success && same(y.down(), ry), 0);
    report("Pooling::backward (bit-exact)", e2 == vl::VLE_Success && same(dx.down(), rdx), 0);
  }
  {  // ---- ROI pooling backward with integer-valued gradient: exact under atomics
    int H = 15, W = 14, C = 3, N = 2, K = 4;
    Buf x(H, W, C, N), rois(5, K, 1, 1, 0), dy(3, 2, C, K), dx(H, W, C, N, 0);
    float r[20] = {1, 1, 1, 14, 15, 2, 3.4f, 2.2f, 7.7f, 9.1f, 1, -3, -2, 20, 30, 2, 5, 5, 5, 5};
    for (int i = 0; i < 20; ++i) rois.h[i] = r[i];
    rois.up();
    for (size_t i = 0; i < dy.h.size(); ++i) dy.h[i] = (float)((int)(urand() * 9) - 4);
    dy.up();
    std::array<int, 2> sub = {{3, 2}};
    std::array<double, 6> tf = {{1, 0, 0, 1, 0, 0}};
    vl::nn::ROIPooling op(context, sub, tf, vl::nn::ROIPooling::Max);
    vl::Tensor tdx = dx.t();
    vl::ErrorCode e = op.backward(tdx, x.t(), rois.t(), dy.t());
    std::vector<float> rdx(dx.h.size());
    ref_roi_bwd(0, rdx.data(), x.h.data(), rois.h.data(), dy.h.data(), H, W, C, N, K, 3, 2, tf.data(), 0);
    report("ROIPooling::backward (bit-exact)", e == vl::VLE_Success && same(dx.down(), rdx), 0);
  }
  {  // ---- bilinear sampler backward
    int H = 8, W = 7, C = 3, N = 2, Ho = 5, Wo = 6, Ng = 4;
    Buf x(H, W, C, N), grid(2, Ho, Wo, Ng, 0), dy(Ho, Wo, C, Ng), dx(H, W, C, N, 0), dgrid(2, Ho, Wo, Ng, 0);
    for (size_t i = 0; i < grid.h.size(); ++i) grid.h[i] = (float)(urand() * 2.2 - 1.1);
    grid.up();
    vl::nn::BilinearSampler op(context);
    vl::Tensor tdx = dx.t(), tdg = dgrid.t();
    vl::ErrorCode e = op.backward(tdx, tdg, x.t(), grid.t(), dy.t());
    std::vector<float> rdx(dx.h.size()), rdg(dgrid.h.size());
    ref_smp_bwd(0, rdx.data(), rdg.data(), x.h.data(), grid.h.data(), dy.h.data(), H, W, C, N, Ho, Wo, Ng);
    report("BilinearSampler::backward derInput", e == vl::VLE_Success && relL2(dx.down(), rdx) < 1e-6, relL2(dx.down(), rdx));
    report("BilinearSampler::backward derGrid", same(dgrid.down(), rdg), 0);
  }
  cudaDeviceSynchronize();
  std::printf("%s\n", g_fail ? "SOME CHECKS FAILED" : "all checks passed");
  return g_fail ? 1 : 0;
}
