/* vlb.h -- C ABI of the B200 engine behind MatConvNet's operator classes.
 *
 * Every entry point takes DEVICE pointers to single-precision tensors in
 * MATLAB order H x W x C x N (H fastest; element (h,w,c,n) at
 * h + H*(w + W*(c + C*n)), reference matlab/src/bits/data.cu:498-505) and
 * enqueues hand-written sm_100a kernels on the context's stream without
 * synchronising, as the reference's GPU functors do.  There is no CPU
 * fallback: host pointers are not accepted and a build without the CUDA
 * kernels does not exist.
 *
 * Return value: the numeric value of vl::ErrorCode (reference
 * matlab/src/bits/data.hpp:38-52); 0 = VLE_Success.  On failure
 * vlb_ctx_last_error() holds a message chain like the reference's
 * Context::getLastErrorMessage() (bits/data.cu:332-377).
 *
 * A NULL output pointer means "null tensor: skip this output", as the
 * reference's `if (derInput)` tests do (bits/nnconv.cu:190-212).
 */
#ifndef VLB_H
#define VLB_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* vl::ErrorCode, bits/data.hpp:38-52 (spelling of OutOfGPUMemeory kept). */
enum {
  VLB_Success = 0, VLB_Unsupported, VLB_Cuda, VLB_Cudnn, VLB_Cublas, VLB_OutOfMemory,
  VLB_OutOfGPUMemeory, VLB_IllegalArgument, VLB_Unknown, VLB_Timeout, VLB_NoData,
  VLB_IllegalMessage, VLB_Interrupted
};

/* Arithmetic of the convolution / fully-connected contractions. */
enum {
  VLB_PRECISION_3XTF32 = 0, /* tcgen05 kind::tf32, hi/lo split, 3 MMAs per product: fp32-faithful (default) */
  VLB_PRECISION_TF32 = 1,   /* tcgen05 kind::tf32, single pass: fast path, about 1e-3 relative error */
  VLB_PRECISION_FP32 = 2    /* CUDA-core FMA implicit GEMM: exact fp32 products, slow; also the path for
                               strides / dilations / groups the tensor-core kernels do not cover */
};

/* ---- context: replaces vl::Context (bits/data.hpp:150-179) and the stream part of
 *      vl::CudaHelper (bits/datacu.hpp:60-158; setStream bits/datacu.cu:70-93) ---- */
typedef struct vlb_ctx vlb_ctx;

int vlb_ctx_create(vlb_ctx** out);               /* binds to the current CUDA device */
int vlb_ctx_destroy(vlb_ctx* ctx);               /* frees scratch; Context::clear, bits/data.cu:288-301 */
int vlb_ctx_set_stream(vlb_ctx* ctx, void* cuda_stream);  /* CudaHelper::setStream; NULL = legacy default stream */
void* vlb_ctx_get_stream(vlb_ctx* ctx);
int vlb_ctx_set_precision(vlb_ctx* ctx, int precision);
int vlb_ctx_get_precision(vlb_ctx* ctx);
char const* vlb_ctx_last_error(vlb_ctx* ctx);    /* Context::getLastErrorMessage, bits/data.cu:372-377 */
void vlb_ctx_reset_error(vlb_ctx* ctx);          /* Context::resetLastError */
int vlb_ctx_reserve_workspace(vlb_ctx* ctx, size_t bytes); /* grow-only scratch, Context::getWorkspace bits/data.cu:395-404 */
size_t vlb_ctx_workspace_bytes(vlb_ctx* ctx);
int vlb_ctx_clear_workspace(vlb_ctx* ctx);       /* Context::clearWorkspace, bits/data.cu:406-410 */
long long vlb_ctx_launch_count(vlb_ctx* ctx);    /* kernels enqueued through this context so far */
/* Synchronises the stream and reads the status word that the tensor-core kernels set when one of
 * their bounded pipeline waits expires (0 = none did).  Returns VLE_Timeout, as the reference's own
 * waits do (matlab/src/vl_tmove.cu:1344-1359), when the word is non-zero, and clears it; VLE_IllegalArgument when the word
 * says that vlb_softmaxloss_* met a class label above the number of classes. */
int vlb_ctx_device_status(vlb_ctx* ctx, int* status);
/* The bound on a single pipeline wait of the tensor-core kernels, in SM clock cycles; 0 restores the default (2e8, about a
 * tenth of a second).  Applies to the current device.  Exists so that a test can make a wait run out quickly. */
int vlb_ctx_set_wait_limit(vlb_ctx* ctx, long long cycles);
/* Test switches (0 = none).  Bit 0: the filter-tile loader of the tensor-memory convolution kernel stays idle, so every
 * wait behind it runs out: the kernel records its status word, releases its tensor memory and returns
 * (vlb_ctx_device_status then gives VLE_Timeout; the output of that call is undefined).  Nothing traps or spins.
 * Bit 1: the tensor-memory convolution kernel gathers its input windows with per-thread loads even where it could have
 * them delivered by tensor-map copies; the two routes give the same result bit for bit, which is what a test compares.
 * Bit 2: the filter gradient of a convolution takes the kernel with both operands in shared memory even where the
 * tensor-memory kernel applies (the two differ in the order of the sums; a test checks both against the CPU checker).
 * Bit 3: the tensor-memory convolution kernel keeps the running sum of an output tile in shared memory even for the tile
 * widths (64 and 128 columns) whose sum fits the registers of its drain warps; same additions in the same order, so the
 * results are equal, which is what a test compares. */
int vlb_ctx_set_test_switch(vlb_ctx* ctx, int switches);
/* Measurement aid: between begin and end every tensor-core contraction (with the launches that prepare its operands
 * and finish its result) is bracketed by CUDA events on the context's stream.  end synchronises and returns the summed kernel time, the summed
 * algorithmic flops (2*M*N*K of each contraction, counted once whatever the arithmetic mode) and the
 * number of launches.  (The reference times whole layers with tic/toc, matlab/simplenn/vl_simplenn.m:297,397.) */
int vlb_ctx_profile_begin(vlb_ctx* ctx);
int vlb_ctx_profile_end(vlb_ctx* ctx, double* ms, double* flops, long long* launches);
/* After vlb_ctx_profile_end: the same three sums for one kind of contraction -- 0 convolution forward, 1 convolution data
 * gradient, 2 convolution filter gradient (its operand tile images, bias gradient and split-reduction pass included),
 * 3 fully connected (all three passes). */
int vlb_ctx_profile_kind(vlb_ctx* ctx, int kind, double* ms, double* flops, long long* count);
char const* vlb_error_message(int code);         /* vl::getErrorMessage, bits/data.cu:83-100 (all 13 codes named) */
int vlb_version(void);

/* ---- convolution: vl::nn::Convolution (bits/nnconv.hpp:23-52) -------------------------------- */
typedef struct {
  int H, W, C, N;            /* input  H x W x C x N */
  int FH, FW, FC, K;         /* filter FH x FW x FC x K; groups = C / FC (bits/nnconv.cu:89-90) */
  int strideY, strideX;
  int padTop, padBottom, padLeft, padRight;
  int dilateY, dilateX;
} vlb_conv_desc;

/* Output extent (matlab/src/vl_nnconv.cu:324-331, bits/impl/im2row_cpu.cpp:70-73). */
int vlb_conv_output_shape(vlb_conv_desc const* d, int* Ho, int* Wo);

/* Convolution::forward (bits/nnconv.cu:71-157): Y = outMult*Y + inMult*conv(X,F) + b.
 * b may be NULL.  Y is read only when outMult != 0. */
int vlb_conv_forward(vlb_ctx* ctx, float* Y, double outMult, float const* X, double inMult,
                     float const* F, float const* b, vlb_conv_desc const* d);

/* Forward convolution followed by ReLU in one call: Y = max(conv(X,F) + b, 0).  No counterpart among the reference's
 * operator classes: vl_simplenn runs vl_nnrelu as a layer of its own (matlab/simplenn/vl_simplenn.m:334-336), and when it
 * has dropped the ReLU's input to save memory (:386) it takes the mask from the ReLU's output (:448-455) -- which is what a
 * caller of this entry point does in the backward pass, vlb_relu_backward(dX, Y, dY).  The result is bit-identical to
 * vlb_conv_forward followed by vlb_relu_forward. */
int vlb_conv_relu_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b,
                          vlb_conv_desc const* d);

/* Convolution::backward (bits/nnconv.cu:163-317).  dX, dF, db are overwritten; any may be NULL. */
int vlb_conv_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X,
                      float const* F, float const* dY, vlb_conv_desc const* d);

/* Backward convolution and the ReLU before it in one call, for a convolution whose input X is the output of a ReLU:
 * dF, db as vlb_conv_backward; dX is the derivative with respect to the ReLU's input, conv_backward's dX zeroed where X is
 * not positive.  vl_simplenn runs the two as separate layers (matlab/simplenn/vl_simplenn.m:410-421 and :448-455, the
 * mask taken from the ReLU's output when its input was dropped); here the data-gradient kernel applies the mask as it
 * stores.  Bit-identical to vlb_conv_backward followed by vlb_relu_backward(dX, X, dX).  Accepts fully connected shapes. */
int vlb_relu_conv_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X,
                           float const* F, float const* dY, vlb_conv_desc const* d);

/* ---- convolution transpose: vl::nn::ConvolutionTranspose (bits/nnconv.hpp:54-80) -----------------
 * Y (Ho x Wo x FD*numGroups x N) from X (H x W x C x N) and F (FH x FW x FD x FN), FN == C
 * (matlab/src/vl_nnconvt.cu:262-301). */
typedef struct {
  int H, W, C, N;            /* input */
  int FH, FW, FD, FN;        /* filter bank: FD output channels per group, FN == C */
  int upsampleY, upsampleX;
  int cropTop, cropBottom, cropLeft, cropRight;
  int numGroups;
} vlb_convt_desc;
/* Ho = (H-1)*upsampleY - (cropTop+cropBottom) + FH, likewise Wo (matlab/src/vl_nnconvt.cu:293-296). */
int vlb_convt_output_shape(vlb_convt_desc const* d, int* Ho, int* Wo);
/* ConvolutionTranspose::forward (bits/nnconv.cu:323-374): the data gradient of the convolution with stride = upsample,
 * pad = crop, then the bias.  b may be NULL. */
int vlb_convt_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b,
                      vlb_convt_desc const* d);
/* ConvolutionTranspose::backward (bits/nnconv.cu:380-421): dX = that convolution's forward pass of dY, dF = its filter
 * gradient with data and output derivative exchanged, db = sum of dY.  Any of dX, dF, db may be NULL. */
int vlb_convt_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                       float const* dY, vlb_convt_desc const* d);

/* ---- fully connected: vl::nn::FullyConnected (bits/nnfullyconnected.hpp:20-37) ---------------
 * The gateway routes here when the output is 1x1, stride 1, no pad, no dilation, one group
 * (matlab/src/vl_nnconv.cu:351-361).  d->FH==d->H, d->FW==d->W, d->FC==d->C.  F == NULL copies. */
int vlb_fc_forward(vlb_ctx* ctx, float* Y, float const* X, float const* F, float const* b,
                   vlb_conv_desc const* d);
int vlb_fc_backward(vlb_ctx* ctx, float* dX, float* dF, float* db, float const* X, float const* F,
                    float const* dY, vlb_conv_desc const* d);

/* ---- bias: vl::nn::Bias (bits/nnbias.hpp:20-35) ---------------------------------------------- */
/* Bias::forward (bits/nnbias.cu:37-96): with b != NULL and bMult != 0, Y = yMult*Y + bMult*b
 * (broadcast over H,W,N); otherwise Y = 0 whatever yMult is; then Y += xMult*X if X != NULL. */
int vlb_bias_forward(vlb_ctx* ctx, float* Y, double yMult, float const* X, double xMult,
                     float const* b, double bMult, int H, int W, int K, int N);
/* Bias::backward (bits/nnbias.cu:102-175): db = dbMult*db + bMult*sum_{h,w,n} dY;
 * dX = dXMult*dX + xMult*dY.  A multiplier of exactly 0 means "overwrite" (the old value is not
 * read), where the reference would multiply uninitialised memory by zero. */
int vlb_bias_backward(vlb_ctx* ctx, float* dX, double dXMult, float* db, double dbMult, double xMult,
                      double bMult, float const* dY, int H, int W, int K, int N);

/* ---- batch normalisation: vl::nn::BatchNorm (bits/nnbnorm.hpp:22-59) --------------------------
 * moments = 2*C floats [mean(0..C-1), sigma(C..2C-1)], sigma = sqrt(var + eps)
 * (matlab/src/vl_nnbnorm.cu:210-213, bits/nnbnorm.cu:65-70). */
int vlb_bnorm_forward(vlb_ctx* ctx, float* Y, float* moments /* may be NULL */, float const* X,
                      float const* g, float const* b, int H, int W, int C, int N, double eps);
/* Training-mode batch normalisation followed by ReLU in one call: Y = max(bnorm(X), 0), moments as vlb_bnorm_forward.  No
 * counterpart among the reference's operator classes; the wrappers short-circuit a ReLU after another layer in the same way
 * (matlab/+dagnn/ReLU.m:21-63).  Bit-identical to vlb_bnorm_forward followed by vlb_relu_forward; in the backward pass the
 * ReLU takes its mask from Y (vlb_relu_backward(dX, Y, dY)), the batch normalisation needs only X. */
int vlb_bnorm_relu_forward(vlb_ctx* ctx, float* Y, float* moments /* may be NULL */, float const* X, float const* g,
                           float const* b, int H, int W, int C, int N, double eps);
int vlb_bnorm_forward_moment(vlb_ctx* ctx, float* Y, float const* moments, float const* X,
                             float const* g, float const* b, int H, int W, int C, int N, double eps);
int vlb_bnorm_backward(vlb_ctx* ctx, float* dX, float* dG, float* dB, float* moments /* may be NULL */,
                       float const* X, float const* g, float const* b, float const* dY,
                       int H, int W, int C, int N, double eps);
int vlb_bnorm_backward_moment(vlb_ctx* ctx, float* dX, float* dG, float* dB, float const* moments,
                              float const* X, float const* g, float const* b, float const* dY,
                              int H, int W, int C, int N, double eps);

/* Batch-norm backward (moments computed from the batch, like vlb_bnorm_backward) for callers that may
 * not allocate device memory: a host whose own allocator owns the whole GPU, or a loop that cannot
 * afford the device-wide synchronisation of cudaMalloc.  It has no counterpart in the reference.
 * It needs no vlb_ctx and calls no cudaMalloc, cudaFree or other allocating routine: the per-channel
 * scratch (moments when `moments` is NULL, and the dx coefficients) is a fixed 96 KB array inside the
 * library image, which every GPU that loads the library holds until the process exits.
 *   - C may be at most 4096 channels; more is refused with VLE_IllegalArgument and a message.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call before any stream capture begins, and from one host thread per device.
 *   - All calls on a device share the one array, so two calls whose kernels overlap on the GPU (different
 *     streams, no dependency) race on it; serialise them.  Nothing in it needs clearing between calls:
 *     each call rewrites the entries of channels [0, C) before reading them.
 * cudaStream: the stream to enqueue on (NULL = default stream).  errbuf/errlen: optional buffer that
 * receives a message when the return value is not 0.  Tensors and results are those of vlb_bnorm_backward. */
int vlb_bnorm_backward_noalloc(void* cudaStream, float* dX, float* dG, float* dB, float* moments /* may be NULL */,
                               float const* X, float const* g, float const* dY, int H, int W, int C, int N,
                               double eps, char* errbuf, size_t errlen);

/* ---- pooling: vl::nn::Pooling (bits/nnpooling.hpp:21-49) ------------------------------------- */
enum { VLB_POOL_MAX = 0, VLB_POOL_AVG = 1 };
typedef struct {
  int H, W, C, N;
  int poolH, poolW, strideY, strideX;
  int padTop, padBottom, padLeft, padRight;
  int method;
} vlb_pool_desc;
int vlb_pool_output_shape(vlb_pool_desc const* d, int* Ho, int* Wo); /* matlab/src/vl_nnpool.cu:240-247 */
int vlb_pool_forward(vlb_ctx* ctx, float* Y, float const* X, vlb_pool_desc const* d);
/* Pooling::backward (bits/nnpooling.cu:170-214).  The reference accumulates into a dX the gateway
 * has zero-filled (matlab/src/vl_nnpool.cu:255-259); here dX is OVERWRITTEN with "0 + contributions",
 * contributions added in the reference's window order, so the result is the same bit for bit and the
 * caller's zero fill is harmless but unnecessary. */
int vlb_pool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, vlb_pool_desc const* d);
/* Pooling backward and the ReLU before it in one call, for a pooling layer whose input X is the output of a ReLU: dX is
 * the derivative with respect to the ReLU's input, pool_backward's dX zeroed where X is not positive (the sequence
 * matlab/simplenn/vl_simplenn.m:423-428 then :448-455).  Bit-identical to vlb_pool_backward followed by
 * vlb_relu_backward(dX, X, dX). */
int vlb_relu_pool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, vlb_pool_desc const* d);

/* ---- ROI pooling: vl::nn::ROIPooling (bits/nnroipooling.hpp:23-45) ----------------------------
 * rois: 5 x numROIs floats [image(1-based); u1; v1; u2; v2]; transform: 6 doubles, 2x3 column-major.
 * Y / dY: S0 x S1 x C x numROIs.  dX is overwritten, as after the reference CPU's memset (bits/nnroipooling.cu:237).
 * Backward gathers: every element of dX adds the derivatives of the bins routed to it in the CPU loop's order (ROI, bin
 * column, bin row), so the result is the CPU's bit for bit and the same from run to run; no atomics.  (Maps of 65535
 * pixels or more, or too large for a shared-memory slab, fall back to a zero fill and an atomic scatter.) */
int vlb_roipool_forward(vlb_ctx* ctx, float* Y, float const* X, float const* rois, int H, int W, int C,
                        int N, int numROIs, int S0, int S1, double const* transform, int method);
int vlb_roipool_backward(vlb_ctx* ctx, float* dX, float const* X, float const* rois, float const* dY,
                         int H, int W, int C, int N, int numROIs, int S0, int S1,
                         double const* transform, int method);
/* Bin geometry alone (bits/nnroipooling.cu:120-165), for checking it bit for bit:
 * bounds[4*(ph + S0*(pw + S1*roi)) + {0,1,2,3}] = hstart,hend,wstart,wend; images[roi] = 0-based image. */
int vlb_roipool_bounds(vlb_ctx* ctx, int* bounds, int* images, float const* rois, int H, int W, int N,
                       int numROIs, int S0, int S1, double const* transform);

/* ---- bilinear sampler: vl::nn::BilinearSampler (bits/nnbilinearsampler.hpp:21-36) -------------
 * X: H x W x C x N; grid: 2 x Ho x Wo x Ng (y first), Ng a multiple of N; Y, dY: Ho x Wo x C x Ng.
 * dX and dGrid are overwritten (either may be NULL).  dGrid is the CPU's bit for bit.  dX is a gather when the planes fit
 * the shared memory (H*W and Ho*Wo up to a few thousand each): every input pixel adds its contributions in the CPU
 * loop's order, bit for bit the CPU's result and run-to-run identical; only when one input pixel receives more than 48
 * contributions from one grid, or for larger planes, dX is accumulated with float atomics instead. */
int vlb_sampler_forward(vlb_ctx* ctx, float* Y, float const* X, float const* grid, int H, int W, int C,
                        int N, int Ho, int Wo, int Ng);
int vlb_sampler_backward(vlb_ctx* ctx, float* dX, float* dGrid, float const* X, float const* grid,
                         float const* dY, int H, int W, int C, int N, int Ho, int Wo, int Ng);

/* ---- blocks the reference implements in MATLAB, needed to run whole networks on the device ---- */
/* matlab/vl_nnrelu.m:43-48 (leak 0). */
int vlb_relu_forward(vlb_ctx* ctx, float* Y, float const* X, size_t n);
int vlb_relu_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, size_t n);
/* matlab/vl_nnsoftmaxloss.m:56-84, one 1-based class label (as float) per image; label 0 skips the image (its loss term
 * and derivative are zero, :55-67).  A label above C (an indexing error in the reference) is skipped likewise and
 * reported by vlb_ctx_device_status.  loss: one float on the device. */
int vlb_softmaxloss_forward(vlb_ctx* ctx, float* loss, float const* X, float const* labels,
                            int H, int W, int C, int N);
int vlb_softmaxloss_backward(vlb_ctx* ctx, float* dX, float const* X, float const* labels, double dzdy,
                             int H, int W, int C, int N);
/* matlab/+dagnn/Sum.m:11-23: Y = A + B (Y may alias A). */
int vlb_sum(vlb_ctx* ctx, float* Y, float const* A, float const* B, size_t n);
/* x *= alpha: the 1/numWorkers scaling of an all-reduced gradient (examples/cnn_train.m:482-483). */
int vlb_scale(vlb_ctx* ctx, float* x, double alpha, size_t n);
/* vl_taccum (matlab/vl_taccum.m, matlab/src/vl_taccummex.cu:50-76): Y = alpha*A + beta*B, computed as the reference does
 * (A scaled, then an axpy of B).  Y may alias A. */
int vlb_taccum(vlb_ctx* ctx, float* Y, double alpha, float const* A, double beta, float const* B, size_t n);
/* The trainer's SGD step on one parameter tensor after the gradient exchange (examples/cnn_train.m:478-499), its four
 * vl_taccum passes fused into one: g = gradMult*G + decay*W (gradMult = 1/numWorkers); M = momentum*M - g;
 * delta = nesterov ? momentum*M - g : M; W += lr*delta.  W (parameters) and M (momentum state) are updated in place, G
 * is only read.  Bit-identical to the four vlb_taccum calls. */
int vlb_sgd_update(vlb_ctx* ctx, float* W, float* M, float const* G, size_t n, double gradMult, double decay,
                   double momentum, double lr, int nesterov);

/* ---- blocks of the reference's other ImageNet models (AlexNet, VGG-F/M/S; examples/imagenet/cnn_imagenet_init.m) ---- */
/* Cross-channel local response normalisation, vl::nn::LRN (bits/nnnormalize.hpp:20-44; matlab/vl_nnnormalize.m, PARAM =
 * [normDepth kappa alpha beta]): y_t = x_t * (kappa + alpha * sum of x_q^2 over q in [t - m1, t + m2])^-beta with
 * m1 = (normDepth - 1) / 2, m2 = normDepth - m1 - 1 (bits/nnnormalize.cu:143-226).  The power is powf, as in the reference's
 * GPU kernels; the reference's CPU code approximates it.  dX is overwritten; backward uses the context's scratch. */
int vlb_lrn_forward(vlb_ctx* ctx, float* Y, float const* X, int H, int W, int C, int N, int normDepth, double kappa,
                    double alpha, double beta);
int vlb_lrn_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, int H, int W, int C, int N, int normDepth,
                     double kappa, double alpha, double beta);
/* matlab/vl_nnsoftmax.m: softmax over the channels; backward takes X (not Y), as the MATLAB function does. */
int vlb_softmax_forward(vlb_ctx* ctx, float* Y, float const* X, int H, int W, int C, int N);
int vlb_softmax_backward(vlb_ctx* ctx, float* dX, float const* X, float const* dY, int H, int W, int C, int N);
/* matlab/vl_nndropout.m: mask = 1/(1-rate) * (u >= rate) with u uniform in [0, 1) from a counter-based generator (element i
 * of a call with the same seed always gets the same number); the forward and backward passes are Y = mask .* X (vlb_mul). */
int vlb_dropout_mask(vlb_ctx* ctx, float* mask, size_t n, double rate, unsigned long long seed);
int vlb_mul(vlb_ctx* ctx, float* Y, float const* A, float const* B, size_t n);

/* The trainer's other solvers after the gradient exchange (examples/+solver/adagrad.m, adadelta.m, adam.m, rmsprop.m, called
 * at examples/cnn_train.m:503-507), each fused with the pass before it: g = gradMult*G + decay*W (cnn_train.m:481-483), then
 * the solver's element-wise update of W and of its state, every MATLAB operation rounded to single as MATLAB does.
 *   adagrad:  S1 = S1*rho + g^2;                 W -= lr*g / (sqrt(S1) + epsilon)
 *   rmsprop:  S1 = S1*rho + g^2*(1-rho);         W -= lr*g / (sqrt(S1) + epsilon)
 *   adadelta: S1 = S1*rho + g^2*(1-rho);  d = -sqrt((S2+epsilon)/(S1+epsilon))*g;  S2 = S2*rho + d^2*(1-rho);  W += d
 *   adam:     S1 = beta1*S1 + (1-beta1)*g;  S2 = beta2*S2 + (1-beta2)*g^2;  W -= lr*sqrt(1-beta2^t)/(1-beta1^t) * S1/(sqrt(S2)+epsilon)
 * S1, S2: state tensors of n floats, zero before the first step (S2 only for adadelta and adam); t: adam's step count
 * after this step (1 on the first).  W, S1, S2 are updated in place, G is only read. */
enum { VLB_SOLVER_ADAGRAD = 0, VLB_SOLVER_ADADELTA = 1, VLB_SOLVER_ADAM = 2, VLB_SOLVER_RMSPROP = 3 };
typedef struct { double rho, epsilon, beta1, beta2; } vlb_solver_opts;
int vlb_solver_update(vlb_ctx* ctx, int solver, float* W, float* S1, float* S2, float const* G, size_t n, double gradMult,
                      double decay, double lr, vlb_solver_opts const* opts, long long t);

#ifdef __cplusplus
}
#endif
#endif /* VLB_H */
