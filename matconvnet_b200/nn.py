"""The reference's building blocks with their MATLAB call signatures, on device tensors.

Forward:  ``y = vl_nnX(x, params...)``;  backward: ``dx, dparams... = vl_nnX(x, params..., dzdy)``
-- the convention of every block of the reference (matlab/vl_nnconv.m, vl_nnbnorm.m,
vl_nnpool.m, vl_nnroipool.m, vl_nnbilinearsampler.m, vl_nnrelu.m, vl_nnsoftmaxloss.m).
Arguments are column-major CUDA float32 tensors (see ``mat``); each function validates
shapes as the corresponding MEX gateway does, allocates the outputs, and calls the C ABI.
Nothing here computes on the host.
"""
import ctypes as C

import numpy as np
import torch

from . import capi, mat

_default_ctx = None


def default_context():
    """Process-wide context (the MEX-file-global `context` of the reference,
    matlab/src/vl_nnconv.cu:64)."""
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = capi.Context()
    return _default_ctx


def _ctx(ctx):
    ctx = ctx or default_context()
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    return ctx


def _need(t, name):
    if t is None:
        return None
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32):
        raise TypeError("%s must be a CUDA float32 tensor (this engine has no CPU path)" % name)
    return mat.as_mat(t)


def _pair(v, name):
    v = np.atleast_1d(np.asarray(v)).astype(int).ravel()
    if v.size == 1:
        return int(v[0]), int(v[0])
    if v.size == 2:
        return int(v[0]), int(v[1])
    raise ValueError("%s must have one or two elements" % name)


def _quad(v, name):
    v = np.atleast_1d(np.asarray(v)).astype(int).ravel()
    if v.size == 1:
        return (int(v[0]),) * 4
    if v.size == 4:
        return tuple(int(i) for i in v)
    raise ValueError("%s must have one or four elements" % name)


# --------------------------------------------------------------------- vl_nnconv
def _conv_desc(x, f, stride, pad, dilate):
    H, W, Cc, N = mat.shape4(x)
    FH, FW, FC, K = mat.shape4(f)
    sy, sx = _pair(stride, "STRIDE")
    pt, pb, pl, pr = _quad(pad, "PAD")
    dy, dx = _pair(dilate, "DILATE")
    return capi.ConvDesc(H, W, Cc, N, FH, FW, FC, K, sy, sx, pt, pb, pl, pr, dy, dx)


def _is_fc(d, Ho, Wo):
    # matlab/src/vl_nnconv.cu:351-361
    return (Ho == 1 and Wo == 1 and d.strideY == 1 and d.strideX == 1 and d.padTop == 0 and d.padBottom == 0
            and d.padLeft == 0 and d.padRight == 0 and d.dilateY == 1 and d.dilateX == 1 and d.FC == d.C
            and d.FH == d.H and d.FW == d.W)


def _der_out(given, shape, device, name):
    """A caller-supplied output for a parameter derivative (e.g. a view into a gradient bucket), checked, else a new one."""
    if given is None:
        return mat.empty(shape, device)
    if not (isinstance(given, torch.Tensor) and given.is_cuda and given.dtype == torch.float32 and mat.is_mat(given)
            and given.numel() == int(np.prod(shape)) and given.data_ptr() % 16 == 0):
        raise ValueError("%s: the supplied output must be a dense 16-byte aligned CUDA float32 tensor of %d elements"
                         % (name, int(np.prod(shape))))
    return given


def vl_nnconv(x, f, b, dzdy=None, stride=1, pad=0, dilate=1, no_der_data=False, no_der_filters=False,
              no_der_biases=False, relu=False, through_relu=False, der_out=None, ctx=None):
    """Y = VL_NNCONV(X, F, B) / [DX, DF, DB] = VL_NNCONV(X, F, B, DZDY) (matlab/vl_nnconv.m;
    gateway matlab/src/vl_nnconv.cu:87-503).  B may be None.  Empty F (the subsampling mode of
    the reference) is not part of this engine.  relu=True (forward only) returns max(Y, 0) from the same kernels,
    bit-identical to vl_nnrelu(vl_nnconv(...)).  through_relu=True (backward only) is for an X that is the output of a
    ReLU: DX is then the derivative with respect to that ReLU's input, bit-identical to vl_nnrelu(X, DX).
    der_out=(DF, DB) (backward only; either may be None) makes the kernels write the parameter derivatives into tensors the
    caller owns -- views into a gradient-exchange bucket -- instead of new ones; they are returned as DF, DB."""
    ctx = _ctx(ctx)
    x, f, b, dzdy = _need(x, "x"), _need(f, "f"), _need(b, "b"), _need(dzdy, "dzdy")
    if f is None or f.numel() == 0:
        raise capi.VlbError(1, "vl_nnconv with empty filters (subsampling) is not supported")
    d = _conv_desc(x, f, stride, pad, dilate)
    if b is not None and b.numel() != d.K:
        raise ValueError("The number of elements of BIASES is not the same as the number of filters.")
    Ho, Wo = C.c_int(), C.c_int()
    lib = ctx.lib
    lib.vlb_conv_output_shape(C.byref(d), C.byref(Ho), C.byref(Wo))
    Ho, Wo = Ho.value, Wo.value
    fc = _is_fc(d, Ho, Wo)
    if dzdy is None:
        y = mat.empty((Ho, Wo, d.K, d.N), x.device)
        if relu:
            ctx.check(lib.vlb_conv_relu_forward(ctx.handle, mat.ptr(y), mat.ptr(x), mat.ptr(f), mat.ptr(b), C.byref(d)))
        elif fc:
            ctx.check(lib.vlb_fc_forward(ctx.handle, mat.ptr(y), mat.ptr(x), mat.ptr(f), mat.ptr(b), C.byref(d)))
        else:
            ctx.check(lib.vlb_conv_forward(ctx.handle, mat.ptr(y), 0.0, mat.ptr(x), 1.0, mat.ptr(f), mat.ptr(b),
                                           C.byref(d)))
        return y
    if mat.shape4(dzdy) != (Ho, Wo, d.K, d.N):
        raise ValueError("DEROUTPUT dimensions are incompatible with X and FILTERS.")
    dx = None if no_der_data else mat.empty(mat.shape4(x), x.device)
    gdf, gdb = der_out if der_out is not None else (None, None)
    df = None if no_der_filters else _der_out(gdf, mat.shape4(f), x.device, "DF")
    db = None if (no_der_biases or b is None) else _der_out(gdb, (1, d.K), x.device, "DB")
    fn = lib.vlb_relu_conv_backward if through_relu else (lib.vlb_fc_backward if fc else lib.vlb_conv_backward)
    ctx.check(fn(ctx.handle, mat.ptr(dx), mat.ptr(df), mat.ptr(db), mat.ptr(x), mat.ptr(f), mat.ptr(dzdy),
                 C.byref(d)))
    return dx, df, db


# --------------------------------------------------------------------- vl_nnconvt
def vl_nnconvt(x, f, b, dzdy=None, upsample=1, crop=0, num_groups=1, no_der_data=False, no_der_filters=False,
               no_der_biases=False, ctx=None):
    """Y = VL_NNCONVT(X, F, B) / [DX, DF, DB] = VL_NNCONVT(X, F, B, DZDY) (matlab/vl_nnconvt.m; gateway
    matlab/src/vl_nnconvt.cu:87-417).  F is FH x FW x FD x C: FD output channels per filter group, its fourth dimension
    the depth of X.  B may be None."""
    ctx = _ctx(ctx)
    x, f, b, dzdy = _need(x, "x"), _need(f, "f"), _need(b, "b"), _need(dzdy, "dzdy")
    H, W, Cc, N = mat.shape4(x)
    FH, FW, FD, FN = mat.shape4(f)
    uy, ux = _pair(upsample, "UPSAMPLE")
    ct, cb, cl, cr = _quad(crop, "CROP")
    d = capi.ConvtDesc(H, W, Cc, N, FH, FW, FD, FN, uy, ux, ct, cb, cl, cr, int(num_groups))
    K = FD * int(num_groups)
    if b is not None and b.numel() != K:
        raise ValueError("The number of elements of BIASES is not the same as the dimenison of the filters.")
    lib = ctx.lib
    Ho, Wo = C.c_int(), C.c_int()
    lib.vlb_convt_output_shape(C.byref(d), C.byref(Ho), C.byref(Wo))
    Ho, Wo = Ho.value, Wo.value
    if dzdy is None:
        y = mat.empty((max(Ho, 0), max(Wo, 0), K, N), x.device)
        ctx.check(lib.vlb_convt_forward(ctx.handle, mat.ptr(y), mat.ptr(x), mat.ptr(f), mat.ptr(b), C.byref(d)))
        return y
    if mat.shape4(dzdy) != (Ho, Wo, K, N):
        raise ValueError("DEROUTPUT dimensions are incompatible with X and FILTERS.")
    dx = None if no_der_data else mat.empty(mat.shape4(x), x.device)
    df = None if no_der_filters else mat.empty(mat.shape4(f), x.device)
    db = None if (no_der_biases or b is None) else mat.empty((1, K), x.device)
    ctx.check(lib.vlb_convt_backward(ctx.handle, mat.ptr(dx), mat.ptr(df), mat.ptr(db), mat.ptr(x), mat.ptr(f),
                                     mat.ptr(dzdy), C.byref(d)))
    return dx, df, db


# --------------------------------------------------------------------- vl_nnbnorm
def vl_nnbnorm(x, g, b, dzdy=None, epsilon=1e-4, moments=None, der_out=None, relu=False, ctx=None):
    """[Y, MOMENTS] = VL_NNBNORM(X, G, B) / [DX, DG, DB, MOMENTS] = VL_NNBNORM(X, G, B, DZDY)
    (matlab/vl_nnbnorm.m; gateway matlab/src/vl_nnbnorm.cu:73-302).  MOMENTS is C x 2:
    [mean, sigma] with sigma = sqrt(var + epsilon).  relu=True (forward, moments from the batch) returns max(Y, 0) from the
    same kernel, bit-identical to vl_nnrelu(vl_nnbnorm(...))."""
    ctx = _ctx(ctx)
    x, g, b, dzdy, moments = _need(x, "x"), _need(g, "g"), _need(b, "b"), _need(dzdy, "dzdy"), _need(moments, "moments")
    H, W, Cc, N = mat.shape4(x)
    if g.numel() != Cc or b.numel() != Cc:
        raise ValueError("The number of elements of MULTIPLIERS / BIASES is not the number of channels.")
    if moments is not None and moments.numel() != 2 * Cc:
        raise ValueError("MOMENTS must have 2*C elements.")
    lib = ctx.lib
    given = moments is not None
    mom = moments if given else mat.empty((Cc, 2), x.device)
    if dzdy is None:
        y = mat.empty((H, W, Cc, N), x.device)
        if given:
            ctx.check(lib.vlb_bnorm_forward_moment(ctx.handle, mat.ptr(y), mat.ptr(mom), mat.ptr(x), mat.ptr(g),
                                                   mat.ptr(b), H, W, Cc, N, float(epsilon)))
        else:
            fwd = lib.vlb_bnorm_relu_forward if relu else lib.vlb_bnorm_forward
            ctx.check(fwd(ctx.handle, mat.ptr(y), mat.ptr(mom), mat.ptr(x), mat.ptr(g), mat.ptr(b), H, W, Cc, N, float(epsilon)))
        if relu and given:
            ctx.check(lib.vlb_relu_forward(ctx.handle, mat.ptr(y), mat.ptr(y), y.numel()))
        return y, mom
    if mat.shape4(dzdy) != (H, W, Cc, N):
        raise ValueError("DZDY dimensions are incompatible with X.")
    dx = mat.empty((H, W, Cc, N), x.device)
    gdg, gdb = der_out if der_out is not None else (None, None)     # caller-owned outputs, as in vl_nnconv
    dg = _der_out(gdg, (Cc, 1), x.device, "DG")
    db = _der_out(gdb, (Cc, 1), x.device, "DB")
    fn = lib.vlb_bnorm_backward_moment if given else lib.vlb_bnorm_backward
    ctx.check(fn(ctx.handle, mat.ptr(dx), mat.ptr(dg), mat.ptr(db), mat.ptr(mom), mat.ptr(x), mat.ptr(g),
                 mat.ptr(b), mat.ptr(dzdy), H, W, Cc, N, float(epsilon)))
    return dx, dg, db, mom


# --------------------------------------------------------------------- vl_nnpool
def vl_nnpool(x, pool, dzdy=None, stride=1, pad=0, method="max", through_relu=False, ctx=None):
    """Y = VL_NNPOOL(X, POOL) / DX = VL_NNPOOL(X, POOL, DZDY) (matlab/vl_nnpool.m; gateway
    matlab/src/vl_nnpool.cu:72-315).  through_relu=True (backward only) is for an X that is the output of a ReLU: DX is
    then the derivative with respect to that ReLU's input, bit-identical to vl_nnrelu(X, DX)."""
    ctx = _ctx(ctx)
    x, dzdy = _need(x, "x"), _need(dzdy, "dzdy")
    H, W, Cc, N = mat.shape4(x)
    ph, pw = _pair(pool, "POOL")
    sy, sx = _pair(stride, "STRIDE")
    pt, pb, pl, pr = _quad(pad, "PAD")
    if method not in ("max", "avg"):
        raise ValueError("METHOD is not a supported method.")
    d = capi.PoolDesc(H, W, Cc, N, ph, pw, sy, sx, pt, pb, pl, pr, capi.POOL_MAX if method == "max" else capi.POOL_AVG)
    lib = ctx.lib
    Ho, Wo = C.c_int(), C.c_int()
    lib.vlb_pool_output_shape(C.byref(d), C.byref(Ho), C.byref(Wo))
    Ho, Wo = Ho.value, Wo.value
    if dzdy is None:
        y = mat.empty((max(Ho, 0), max(Wo, 0), Cc, N), x.device)
        ctx.check(lib.vlb_pool_forward(ctx.handle, mat.ptr(y), mat.ptr(x), C.byref(d)))
        return y
    if mat.shape4(dzdy) != (Ho, Wo, Cc, N):
        raise ValueError("DZDY dimensions are incompatible with X and POOL.")
    dx = mat.empty((H, W, Cc, N), x.device)
    fn = lib.vlb_relu_pool_backward if through_relu else lib.vlb_pool_backward
    ctx.check(fn(ctx.handle, mat.ptr(dx), mat.ptr(x), mat.ptr(dzdy), C.byref(d)))
    return dx


# --------------------------------------------------------------------- vl_nnroipool
def _transform(t):
    t = np.asarray(t, dtype=np.float64).ravel(order="F")
    if t.size == 1:      # matlab/src/vl_nnroipool.cu:150-155
        s = float(t[0])
        t = np.array([s, 0.0, 0.0, s, 1.0 - s, 1.0 - s])
    if t.size != 6:
        raise ValueError("TRANSFORM must be a scalar or a 2 x 3 matrix.")
    return (C.c_double * 6)(*[float(v) for v in t])


def vl_nnroipool(x, rois, dzdy=None, subdivisions=(1, 1), transform=1.0, method="max", ctx=None):
    """Y = VL_NNROIPOOL(X, ROIS) / DX = VL_NNROIPOOL(X, ROIS, DZDY) (matlab/vl_nnroipool.m; gateway
    matlab/src/vl_nnroipool.cu:70-271).  ROIS is 5 x K: [image; u1; v1; u2; v2], 1-based."""
    ctx = _ctx(ctx)
    x, rois, dzdy = _need(x, "x"), _need(rois, "rois"), _need(dzdy, "dzdy")
    H, W, Cc, N = mat.shape4(x)
    if rois.numel() % 5 != 0:
        raise ValueError("ROIs is not a 5 x K array.")
    K = rois.numel() // 5
    S0, S1 = _pair(subdivisions, "SUBDIVISIONS")
    tf = _transform(transform)
    m = capi.POOL_MAX if method == "max" else capi.POOL_AVG
    lib = ctx.lib
    if dzdy is None:
        y = mat.empty((S0, S1, Cc, K), x.device)
        ctx.check(lib.vlb_roipool_forward(ctx.handle, mat.ptr(y), mat.ptr(x), mat.ptr(rois), H, W, Cc, N, K, S0, S1, tf, m))
        return y
    if mat.shape4(dzdy) != (S0, S1, Cc, K):
        raise ValueError("DZDY dimensions are incompatible with X and ROIS.")
    dx = mat.empty((H, W, Cc, N), x.device)
    ctx.check(lib.vlb_roipool_backward(ctx.handle, mat.ptr(dx), mat.ptr(x), mat.ptr(rois), mat.ptr(dzdy), H, W, Cc, N,
                                       K, S0, S1, tf, m))
    return dx


def roipool_bounds(rois, x_shape, subdivisions=(1, 1), transform=1.0, ctx=None):
    """Device bin geometry: (bounds int32 [4,S0,S1,K] = hstart,hend,wstart,wend; images int32 [K])."""
    ctx = _ctx(ctx)
    rois = _need(rois, "rois")
    H, W, _, N = x_shape
    K = rois.numel() // 5
    S0, S1 = _pair(subdivisions, "SUBDIVISIONS")
    bounds = mat.zeros((4, S0, S1, K), rois.device, torch.int32)
    images = torch.zeros(K, device=rois.device, dtype=torch.int32)
    ctx.check(ctx.lib.vlb_roipool_bounds(ctx.handle, mat.ptr(bounds), mat.ptr(images), mat.ptr(rois), H, W, N, K,
                                         S0, S1, _transform(transform)))
    return bounds, images


# --------------------------------------------------------------------- vl_nnbilinearsampler
def vl_nnbilinearsampler(x, grid, dzdy=None, ctx=None):
    """Y = VL_NNBILINEARSAMPLER(X, GRID) / [DX, DGRID] = VL_NNBILINEARSAMPLER(X, GRID, DZDY)
    (matlab/vl_nnbilinearsampler.m; gateway matlab/src/vl_nnbilinearsampler.cu:66-223)."""
    ctx = _ctx(ctx)
    x, grid, dzdy = _need(x, "x"), _need(grid, "grid"), _need(dzdy, "dzdy")
    H, W, Cc, N = mat.shape4(x)
    two, Ho, Wo, Ng = mat.shape4(grid)
    if two != 2:
        raise ValueError("GRID has more than 2 channels.")
    if Ng % N != 0:
        raise ValueError("The number of GRIDs is not a multiple of the number of images.")
    lib = ctx.lib
    if dzdy is None:
        y = mat.empty((Ho, Wo, Cc, Ng), x.device)
        ctx.check(lib.vlb_sampler_forward(ctx.handle, mat.ptr(y), mat.ptr(x), mat.ptr(grid), H, W, Cc, N, Ho, Wo, Ng))
        return y
    if mat.shape4(dzdy) != (Ho, Wo, Cc, Ng):
        raise ValueError("DZDY dimensions are incompatible with X and GRID.")
    dx = mat.empty((H, W, Cc, N), x.device)
    dgrid = mat.empty((2, Ho, Wo, Ng), x.device)
    ctx.check(lib.vlb_sampler_backward(ctx.handle, mat.ptr(dx), mat.ptr(dgrid), mat.ptr(x), mat.ptr(grid),
                                       mat.ptr(dzdy), H, W, Cc, N, Ho, Wo, Ng))
    return dx, dgrid


# --------------------------------------------------------------------- gradient scaling
def scale_(t, alpha, ctx=None):
    """t *= alpha in place: the division by the number of workers of an all-reduced gradient
    (examples/cnn_train.m:482-483)."""
    ctx = _ctx(ctx)
    if not (t.is_cuda and t.dtype == torch.float32):
        raise TypeError("CUDA float32 tensor expected")
    ctx.check(ctx.lib.vlb_scale(ctx.handle, t.data_ptr(), float(alpha), t.numel()))
    return t


def _flat32(t, name):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32):
        raise TypeError("%s must be a CUDA float32 tensor" % name)
    return t


def vl_taccum(alpha, a, beta, b, out=None, ctx=None):
    """Y = VL_TACCUM(ALPHA, A, BETA, B) = ALPHA*A + BETA*B (matlab/vl_taccum.m); out=a updates A in place."""
    ctx = _ctx(ctx)
    a, b = _flat32(a, "a"), _flat32(b, "b")
    if a.numel() != b.numel():
        raise ValueError("A and B do not have the same number of elements.")
    y = torch.empty_like(a) if out is None else out
    ctx.check(ctx.lib.vlb_taccum(ctx.handle, y.data_ptr(), float(alpha), a.data_ptr(), float(beta), b.data_ptr(), a.numel()))
    return y


def sgd_update_(w, momentum_state, grad, grad_mult, decay, momentum, lr, nesterov=False, ctx=None):
    """The trainer's momentum-SGD step on one parameter tensor, in place on w and momentum_state
    (examples/cnn_train.m:478-499: four vl_taccum passes, here one kernel)."""
    ctx = _ctx(ctx)
    w, m, g = _flat32(w, "w"), _flat32(momentum_state, "momentum_state"), _flat32(grad, "grad")
    if not (w.numel() == m.numel() == g.numel()):
        raise ValueError("parameter, momentum and gradient do not have the same number of elements.")
    ctx.check(ctx.lib.vlb_sgd_update(ctx.handle, w.data_ptr(), m.data_ptr(), g.data_ptr(), w.numel(), float(grad_mult),
                                     float(decay), float(momentum), float(lr), 1 if nesterov else 0))
    return w


def solver_update_(solver, w, state, grad, grad_mult, decay, lr, opts=None, ctx=None):
    """One step of examples/+solver/<solver>.m on one parameter tensor, fused with the trainer's normalisation and weight
    decay pass (examples/cnn_train.m:481-507), in place on w and on the solver state.  state: {} before the first step;
    afterwards it holds the solver's tensors (g_sqr; g_sqr and delta_sqr; m, v and the step count t)."""
    ctx = _ctx(ctx)
    if solver not in capi.SOLVERS:
        raise ValueError("unknown solver '%s'" % solver)
    w, g = _flat32(w, "w"), _flat32(grad, "grad")
    if w.numel() != g.numel():
        raise ValueError("parameter and gradient do not have the same number of elements.")
    o = dict(capi.SOLVER_DEFAULTS[solver])
    o.update(opts or {})
    two = solver in ("adadelta", "adam")
    if "s1" not in state:
        state["s1"] = torch.zeros_like(w)
        if two:
            state["s2"] = torch.zeros_like(w)
        state["t"] = 0
    state["t"] += 1
    so = capi.SolverOpts(float(o.get("rho", 0.0)), float(o["epsilon"]), float(o.get("beta1", 0.0)), float(o.get("beta2", 0.0)))
    ctx.check(ctx.lib.vlb_solver_update(ctx.handle, capi.SOLVERS[solver], w.data_ptr(), state["s1"].data_ptr(),
                                        state["s2"].data_ptr() if two else None, g.data_ptr(), w.numel(), float(grad_mult),
                                        float(decay), float(lr), C.byref(so), state["t"]))
    return w


# --------------------------------------------------------------------- MATLAB-only blocks
def vl_nnrelu(x, dzdy=None, ctx=None):
    """matlab/vl_nnrelu.m:43-48 with LEAK = 0."""
    ctx = _ctx(ctx)
    x, dzdy = _need(x, "x"), _need(dzdy, "dzdy")
    out = mat.empty(x.shape, x.device)
    if dzdy is None:
        ctx.check(ctx.lib.vlb_relu_forward(ctx.handle, mat.ptr(out), mat.ptr(x), x.numel()))
    else:
        ctx.check(ctx.lib.vlb_relu_backward(ctx.handle, mat.ptr(out), mat.ptr(x), mat.ptr(dzdy), x.numel()))
    return out


def vl_nnnormalize(x, param, dzdy=None, ctx=None):
    """Y = VL_NNNORMALIZE(X, PARAM) / DZDX = VL_NNNORMALIZE(X, PARAM, DZDY), PARAM = [N KAPPA ALPHA BETA]
    (matlab/vl_nnnormalize.m; gateway matlab/src/vl_nnnormalize.cu:117-162)."""
    ctx = _ctx(ctx)
    x, dzdy = _need(x, "x"), _need(dzdy, "dzdy")
    param = [float(v) for v in np.asarray(param, dtype=np.float64).ravel()]
    if len(param) != 4:
        raise ValueError("PARAM is not a plain 4 vector.")
    depth = int(param[0])
    if depth < 1:
        raise ValueError("The normalization depth is smaller than 1.")
    H, W, Cc, N = mat.shape4(x)
    out = mat.empty((H, W, Cc, N), x.device)
    if dzdy is None:
        ctx.check(ctx.lib.vlb_lrn_forward(ctx.handle, mat.ptr(out), mat.ptr(x), H, W, Cc, N, depth, param[1], param[2], param[3]))
    else:
        if mat.shape4(dzdy) != (H, W, Cc, N):
            raise ValueError("DZDY dimensions are incompatible with X.")
        ctx.check(ctx.lib.vlb_lrn_backward(ctx.handle, mat.ptr(out), mat.ptr(x), mat.ptr(dzdy), H, W, Cc, N, depth, param[1],
                                           param[2], param[3]))
    return out


def vl_nnsoftmax(x, dzdy=None, ctx=None):
    """Y = VL_NNSOFTMAX(X) / DZDX = VL_NNSOFTMAX(X, DZDY): softmax over the channels (matlab/vl_nnsoftmax.m)."""
    ctx = _ctx(ctx)
    x, dzdy = _need(x, "x"), _need(dzdy, "dzdy")
    H, W, Cc, N = mat.shape4(x)
    out = mat.empty((H, W, Cc, N), x.device)
    if dzdy is None:
        ctx.check(ctx.lib.vlb_softmax_forward(ctx.handle, mat.ptr(out), mat.ptr(x), H, W, Cc, N))
    else:
        ctx.check(ctx.lib.vlb_softmax_backward(ctx.handle, mat.ptr(out), mat.ptr(x), mat.ptr(dzdy), H, W, Cc, N))
    return out


def vl_nndropout(x, dzdy=None, rate=0.5, mask=None, seed=0, ctx=None):
    """[Y, MASK] = VL_NNDROPOUT(X, 'rate', R) / [DZDX, MASK] = VL_NNDROPOUT(X, DZDY, 'mask', MASK) (matlab/vl_nndropout.m).
    MASK is drawn when it is not given: 1/(1-rate) where a uniform number is at least the rate, else 0; `seed` selects the
    stream of the counter-based generator (the reference draws from MATLAB's global stream)."""
    ctx = _ctx(ctx)
    x, dzdy, mask = _need(x, "x"), _need(dzdy, "dzdy"), _need(mask, "mask")
    if mask is None:
        mask = mat.empty(x.shape, x.device)
        ctx.check(ctx.lib.vlb_dropout_mask(ctx.handle, mat.ptr(mask), x.numel(), float(rate), int(seed)))
    elif mask.numel() != x.numel():
        raise ValueError("MASK and X do not have the same number of elements.")
    src = x if dzdy is None else dzdy
    out = mat.empty(x.shape, x.device)
    ctx.check(ctx.lib.vlb_mul(ctx.handle, mat.ptr(out), mat.ptr(mask), mat.ptr(src), x.numel()))
    return out, mask


def vl_nnsoftmaxloss(x, c, dzdy=None, ctx=None):
    """matlab/vl_nnsoftmaxloss.m:56-84 with one class label (1-based) per image."""
    ctx = _ctx(ctx)
    x, c = _need(x, "x"), _need(c, "c")
    H, W, Cc, N = mat.shape4(x)
    if c.numel() != N:
        raise ValueError("one label per image expected")
    if dzdy is None:
        loss = torch.empty(1, device=x.device)
        ctx.check(ctx.lib.vlb_softmaxloss_forward(ctx.handle, mat.ptr(loss), mat.ptr(x), mat.ptr(c), H, W, Cc, N))
        return loss
    dx = mat.empty((H, W, Cc, N), x.device)
    ctx.check(ctx.lib.vlb_softmaxloss_backward(ctx.handle, mat.ptr(dx), mat.ptr(x), mat.ptr(c), float(dzdy), H, W, Cc, N))
    return dx
