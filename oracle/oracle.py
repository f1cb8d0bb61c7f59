"""ctypes front end to the two CPU checkers (TEST INFRASTRUCTURE ONLY).

``restatement()`` loads ``libmcn_oracle.so`` (the plain-C restatement,
``mcn_oracle.c``); ``reference()`` loads ``_ref/libmcn_ref.so`` (the
reference's own CPU backend compiled unmodified) or returns None when it has
not been built.  Both expose the same methods.

Tensors are numpy arrays with MATLAB semantics: logical shape (H, W, C, N),
Fortran (column-major) memory order, so element (h,w,c,n) is at
h + H*(w + W*(c + C*n)) exactly as in the reference (bits/data.cu:498-505).
dtype float32 or float64 selects the reference's single or double
instantiation.

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import
this module.
"""
import ctypes as C
import glob
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

c_int_p = C.POINTER(C.c_int)
c_double_p = C.POINTER(C.c_double)


def fa(a, dtype=None):
    """Fortran-contiguous array of the given dtype (copy only when needed)."""
    return np.asfortranarray(a, dtype=dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _ints(v):
    arr = (C.c_int * len(v))(*[int(i) for i in v])
    return arr


def conv_out_shape(x_shape, f_shape, stride=(1, 1), pad=(0, 0, 0, 0), dilate=(1, 1)):
    """Output shape of vl_nnconv (reference matlab/src/vl_nnconv.cu:324-331)."""
    H, W, _, N = x_shape
    FH, FW, _, K = f_shape
    Ho = (H + pad[0] + pad[1] - ((FH - 1) * dilate[0] + 1)) // stride[0] + 1
    Wo = (W + pad[2] + pad[3] - ((FW - 1) * dilate[1] + 1)) // stride[1] + 1
    return (Ho, Wo, K, N)


def convt_out_shape(x_shape, f_shape, upsample=(1, 1), crop=(0, 0, 0, 0), num_groups=1):
    # matlab/src/vl_nnconvt.cu:293-296
    H, W, _, N = x_shape
    FH, FW, FD, _ = f_shape
    return ((H - 1) * upsample[0] - (crop[0] + crop[1]) + FH, (W - 1) * upsample[1] - (crop[2] + crop[3]) + FW,
            FD * num_groups, N)


def pool_out_shape(x_shape, pool, stride=(1, 1), pad=(0, 0, 0, 0)):
    """Output shape of vl_nnpool (reference matlab/src/vl_nnpool.cu:240-247)."""
    H, W, Cc, N = x_shape
    Ho = (H + pad[0] + pad[1] - pool[0]) // stride[0] + 1
    Wo = (W + pad[2] + pad[3] - pool[1]) // stride[1] + 1
    return (Ho, Wo, Cc, N)


class CpuBackend:
    """Same call surface for the restatement (prefix ``mcno_``) and the compiled
    reference (prefix ``mcnref_``)."""

    def __init__(self, lib, prefix, name):
        self.lib = lib
        self.prefix = prefix
        self.name = name

    def _fn(self, name, argtypes):
        f = getattr(self.lib, self.prefix + name)
        f.restype = C.c_int
        f.argtypes = argtypes
        return f

    @staticmethod
    def _dt(a):
        if a.dtype == np.float32:
            return 0
        if a.dtype == np.float64:
            return 1
        raise TypeError("float32 or float64 expected")

    @staticmethod
    def _check(rc, what):
        if rc != 0:
            raise RuntimeError("%s failed with vl::ErrorCode %d" % (what, rc))

    # --- convolution -------------------------------------------------
    def conv_forward(self, x, f, b=None, stride=(1, 1), pad=(0, 0, 0, 0), dilate=(1, 1)):
        x, f = fa(x), fa(f)
        b = None if b is None else fa(b, x.dtype)
        y = np.zeros(conv_out_shape(x.shape, f.shape, stride, pad, dilate), dtype=x.dtype, order="F")
        shape = _ints(list(x.shape) + list(f.shape))
        prm = _ints(list(stride) + list(pad) + list(dilate))
        fn = self._fn("conv_forward", [C.c_int] + [C.c_void_p] * 4 + [c_int_p, c_int_p])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), _ptr(f), _ptr(b), shape, prm), "conv_forward")
        return y

    def conv_backward(self, x, f, dy, stride=(1, 1), pad=(0, 0, 0, 0), dilate=(1, 1),
                      want=(True, True, True)):
        x, f, dy = fa(x), fa(f), fa(dy)
        dx = np.zeros(x.shape, x.dtype, order="F") if want[0] else None
        df = np.zeros(f.shape, x.dtype, order="F") if want[1] else None
        db = np.zeros((f.shape[3],), x.dtype) if want[2] else None
        shape = _ints(list(x.shape) + list(f.shape))
        prm = _ints(list(stride) + list(pad) + list(dilate))
        fn = self._fn("conv_backward", [C.c_int] + [C.c_void_p] * 6 + [c_int_p, c_int_p])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(df), _ptr(db), _ptr(x), _ptr(f), _ptr(dy), shape, prm),
                    "conv_backward")
        return dx, df, db

    # --- convolution transpose ---------------------------------------
    def convt_forward(self, x, f, b=None, upsample=(1, 1), crop=(0, 0, 0, 0), num_groups=1):
        x, f = fa(x), fa(f)
        b = None if b is None else fa(b, x.dtype)
        y = np.zeros(convt_out_shape(x.shape, f.shape, upsample, crop, num_groups), dtype=x.dtype, order="F")
        shape = _ints(list(x.shape) + list(f.shape))
        prm = _ints(list(upsample) + list(crop) + [num_groups])
        fn = self._fn("convt_forward", [C.c_int] + [C.c_void_p] * 4 + [c_int_p, c_int_p])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), _ptr(f), _ptr(b), shape, prm), "convt_forward")
        return y

    def convt_backward(self, x, f, dy, upsample=(1, 1), crop=(0, 0, 0, 0), num_groups=1, want=(True, True, True)):
        x, f, dy = fa(x), fa(f), fa(dy)
        dx = np.zeros(x.shape, x.dtype, order="F") if want[0] else None
        df = np.zeros(f.shape, x.dtype, order="F") if want[1] else None
        db = np.zeros((f.shape[2] * num_groups,), x.dtype) if want[2] else None
        shape = _ints(list(x.shape) + list(f.shape))
        prm = _ints(list(upsample) + list(crop) + [num_groups])
        fn = self._fn("convt_backward", [C.c_int] + [C.c_void_p] * 6 + [c_int_p, c_int_p])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(df), _ptr(db), _ptr(x), _ptr(f), _ptr(dy), shape, prm),
                    "convt_backward")
        return dx, df, db

    def fc_forward(self, x, f, b=None):
        x, f = fa(x), fa(f)
        b = None if b is None else fa(b, x.dtype)
        y = np.zeros((1, 1, f.shape[3], x.shape[3]), x.dtype, order="F")
        shape = _ints(list(x.shape) + list(f.shape))
        fn = self._fn("fc_forward", [C.c_int] + [C.c_void_p] * 4 + [c_int_p])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), _ptr(f), _ptr(b), shape), "fc_forward")
        return y

    def fc_backward(self, x, f, dy, want=(True, True, True)):
        x, f, dy = fa(x), fa(f), fa(dy)
        dx = np.zeros(x.shape, x.dtype, order="F") if want[0] else None
        df = np.zeros(f.shape, x.dtype, order="F") if want[1] else None
        db = np.zeros((f.shape[3],), x.dtype) if want[2] else None
        shape = _ints(list(x.shape) + list(f.shape))
        fn = self._fn("fc_backward", [C.c_int] + [C.c_void_p] * 6 + [c_int_p])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(df), _ptr(db), _ptr(x), _ptr(f), _ptr(dy), shape), "fc_backward")
        return dx, df, db

    # --- bias ----------------------------------------------------------
    def bias_forward(self, y, ymult, x, xmult, b, bmult):
        y = fa(y).copy(order="F")
        x = None if x is None else fa(x, y.dtype)
        b = None if b is None else fa(b, y.dtype)
        H, W, K, N = y.shape
        fn = self._fn("bias_forward", [C.c_int, C.c_void_p, C.c_double, C.c_void_p, C.c_double, C.c_void_p,
                                       C.c_double] + [C.c_int] * 4)
        self._check(fn(self._dt(y), _ptr(y), ymult, _ptr(x), xmult, _ptr(b), bmult, H, W, K, N), "bias_forward")
        return y

    def bias_backward(self, dx, dxmult, db, dbmult, xmult, bmult, dy):
        dy = fa(dy)
        dx = None if dx is None else fa(dx, dy.dtype).copy(order="F")
        db = None if db is None else fa(db, dy.dtype).copy()
        H, W, K, N = dy.shape
        fn = self._fn("bias_backward", [C.c_int, C.c_void_p, C.c_double, C.c_void_p, C.c_double, C.c_double,
                                        C.c_double, C.c_void_p] + [C.c_int] * 4)
        self._check(fn(self._dt(dy), _ptr(dx), dxmult, _ptr(db), dbmult, xmult, bmult, _ptr(dy), H, W, K, N),
                    "bias_backward")
        return dx, db

    # --- batch normalisation ------------------------------------------
    def bnorm_forward(self, x, g, b, eps=1e-4, moments=None):
        x = fa(x)
        g, b = fa(g, x.dtype), fa(b, x.dtype)
        H, W, Cc, N = x.shape
        y = np.zeros(x.shape, x.dtype, order="F")
        if moments is None:
            mom = np.zeros((Cc, 2), x.dtype, order="F")
            fn = self._fn("bnorm_forward", [C.c_int] + [C.c_void_p] * 5 + [C.c_int] * 4 + [C.c_double])
            self._check(fn(self._dt(x), _ptr(y), _ptr(mom), _ptr(x), _ptr(g), _ptr(b), H, W, Cc, N, eps),
                        "bnorm_forward")
        else:
            mom = fa(moments, x.dtype)
            fn = self._fn("bnorm_forward_moment", [C.c_int] + [C.c_void_p] * 5 + [C.c_int] * 4 + [C.c_double])
            self._check(fn(self._dt(x), _ptr(y), _ptr(mom), _ptr(x), _ptr(g), _ptr(b), H, W, Cc, N, eps),
                        "bnorm_forward_moment")
        return y, mom

    def bnorm_backward(self, x, g, b, dy, eps=1e-4, moments=None):
        x, dy = fa(x), fa(dy)
        g, b = fa(g, x.dtype), fa(b, x.dtype)
        H, W, Cc, N = x.shape
        dx = np.zeros(x.shape, x.dtype, order="F")
        dg = np.zeros((Cc,), x.dtype)
        db = np.zeros((Cc,), x.dtype)
        name = "bnorm_backward" if moments is None else "bnorm_backward_moment"
        mom = np.zeros((Cc, 2), x.dtype, order="F") if moments is None else fa(moments, x.dtype)
        fn = self._fn(name, [C.c_int] + [C.c_void_p] * 8 + [C.c_int] * 4 + [C.c_double])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(dg), _ptr(db), _ptr(mom), _ptr(x), _ptr(g), _ptr(b), _ptr(dy),
                       H, W, Cc, N, eps), name)
        return dx, dg, db, mom

    # --- pooling -------------------------------------------------------
    def pool_forward(self, x, pool, stride=(1, 1), pad=(0, 0, 0, 0), method="max"):
        x = fa(x)
        y = np.zeros(pool_out_shape(x.shape, pool, stride, pad), x.dtype, order="F")
        prm = _ints(list(pool) + list(stride) + list(pad) + [0 if method == "max" else 1])
        fn = self._fn("pool_forward", [C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [c_int_p])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), *x.shape, prm), "pool_forward")
        return y

    def pool_backward(self, x, dy, pool, stride=(1, 1), pad=(0, 0, 0, 0), method="max"):
        x, dy = fa(x), fa(dy)
        dx = np.zeros(x.shape, x.dtype, order="F")
        prm = _ints(list(pool) + list(stride) + list(pad) + [0 if method == "max" else 1])
        fn = self._fn("pool_backward", [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [c_int_p])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(x), _ptr(dy), *x.shape, prm), "pool_backward")
        return dx

    # --- ROI pooling ---------------------------------------------------
    @staticmethod
    def _tf(transform):
        t = np.asarray(transform, dtype=np.float64).ravel(order="F")
        if t.size == 1:                       # scalar s => [s 0 0 s 1-s 1-s] (vl_nnroipool.cu:150-155)
            s = float(t[0])
            t = np.array([s, 0, 0, s, 1 - s, 1 - s], dtype=np.float64)
        assert t.size == 6
        return np.ascontiguousarray(t)

    def roipool_forward(self, x, rois, subdivisions=(1, 1), transform=1.0, method="max"):
        x = fa(x)
        rois = fa(rois, x.dtype)
        K = rois.size // 5
        tf = self._tf(transform)
        y = np.zeros((subdivisions[0], subdivisions[1], x.shape[2], K), x.dtype, order="F")
        fn = self._fn("roipool_forward", [C.c_int] + [C.c_void_p] * 3 + [C.c_int] * 7 + [c_double_p, C.c_int])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), _ptr(rois), *x.shape, K, subdivisions[0], subdivisions[1],
                       tf.ctypes.data_as(c_double_p), 0 if method == "max" else 1), "roipool_forward")
        return y

    def roipool_backward(self, x, rois, dy, subdivisions=(1, 1), transform=1.0, method="max"):
        x, dy = fa(x), fa(dy)
        rois = fa(rois, x.dtype)
        K = rois.size // 5
        tf = self._tf(transform)
        dx = np.zeros(x.shape, x.dtype, order="F")
        fn = self._fn("roipool_backward", [C.c_int] + [C.c_void_p] * 4 + [C.c_int] * 7 + [c_double_p, C.c_int])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(x), _ptr(rois), _ptr(dy), *x.shape, K, subdivisions[0],
                       subdivisions[1], tf.ctypes.data_as(c_double_p), 0 if method == "max" else 1),
                    "roipool_backward")
        return dx

    def roipool_bounds(self, rois, x_shape, subdivisions=(1, 1), transform=1.0):
        """Restatement only: (bounds[4,S0,S1,K] int32 = hstart,hend,wstart,wend; images[K])."""
        rois = fa(rois)
        K = rois.size // 5
        tf = self._tf(transform)
        H, W, _, N = x_shape
        bounds = np.zeros((4, subdivisions[0], subdivisions[1], K), np.int32, order="F")
        images = np.zeros((K,), np.int32)
        fn = self._fn("roipool_bounds", [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [c_double_p])
        self._check(fn(self._dt(rois), _ptr(bounds), _ptr(images), _ptr(rois), H, W, N, K, subdivisions[0],
                       subdivisions[1], tf.ctypes.data_as(c_double_p)), "roipool_bounds")
        return bounds, images

    # --- bilinear sampler ----------------------------------------------
    def sampler_forward(self, x, grid):
        x = fa(x)
        grid = fa(grid, x.dtype)
        _, Ho, Wo, Ng = grid.shape
        y = np.zeros((Ho, Wo, x.shape[2], Ng), x.dtype, order="F")
        fn = self._fn("sampler_forward", [C.c_int] + [C.c_void_p] * 3 + [C.c_int] * 7)
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), _ptr(grid), *x.shape, Ho, Wo, Ng), "sampler_forward")
        return y

    def sampler_backward(self, x, grid, dy, want=(True, True)):
        x, dy = fa(x), fa(dy)
        grid = fa(grid, x.dtype)
        _, Ho, Wo, Ng = grid.shape
        dx = np.zeros(x.shape, x.dtype, order="F") if want[0] else None
        dgrid = np.zeros(grid.shape, x.dtype, order="F") if want[1] else None
        fn = self._fn("sampler_backward", [C.c_int] + [C.c_void_p] * 5 + [C.c_int] * 7)
        self._check(fn(self._dt(x), _ptr(dx), _ptr(dgrid), _ptr(x), _ptr(grid), _ptr(dy), *x.shape, Ho, Wo, Ng),
                    "sampler_backward")
        return dx, dgrid

    # --- local response normalisation ---------------------------------
    def lrn_forward(self, x, param):
        x = fa(x)
        y = np.zeros(x.shape, x.dtype, order="F")
        prm = (C.c_double * 4)(*[float(v) for v in param])
        fn = self._fn("lrn_forward", [C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [c_double_p])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), *x.shape, prm), "lrn_forward")
        return y

    def lrn_backward(self, x, param, dy):
        x = fa(x)
        dy = fa(dy, x.dtype)
        dx = np.zeros(x.shape, x.dtype, order="F")
        prm = (C.c_double * 4)(*[float(v) for v in param])
        fn = self._fn("lrn_backward", [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [c_double_p])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(x), _ptr(dy), *x.shape, prm), "lrn_backward")
        return dx

    def softmax(self, x, dzdy=None):
        """Restatement only (matlab/vl_nnsoftmax.m)."""
        x = fa(x)
        dz = None if dzdy is None else fa(dzdy, x.dtype)
        out = np.zeros(x.shape, x.dtype, order="F")
        fn = self._fn("softmax", [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 4)
        self._check(fn(self._dt(x), _ptr(out), _ptr(x), _ptr(dz), *x.shape), "softmax")
        return out

    # --- glue (restatement only: the reference has these in MATLAB) ----
    def relu_forward(self, x):
        x = fa(x)
        y = np.zeros(x.shape, x.dtype, order="F")
        fn = self._fn("relu_forward", [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t])
        self._check(fn(self._dt(x), _ptr(y), _ptr(x), x.size), "relu_forward")
        return y

    def relu_backward(self, x, dy):
        x, dy = fa(x), fa(dy)
        dx = np.zeros(x.shape, x.dtype, order="F")
        fn = self._fn("relu_backward", [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t])
        self._check(fn(self._dt(x), _ptr(dx), _ptr(x), _ptr(dy), x.size), "relu_backward")
        return dx

    def softmaxloss_forward(self, x, labels):
        x = fa(x)
        labels = np.ascontiguousarray(labels, dtype=x.dtype)
        loss = np.zeros((1,), x.dtype)
        fn = self._fn("softmaxloss_forward", [C.c_int] + [C.c_void_p] * 3 + [C.c_int] * 4)
        self._check(fn(self._dt(x), _ptr(loss), _ptr(x), _ptr(labels), *x.shape), "softmaxloss_forward")
        return loss[0]

    def softmaxloss_backward(self, x, labels, dzdy=1.0):
        x = fa(x)
        labels = np.ascontiguousarray(labels, dtype=x.dtype)
        dx = np.zeros(x.shape, x.dtype, order="F")
        fn = self._fn("softmaxloss_backward", [C.c_int] + [C.c_void_p] * 3 + [C.c_double] + [C.c_int] * 4)
        self._check(fn(self._dt(x), _ptr(dx), _ptr(x), _ptr(labels), dzdy, *x.shape), "softmaxloss_backward")
        return dx


_restatement = None
_reference = None


def restatement():
    """The plain-C restatement; built on first use (needs gcc)."""
    global _restatement
    if _restatement is None:
        path = os.path.join(HERE, "libmcn_oracle.so")
        if not os.path.exists(path):
            import importlib.util
            spec = importlib.util.spec_from_file_location("build_oracle", os.path.join(HERE, "build_oracle.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_restatement()
        _restatement = CpuBackend(C.CDLL(path), "mcno_", "restatement")
    return _restatement


def reference():
    """The reference's compiled CPU backend, or None when it has not been built."""
    global _reference
    if _reference is None:
        path = os.path.join(HERE, "_ref", "libmcn_ref.so")
        if not os.path.exists(path):
            return None
        _reference = CpuBackend(C.CDLL(path), "mcnref_", "reference")
    return _reference


def reference_use_openblas(threads):
    """Route the compiled reference's gemm/gemv to numpy's bundled ILP64 OpenBLAS.
    Returns True on success; the plain BLAS stays in place otherwise."""
    ref = reference()
    if ref is None:
        return False
    libs = glob.glob(os.path.join(os.path.dirname(np.__file__), "..", "numpy.libs", "libscipy_openblas64_*.so"))
    fn = ref.lib.mcnref_use_openblas
    fn.restype = C.c_int
    fn.argtypes = [C.c_char_p, C.c_int]
    for p in libs:
        if fn(os.path.abspath(p).encode(), int(threads)):
            return True
    return False


def reference_use_plain_blas():
    ref = reference()
    if ref is not None:
        ref.lib.mcnref_use_plain_blas()
