"""ctypes binding of include/vlb.h.  Loads the in-tree libvlb.so and nothing else."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvlb.so")

ERROR_NAMES = ["VLE_Success", "VLE_Unsupported", "VLE_Cuda", "VLE_Cudnn", "VLE_Cublas", "VLE_OutOfMemory",
               "VLE_OutOfGPUMemeory", "VLE_IllegalArgument", "VLE_Unknown", "VLE_Timeout", "VLE_NoData",
               "VLE_IllegalMessage", "VLE_Interrupted"]

PRECISION_3XTF32, PRECISION_TF32, PRECISION_FP32 = 0, 1, 2
POOL_MAX, POOL_AVG = 0, 1


class VlbError(RuntimeError):
    """Raised when an entry point returns a non-zero vl::ErrorCode."""

    def __init__(self, code, message):
        self.code = code
        name = ERROR_NAMES[code] if 0 <= code < len(ERROR_NAMES) else str(code)
        super().__init__("%s: %s" % (name, message))


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("H", "W", "C", "N", "FH", "FW", "FC", "K", "strideY", "strideX",
                                       "padTop", "padBottom", "padLeft", "padRight", "dilateY", "dilateX")]


class ConvtDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("H", "W", "C", "N", "FH", "FW", "FD", "FN", "upsampleY", "upsampleX",
                                       "cropTop", "cropBottom", "cropLeft", "cropRight", "numGroups")]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("H", "W", "C", "N", "poolH", "poolW", "strideY", "strideX",
                                       "padTop", "padBottom", "padLeft", "padRight", "method")]


class SolverOpts(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("rho", "epsilon", "beta1", "beta2")]


SOLVERS = {"adagrad": 0, "adadelta": 1, "adam": 2, "rmsprop": 3}
# the defaults each solver returns when called without arguments (examples/+solver/*.m)
SOLVER_DEFAULTS = {"adagrad": dict(epsilon=1e-10, rho=1.0), "adadelta": dict(epsilon=1e-6, rho=0.9),
                   "adam": dict(beta1=0.9, beta2=0.999, epsilon=1e-8), "rmsprop": dict(epsilon=1e-8, rho=0.99)}

_P = C.c_void_p
_I = C.c_int
_D = C.c_double
_Z = C.c_size_t

# name -> (restype, argtypes); every symbol include/vlb.h declares
SIGNATURES = {
    "vlb_version": (_I, []),
    "vlb_error_message": (C.c_char_p, [_I]),
    "vlb_ctx_create": (_I, [C.POINTER(_P)]),
    "vlb_ctx_destroy": (_I, [_P]),
    "vlb_ctx_set_stream": (_I, [_P, _P]),
    "vlb_ctx_get_stream": (_P, [_P]),
    "vlb_ctx_set_precision": (_I, [_P, _I]),
    "vlb_ctx_get_precision": (_I, [_P]),
    "vlb_ctx_last_error": (C.c_char_p, [_P]),
    "vlb_ctx_reset_error": (None, [_P]),
    "vlb_ctx_reserve_workspace": (_I, [_P, _Z]),
    "vlb_ctx_workspace_bytes": (_Z, [_P]),
    "vlb_ctx_clear_workspace": (_I, [_P]),
    "vlb_ctx_launch_count": (C.c_longlong, [_P]),
    "vlb_ctx_device_status": (_I, [_P, C.POINTER(_I)]),
    "vlb_ctx_set_wait_limit": (_I, [_P, C.c_longlong]),
    "vlb_ctx_set_test_switch": (_I, [_P, _I]),
    "vlb_ctx_profile_begin": (_I, [_P]),
    "vlb_ctx_profile_end": (_I, [_P, C.POINTER(_D), C.POINTER(_D), C.POINTER(C.c_longlong)]),
    "vlb_ctx_profile_kind": (_I, [_P, _I, C.POINTER(_D), C.POINTER(_D), C.POINTER(C.c_longlong)]),
    "vlb_conv_output_shape": (_I, [C.POINTER(ConvDesc), C.POINTER(_I), C.POINTER(_I)]),
    "vlb_conv_forward": (_I, [_P, _P, _D, _P, _D, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_conv_relu_forward": (_I, [_P, _P, _P, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_conv_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_relu_conv_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_convt_output_shape": (_I, [C.POINTER(ConvtDesc), C.POINTER(_I), C.POINTER(_I)]),
    "vlb_convt_forward": (_I, [_P, _P, _P, _P, _P, C.POINTER(ConvtDesc)]),
    "vlb_convt_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(ConvtDesc)]),
    "vlb_fc_forward": (_I, [_P, _P, _P, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_fc_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(ConvDesc)]),
    "vlb_bias_forward": (_I, [_P, _P, _D, _P, _D, _P, _D, _I, _I, _I, _I]),
    "vlb_bias_backward": (_I, [_P, _P, _D, _P, _D, _D, _D, _P, _I, _I, _I, _I]),
    "vlb_bnorm_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _D]),
    "vlb_bnorm_relu_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _D]),
    "vlb_bnorm_forward_moment": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _D]),
    "vlb_bnorm_backward": (_I, [_P] * 9 + [_I, _I, _I, _I, _D]),
    "vlb_bnorm_backward_moment": (_I, [_P] * 9 + [_I, _I, _I, _I, _D]),
    "vlb_bnorm_backward_noalloc": (_I, [_P] * 8 + [_I, _I, _I, _I, _D, C.c_char_p, _Z]),
    "vlb_pool_output_shape": (_I, [C.POINTER(PoolDesc), C.POINTER(_I), C.POINTER(_I)]),
    "vlb_pool_forward": (_I, [_P, _P, _P, C.POINTER(PoolDesc)]),
    "vlb_pool_backward": (_I, [_P, _P, _P, _P, C.POINTER(PoolDesc)]),
    "vlb_relu_pool_backward": (_I, [_P, _P, _P, _P, C.POINTER(PoolDesc)]),
    "vlb_roipool_forward": (_I, [_P, _P, _P, _P] + [_I] * 7 + [C.POINTER(_D), _I]),
    "vlb_roipool_backward": (_I, [_P, _P, _P, _P, _P] + [_I] * 7 + [C.POINTER(_D), _I]),
    "vlb_roipool_bounds": (_I, [_P, _P, _P, _P] + [_I] * 6 + [C.POINTER(_D)]),
    "vlb_sampler_forward": (_I, [_P, _P, _P, _P] + [_I] * 7),
    "vlb_sampler_backward": (_I, [_P, _P, _P, _P, _P, _P] + [_I] * 7),
    "vlb_relu_forward": (_I, [_P, _P, _P, _Z]),
    "vlb_relu_backward": (_I, [_P, _P, _P, _P, _Z]),
    "vlb_softmaxloss_forward": (_I, [_P, _P, _P, _P, _I, _I, _I, _I]),
    "vlb_softmaxloss_backward": (_I, [_P, _P, _P, _P, _D, _I, _I, _I, _I]),
    "vlb_sum": (_I, [_P, _P, _P, _P, _Z]),
    "vlb_scale": (_I, [_P, _P, _D, _Z]),
    "vlb_taccum": (_I, [_P, _P, _D, _P, _D, _P, _Z]),
    "vlb_sgd_update": (_I, [_P, _P, _P, _P, _Z, _D, _D, _D, _D, _I]),
    "vlb_lrn_forward": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _D, _D, _D]),
    "vlb_lrn_backward": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _D, _D, _D]),
    "vlb_softmax_forward": (_I, [_P, _P, _P, _I, _I, _I, _I]),
    "vlb_softmax_backward": (_I, [_P, _P, _P, _P, _I, _I, _I, _I]),
    "vlb_dropout_mask": (_I, [_P, _P, _Z, _D, C.c_ulonglong]),
    "vlb_mul": (_I, [_P, _P, _P, _P, _Z]),
    "vlb_solver_update": (_I, [_P, _I, _P, _P, _P, _P, _Z, _D, _D, _D, C.POINTER(SolverOpts), C.c_longlong]),
}

_lib = None


def load():
    """Returns the loaded library; raises if libvlb.so has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libvlb.so is missing: build it with `python -m matconvnet_b200.build` "
                              "(this package has no other implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class Context:
    """One per GPU/process: stream, scratch, error state (vl::Context of the reference)."""

    def __init__(self, stream=None, precision=None):
        self.lib = load()
        h = _P()
        rc = self.lib.vlb_ctx_create(C.byref(h))
        if rc != 0:
            raise VlbError(rc, "vlb_ctx_create failed (is a B200 the current CUDA device?)")
        self.handle = h
        if stream is not None:
            self.set_stream(stream)
        if precision is not None:
            self.set_precision(precision)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.vlb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, stream):
        """stream: integer cudaStream_t handle (e.g. torch.cuda.Stream().cuda_stream) or 0."""
        self.check(self.lib.vlb_ctx_set_stream(self.handle, _P(int(stream))))

    def set_precision(self, p):
        self.check(self.lib.vlb_ctx_set_precision(self.handle, int(p)))

    @property
    def precision(self):
        return self.lib.vlb_ctx_get_precision(self.handle)

    @property
    def launches(self):
        return int(self.lib.vlb_ctx_launch_count(self.handle))

    @property
    def workspace_bytes(self):
        return int(self.lib.vlb_ctx_workspace_bytes(self.handle))

    def reserve_workspace(self, nbytes):
        self.check(self.lib.vlb_ctx_reserve_workspace(self.handle, int(nbytes)))

    def device_status(self):
        """Synchronises and raises VlbError(VLE_Timeout) if a tensor-core kernel gave up a wait."""
        st = C.c_int(0)
        self.check(self.lib.vlb_ctx_device_status(self.handle, C.byref(st)))
        return st.value

    def profile_begin(self):
        self.check(self.lib.vlb_ctx_profile_begin(self.handle))

    def profile_end(self):
        """(milliseconds, algorithmic flops, launches) of the tensor-core kernels since profile_begin."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_longlong()
        self.check(self.lib.vlb_ctx_profile_end(self.handle, C.byref(ms), C.byref(fl), C.byref(n)))
        return ms.value, fl.value, n.value

    def profile_kind(self, kind):
        """(milliseconds, flops, count) of one kind of contraction in the last profile: 0 fprop, 1 dgrad, 2 wgrad, 3 fc."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_longlong()
        self.check(self.lib.vlb_ctx_profile_kind(self.handle, int(kind), C.byref(ms), C.byref(fl), C.byref(n)))
        return ms.value, fl.value, n.value

    def last_error(self):
        return self.lib.vlb_ctx_last_error(self.handle).decode()

    def check(self, rc):
        if rc != 0:
            msg = self.last_error()
            self.lib.vlb_ctx_reset_error(self.handle)
            raise VlbError(rc, msg)
