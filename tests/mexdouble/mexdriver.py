"""Calls the reference's MEX gateways, built over the vlb engine, the way MATLAB would (TEST INFRASTRUCTURE ONLY).

    mex = MexDouble()                      # loads tests/mexdouble/_build/*.so
    y = mex.call("vl_nnconv", 1, gpu(x), gpu(f), gpu(b), "Stride", [2, 2], "Pad", 1)

Arguments: GpuArray(numpy array) is uploaded as a single gpuArray in MATLAB order; a numpy array stays a plain array of
its dtype (float32 -> single, float64 -> double); a str becomes a char row; numbers and lists become double row vectors,
as typed at the MATLAB prompt.  Results come back as numpy arrays in MATLAB order.  A gateway error (mexErrMsgTxt)
raises MexError carrying MATLAB's message.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")

# mxClassID values of the stand-in's matrix.h (the same as MATLAB's)
CLASS = {np.dtype(np.float64): 6, np.dtype(np.float32): 7, np.dtype(np.int32): 12, np.dtype(np.bool_): 3}
DTYPE = {v: k for k, v in CLASS.items()}
DTYPE[4] = np.dtype(np.uint16)          # char
GATEWAY = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p))


class MexError(RuntimeError):
    pass


class GpuArray:
    """Marks a numpy array to be passed as a gpuArray."""
    def __init__(self, array):
        self.array = np.asarray(array)


def gpu(array):
    return GpuArray(array)


class MexDouble:
    def __init__(self):
        common = os.path.join(OUT, "libmexdouble.so")
        if not os.path.exists(common):
            raise RuntimeError("the MEX test double is not built: run tests/mexdouble/build_mexdouble.py where the reference is")
        self.lib = L = ctypes.CDLL(common)      # local scope: the checker loads the reference's CPU build of the same classes
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        L.mxd_from_host.restype = vp
        L.mxd_from_host.argtypes = [vp, ctypes.c_int, ctypes.POINTER(sz), ctypes.c_int, ctypes.c_int]
        L.mxd_to_host.restype = ctypes.c_int
        L.mxd_to_host.argtypes = [vp, vp]
        L.mxd_call.restype = ctypes.c_int
        L.mxd_call.argtypes = [vp, ctypes.c_int, ctypes.POINTER(vp), ctypes.c_int, ctypes.POINTER(vp), ctypes.c_char_p, sz]
        L.mxCreateString.restype = vp
        L.mxCreateString.argtypes = [ctypes.c_char_p]
        L.mxDestroyArray.argtypes = [vp]
        L.mxGetClassID.restype = ctypes.c_int
        L.mxGetClassID.argtypes = [vp]
        L.mxGetNumberOfDimensions.restype = sz
        L.mxGetNumberOfDimensions.argtypes = [vp]
        L.mxGetDimensions.restype = ctypes.POINTER(sz)
        L.mxGetDimensions.argtypes = [vp]
        L.mxIsGPUArray.restype = ctypes.c_bool
        L.mxIsGPUArray.argtypes = [vp]
        L.mxd_warnings.restype = ctypes.c_char_p
        L.vlb_functors_launch_count.restype = ctypes.c_longlong
        self.gateways = {}

    def gateway(self, name):
        if name not in self.gateways:
            lib = ctypes.CDLL(os.path.join(OUT, name + ".so"))
            self.gateways[name] = (lib, ctypes.cast(lib.mexFunction, ctypes.c_void_p))
        return self.gateways[name][1]

    # ------------------------------------------------------------------ arguments
    def _array(self, a, on_gpu):
        a = np.asarray(a)
        if a.dtype not in CLASS:
            raise TypeError("no MATLAB class for dtype %s" % a.dtype)
        flat = np.ascontiguousarray(a.ravel(order="F"))
        shape = a.shape if a.ndim >= 2 else ((1, a.size) if a.ndim == 1 else (1, 1))
        dims = (ctypes.c_size_t * len(shape))(*shape)
        h = self.lib.mxd_from_host(flat.ctypes.data_as(ctypes.c_void_p), len(shape), dims, CLASS[a.dtype], int(on_gpu))
        if not h:
            raise MemoryError("could not create a %s array of shape %s" % ("gpu" if on_gpu else "host", shape))
        return h

    def to_mx(self, v):
        if isinstance(v, GpuArray):
            return self._array(v.array.astype(np.float32, copy=False), True)
        if isinstance(v, str):
            return self.lib.mxCreateString(v.encode())
        if isinstance(v, np.ndarray):
            return self._array(v, False)
        if isinstance(v, bool):
            return self._array(np.array([[v]], dtype=np.bool_), False)
        return self._array(np.atleast_2d(np.asarray(v, dtype=np.float64)), False)

    def from_mx(self, h):
        L = self.lib
        nd = L.mxGetNumberOfDimensions(h)
        dims = tuple(int(L.mxGetDimensions(h)[i]) for i in range(nd))
        out = np.empty(dims, dtype=DTYPE[L.mxGetClassID(h)], order="F")
        if out.size:
            status = L.mxd_to_host(h, out.ctypes.data_as(ctypes.c_void_p))
            if status:
                raise MexError("reading a result back failed with CUDA error %d" % status)
        return out

    # ------------------------------------------------------------------ the call
    def call(self, name, nout, *args, with_placement=False):
        """[out1, ..., out_nout] = name(args...).  Returns one array when nout == 1, else a list; with_placement=True
        returns (results, [True where the result is a gpuArray])."""
        L = self.lib
        fn = self.gateway(name)
        rhs = [self.to_mx(a) for a in args]
        rhs_arr = (ctypes.c_void_p * max(len(rhs), 1))(*rhs)
        # MATLAB hands a gateway room for at least one output even when nargout is 0
        lhs_arr = (ctypes.c_void_p * max(nout, 1))()
        err = ctypes.create_string_buffer(4096)
        try:
            failed = L.mxd_call(fn, nout, lhs_arr, len(rhs), rhs_arr, err, len(err))
            if failed:
                raise MexError(err.value.decode(errors="replace"))
            handles = [lhs_arr[i] for i in range(max(nout, 1)) if lhs_arr[i]]
            outs = [self.from_mx(h) for h in handles]
            placement = [bool(L.mxIsGPUArray(h)) for h in handles]
            for h in handles:
                L.mxDestroyArray(h)
        finally:
            for h in rhs:
                L.mxDestroyArray(h)
        outs = outs[:nout] if nout else outs[:1]
        res = outs[0] if nout <= 1 else outs
        return (res, placement) if with_placement else res

    def launches(self):
        """Kernels the engine has enqueued on behalf of the gateways so far."""
        return int(self.lib.vlb_functors_launch_count())

    def close(self):
        """What clearing the MEX files does: their at-exit handlers, then the engine contexts."""
        self.lib.mxd_run_at_exit()
        self.lib.vlb_functors_release()
