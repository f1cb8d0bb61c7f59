"""matconvnet_b200: a B200 (sm_100a) engine behind MatConvNet's operator API.

``capi``  -- ctypes binding of the C ABI declared in include/vlb.h (libvlb.so).
``mat``   -- helpers for MATLAB-order (H x W x C x N, H fastest) device tensors.
``nn``    -- the building blocks with the reference's call signatures
             (vl_nnconv, vl_nnbnorm, vl_nnpool, vl_nnroipool, vl_nnbilinearsampler,
             vl_nnrelu, vl_nnsoftmaxloss).
``simplenn`` / ``dataparallel`` -- linear-chain forward/backward in the reference's
             schedule and the NCCL gradient exchange that replaces its parameter server.

There is no CPU implementation in this package: importing ``capi`` without a built
libvlb.so raises, and every operator requires CUDA tensors.
"""
__version__ = "0.1.0"
