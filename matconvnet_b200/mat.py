"""MATLAB-order tensors on the device.

A "mat tensor" is a torch tensor whose logical shape is (H, W, C, N) -- or any
MATLAB shape -- and whose memory is column-major (first index fastest), the
layout of vl::Tensor in the reference (bits/data.cu:498-505).  It is made by
allocating the reversed shape contiguously and permuting the view, so indexing
reads like MATLAB (0-based) while the bytes are what the C ABI expects.
"""
import numpy as np
import torch


def _rev(n):
    return tuple(range(n - 1, -1, -1))


def empty(shape, device="cuda", dtype=torch.float32):
    shape = tuple(int(s) for s in shape)
    return torch.empty(shape[::-1], device=device, dtype=dtype).permute(_rev(len(shape)))


def zeros(shape, device="cuda", dtype=torch.float32):
    shape = tuple(int(s) for s in shape)
    return torch.zeros(shape[::-1], device=device, dtype=dtype).permute(_rev(len(shape)))


def is_mat(t):
    return t.permute(_rev(t.dim())).is_contiguous()


def as_mat(t):
    """Returns t if it is already column-major, else a column-major copy."""
    if is_mat(t):
        return t
    out = empty(t.shape, t.device, t.dtype)
    out.copy_(t)
    return out


def from_numpy(a, device="cuda", dtype=torch.float32):
    """numpy array (any order) -> column-major device tensor of the same logical shape."""
    a = np.asarray(a)
    t = torch.from_numpy(np.ascontiguousarray(a.T)).to(device=device, dtype=dtype)
    return t.permute(_rev(a.ndim))


def to_numpy(t):
    """Column-major device tensor -> Fortran-ordered numpy array of the same logical shape."""
    t = as_mat(t)
    return t.permute(_rev(t.dim())).contiguous().cpu().numpy().T


def ptr(t):
    return None if t is None else t.data_ptr()


def shape4(t):
    """MATLAB size(t, 1..4): trailing dimensions folded into the 4th, missing ones are 1
    (TensorShape::reshape(4), reference bits/data.cu:585-601)."""
    s = list(t.shape)
    while len(s) < 4:
        s.append(1)
    if len(s) > 4:
        s = s[:3] + [int(np.prod(s[3:]))]
    return tuple(int(v) for v in s)
