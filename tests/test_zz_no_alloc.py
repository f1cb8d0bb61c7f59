"""vlb_bnorm_backward_noalloc: batch-norm backward for hosts that may not allocate device memory.

Some callers hand the whole GPU to an allocator of their own, or run where the device-wide
synchronisation of cudaMalloc is not acceptable; they cannot create a context or let its scratch
grow.  This entry point keeps its per-channel scratch in a fixed array inside the library.  The test
calls it through the C ABI twice in a row, with different shapes and data so that anything left in the
shared scratch by the first call would show in the second, and compares each result with the regular
vlb_bnorm_backward.  It also checks that more channels than the built-in scratch holds are refused.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _run_pair(nn, mat, ctx, shape, seed, with_moments):
    import torch
    rng = np.random.default_rng(seed)
    H, W, Cc, N = shape
    x = mat.from_numpy(np.asfortranarray((rng.standard_normal(shape) * 2 + 0.5).astype(np.float32)))
    dy = mat.from_numpy(np.asfortranarray(rng.standard_normal(shape).astype(np.float32)))
    g = mat.from_numpy((rng.standard_normal((Cc, 1)) + 1).astype(np.float32))
    b = mat.from_numpy(rng.standard_normal((Cc, 1)).astype(np.float32))
    eps = 1e-5
    ref = nn.vl_nnbnorm(x, g, b, dy, epsilon=eps)                 # dx, dg, db, moments through vlb_bnorm_backward
    dx, dg, db = mat.empty(shape), mat.empty((Cc, 1)), mat.empty((Cc, 1))
    mom = mat.empty((Cc, 2)) if with_moments else None
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = ctx.lib.vlb_bnorm_backward_noalloc(C.c_void_p(stream), mat.ptr(dx), mat.ptr(dg), mat.ptr(db), mat.ptr(mom),
                                            mat.ptr(x), mat.ptr(g), mat.ptr(dy), H, W, Cc, N, eps, err, 256)
    assert rc == 0, err.value
    torch.cuda.synchronize()
    got = [dx, dg, db] + ([mom] if with_moments else [])
    for a, r, name in zip(got, ref, ("dx", "dg", "db", "moments")):
        # same kernels, same order of operations: the tolerance of the batch-norm parity tests is far from reached
        assert rel_l2(mat.to_numpy(a).ravel(), mat.to_numpy(r).ravel()) < 1e-5, name
        assert np.array_equal(mat.to_numpy(a), mat.to_numpy(r)), name


def test_noalloc_matches_regular_entry_point_twice(gpu):
    nn, mat, ctx = gpu
    _run_pair(nn, mat, ctx, (28, 28, 128, 4), seed=1, with_moments=True)     # vectorised path, moments returned
    _run_pair(nn, mat, ctx, (7, 5, 33, 3), seed=2, with_moments=False)       # scalar path, moments kept in the scratch
    _run_pair(nn, mat, ctx, (8, 8, 16, 2), seed=3, with_moments=False)       # fewer channels than the call before


def test_noalloc_refuses_too_many_channels(gpu):
    nn, mat, ctx = gpu
    Cc = 4097
    x, dy = mat.zeros((1, 1, Cc, 2)), mat.zeros((1, 1, Cc, 2))
    g = mat.zeros((Cc, 1))
    dx, dg, db = mat.empty((1, 1, Cc, 2)), mat.empty((Cc, 1)), mat.empty((Cc, 1))
    err = C.create_string_buffer(256)
    rc = ctx.lib.vlb_bnorm_backward_noalloc(None, mat.ptr(dx), mat.ptr(dg), mat.ptr(db), None, mat.ptr(x), mat.ptr(g),
                                            mat.ptr(dy), 1, 1, Cc, 2, 1e-5, err, 256)
    assert rc == 7 and b"4096" in err.value          # VLE_IllegalArgument with the limit in the message
