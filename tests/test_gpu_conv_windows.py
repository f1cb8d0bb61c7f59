"""The tensor-memory convolution kernel fed by tensor-map copies against the same kernel fed by per-thread loads.

Where the geometry allows (unit stride, channels a multiple of 32, rows a multiple of four elements, an output map that
boxes of up to 128 pixels cover almost exactly) the forward convolution and the stride-1 data gradient take their input windows
from shared memory, filled by cp.async.bulk.tensor copies that zero-fill the padding; elsewhere, and when test switch
bit 1 of the context is set, the producer threads gather the windows from global memory themselves.  Both routes feed the
same k-blocks to the same accumulation chains, so the results must agree bit for bit -- on full boxes, on boxes that
hang over the right edge of the map, with dilation, with 5x5 and 1x1 filters, with
the fused ReLU in both directions, in both tensor-core arithmetic modes.  (The kernel itself is checked against the CPU
reference by the other convolution tests, which now run through the tensor-map route wherever it applies.)
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# (H, W, C, N), (FH, FW, C, K), options
CASES = [((32, 32, 32, 5), (3, 3, 32, 48), dict(pad=1)),             # boxes of 32 x 4, several row tiles per image
         ((64, 48, 64, 6), (3, 3, 64, 128), dict(pad=1)),            # more tiles than SMs: every CTA walks several
         ((56, 56, 64, 3), (3, 3, 64, 64), dict(pad=1)),             # 112 of 128 rows would be in use: both sides gather
         ((64, 62, 32, 3), (3, 3, 32, 40), dict(pad=1)),             # boxes of 64 x 2 (31 column tiles)
         ((32, 31, 32, 3), (3, 3, 32, 40), dict(pad=1)),             # boxes of 32 x 4, the last one hanging over the right edge
         ((16, 24, 32, 7), (5, 5, 32, 32), dict(pad=2)),             # 5 x 5 filters
         ((32, 16, 32, 2), (3, 3, 32, 16), dict(pad=2, dilate=2)),   # dilation
         ((28, 28, 128, 9), (1, 1, 128, 64), dict()),                # 1 x 1: one tap per window
         ((112, 112, 32, 2), (3, 3, 32, 64), dict(pad=1))]           # boxes of 16 x 8


@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_tensor_map_route_equals_the_per_thread_gather(gpu, case, precision):
    import torch
    nn, mat, ctx = gpu
    xs, fs, kw = CASES[case]
    g = torch.Generator(device="cuda").manual_seed(100 + case)
    x = mat.as_mat(torch.randn(*xs, device="cuda", generator=g))
    f = mat.as_mat(torch.randn(*fs, device="cuda", generator=g) * (2.0 / (fs[0] * fs[1] * fs[2])) ** 0.5)
    b = mat.as_mat(torch.randn(1, fs[3], device="cuda", generator=g))
    ctx.set_precision(precision)
    lib = ctx.lib
    try:
        out = {}
        for switch in (2, 0):
            ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, switch))
            y = nn.vl_nnconv(x, f, b, ctx=ctx, **kw)
            yr = nn.vl_nnconv(x, f, b, relu=True, ctx=ctx, **kw)
            dy = mat.as_mat(torch.randn(*y.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)))
            dx, df, db = nn.vl_nnconv(x, f, b, dy, ctx=ctx, **kw)
            xr = nn.vl_nnrelu(x, ctx=ctx)
            dxm, _, _ = nn.vl_nnconv(xr, f, b, dy, through_relu=True, no_der_filters=True, no_der_biases=True, ctx=ctx, **kw)
            assert ctx.device_status() == 0
            out[switch] = (y, yr, dx, dxm)
        for a, c in zip(out[2], out[0]):
            assert torch.equal(a, c)
        assert torch.equal(out[0][1], torch.clamp(out[0][0], min=0))
    finally:
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
        ctx.set_precision(0)


@pytest.mark.parametrize("case", [0, 1, 2, 7])
def test_running_sum_in_registers_equals_running_sum_in_shared_memory(gpu, case):
    """The drain warps keep the fp32 running sum of a 64- or 128-column tile in registers (taken over from the issuing warps
    with setmaxnreg); test switch bit 3 keeps it in shared memory, as narrower tiles and very short tiles do.  Same additions in
    the same order: equal results, forward, data gradient (with the fused ReLU mask) and filter gradient."""
    import torch
    nn, mat, ctx = gpu
    xs, fs, kw = CASES[case]
    g = torch.Generator(device="cuda").manual_seed(200 + case)
    x = mat.as_mat(torch.randn(*xs, device="cuda", generator=g))
    f = mat.as_mat(torch.randn(*fs, device="cuda", generator=g) * (2.0 / (fs[0] * fs[1] * fs[2])) ** 0.5)
    b = mat.as_mat(torch.randn(1, fs[3], device="cuda", generator=g))
    lib = ctx.lib
    try:
        out = {}
        for switch in (8, 0):
            ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, switch))
            y = nn.vl_nnconv(x, f, b, ctx=ctx, **kw)
            dy = mat.as_mat(torch.randn(*y.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)))
            dx, df, db = nn.vl_nnconv(x, f, b, dy, ctx=ctx, **kw)
            xr = nn.vl_nnrelu(x, ctx=ctx)
            dxm, _, _ = nn.vl_nnconv(xr, f, b, dy, through_relu=True, no_der_filters=True, no_der_biases=True, ctx=ctx, **kw)
            assert ctx.device_status() == 0
            out[switch] = (y, dx, df, dxm)
        for a, c in zip(out[8], out[0]):
            assert torch.equal(a, c)
    finally:
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
