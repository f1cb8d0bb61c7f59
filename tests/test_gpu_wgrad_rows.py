"""The filter gradient through the tensor-memory kernel: rows (filter tap, channel), reduction over the output pixels.

For a stride-1 convolution whose output has the input's height, planes of a multiple of 32 pixels and channels in blocks of
32, dF[(fh,fw,c), k] = sum over pixels of x(pixel shifted by the tap, c) * dY(pixel, k) runs with the x rows in tensor
memory -- every row's run of 32 pixels is delivered per k-block by a tensor-map copy that zero-fills what lies left or right
of the image; rows above or below it are masked by the producers -- and dY as pre-split tile images; the reduction is cut
into ranges whose partial results are added in fixed order; planes that are not whole k-blocks are padded (zeros in the
tile images).  Checked here against the CPU checker (double precision) and
against the kernel with both operands in shared memory (test switch bit 2), which every other layer shape still takes:
small planes, 64- and 128-channel tiles with two or four taps per tile, a tap group that is not full, 5x5 and 1x1 filters,
dilation, an output narrower than the input, several ranges, both tensor-core arithmetic modes, run-to-run identical.
"""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

# (H, W, C, N), (FH, FW, C, K), options
CASES = [((8, 4, 32, 3), (3, 3, 32, 16), dict(pad=1)),                # one k-block per image, four taps per tile, 9 taps = 2 1/4 groups
         ((16, 16, 64, 5), (3, 3, 64, 48), dict(pad=1)),              # two taps per tile, the last group half empty
         ((16, 8, 128, 4), (3, 3, 128, 130), dict(pad=1)),            # one tap per tile, two column tiles (the second nearly empty)
         ((32, 32, 256, 2), (3, 3, 256, 64), dict(pad=1)),            # two channel blocks
         ((16, 12, 32, 6), (5, 5, 32, 24), dict(pad=2)),              # 5 x 5: shifts of -2 .. 2 rows
         ((16, 16, 32, 3), (3, 3, 32, 32), dict(pad=(1, 1, 0, 0))),   # no padding left and right: the output is narrower than the input
         ((32, 8, 32, 3), (3, 3, 32, 16), dict(pad=2, dilate=2)),     # dilation
         ((8, 8, 96, 5), (1, 1, 96, 40), dict()),                     # 96 channels: not a tile shape, stays on the other kernel
         ((8, 8, 64, 9), (1, 1, 64, 40), dict()),                     # 1 x 1
         ((56, 56, 64, 8), (3, 3, 64, 64), dict(pad=1)),              # a VGG-like plane, 64-column tiles, many ranges
         ((28, 32, 128, 16), (3, 3, 128, 128), dict(pad=1)),          # rows of 28: row masks at changing places
         ((28, 28, 32, 5), (3, 3, 32, 32), dict(pad=1)),              # planes of 784 pixels: padded to 25 k-blocks per image
         ((12, 20, 64, 3), (3, 3, 64, 16), dict(pad=1)),              # 240 pixels padded to 256
         ((14, 14, 32, 4), (3, 3, 32, 32), dict(pad=1)),              # 196 pixels padded to 224: the most padding the route accepts (1/8)
         ((10, 10, 32, 4), (3, 3, 32, 32), dict(pad=1))]              # 100 pixels would need 128: stays on the other kernel


@pytest.mark.parametrize("precision,tol", [(0, 1e-5), (1, 2e-3)])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_filter_gradient_rows_in_tensor_memory(gpu, oracle, case, precision, tol):
    nn, mat, ctx = gpu
    xs, fs, kw = CASES[case]
    rng = np.random.default_rng(300 + case)
    x = np.asfortranarray(rng.standard_normal(xs).astype(np.float32))
    f = np.asfortranarray((rng.standard_normal(fs) * (2.0 / (fs[0] * fs[1] * fs[2])) ** 0.5).astype(np.float32))
    pad = kw.get("pad", 0)
    pad = (pad,) * 4 if np.isscalar(pad) else pad
    dil = kw.get("dilate", 1)
    Ho = xs[0] + pad[0] + pad[1] - (fs[0] - 1) * dil
    Wo = xs[1] + pad[2] + pad[3] - (fs[1] - 1) * dil
    dy = np.asfortranarray(rng.standard_normal((Ho, Wo, fs[3], xs[3])).astype(np.float32))
    _, dfr, dbr = oracle.conv_backward(x.astype(np.float64), f.astype(np.float64), dy.astype(np.float64), (1, 1), pad, (dil, dil))
    xd, fd, dyd = mat.from_numpy(x), mat.from_numpy(f), mat.from_numpy(dy)
    bd = mat.from_numpy(np.zeros((1, fs[3]), np.float32))
    ctx.set_precision(precision)
    lib = ctx.lib
    try:
        got = {}
        for switch in (0, 8, 4):
            ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, switch))
            _, df, db = nn.vl_nnconv(xd, fd, bd, dyd, no_der_data=True, ctx=ctx, **kw)
            assert ctx.device_status() == 0
            got[switch] = (mat.to_numpy(df), mat.to_numpy(db))
            assert rel_l2(got[switch][0], dfr) < tol, (switch, "df")
            assert rel_l2(got[switch][1].ravel(), dbr.ravel()) < 1e-5, (switch, "db")
        # the running sum of a tile in the drain warps' registers (default) or in shared memory (switch bit 3): same additions
        assert np.array_equal(got[0][0], got[8][0]) and np.array_equal(got[0][1], got[8][1])
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
        _, df2, db2 = nn.vl_nnconv(xd, fd, bd, dyd, no_der_data=True, ctx=ctx, **kw)
        assert np.array_equal(mat.to_numpy(df2), got[0][0]) and np.array_equal(mat.to_numpy(db2), got[0][1])     # no atomics: run to run identical
    finally:
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
        ctx.set_precision(0)


# Fully connected layers with a large weight matrix take the same kernel for all three passes: the forward pass in the row
# mode (rows = filters), the two backward passes as 1 x 1 convolutions over the weight matrix / the input seen as a plane.
FC_CASES = [((4, 4, 512, 64), 256),       # V = 8192, two row tiles of filters, batch 64: 64-column tiles
            ((8, 8, 128, 96), 128),       # batch 96: 128-column tiles, one of them partly empty
            ((4, 4, 512, 40), 384),       # batch 40: the weight gradient (reduction over the batch, not a multiple of 32) stays on the other kernel
            ((2, 2, 2048, 96), 1000)]     # 1000 filters: the forward pass (rows in blocks of 128) stays on the other kernel; two column tiles


@pytest.mark.parametrize("precision,tol", [(0, 1e-5), (1, 2e-3)])
@pytest.mark.parametrize("case", range(len(FC_CASES)))
def test_fully_connected_through_the_tensor_memory_kernel(gpu, oracle, case, precision, tol):
    nn, mat, ctx = gpu
    xs, K = FC_CASES[case]
    rng = np.random.default_rng(400 + case)
    V = xs[0] * xs[1] * xs[2]
    x = np.asfortranarray(rng.standard_normal(xs).astype(np.float32))
    f = np.asfortranarray((rng.standard_normal(xs[:3] + (K,)) * (2.0 / V) ** 0.5).astype(np.float32))
    b = rng.standard_normal(K).astype(np.float32)
    dy = np.asfortranarray(rng.standard_normal((1, 1, K, xs[3])).astype(np.float32))
    x64, f64, dy64 = x.astype(np.float64), f.astype(np.float64), dy.astype(np.float64)
    yr = oracle.fc_forward(x64, f64, b.astype(np.float64))
    dxr, dfr, dbr = oracle.fc_backward(x64, f64, dy64)
    xd, fd, bd, dyd = mat.from_numpy(x), mat.from_numpy(f), mat.from_numpy(b.reshape(1, -1)), mat.from_numpy(dy)
    ctx.set_precision(precision)
    lib = ctx.lib
    try:
        first = None
        for switch in (0, 4, 0):
            ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, switch))
            y = mat.to_numpy(nn.vl_nnconv(xd, fd, bd, ctx=ctx))
            yrelu = mat.to_numpy(nn.vl_nnconv(xd, fd, bd, relu=True, ctx=ctx))
            dx, df, db = (mat.to_numpy(a) for a in nn.vl_nnconv(xd, fd, bd, dyd, ctx=ctx))
            assert ctx.device_status() == 0
            assert rel_l2(y, yr) < tol and rel_l2(dx, dxr) < tol and rel_l2(df, dfr) < tol and rel_l2(db.ravel(), dbr.ravel()) < 1e-5, switch
            assert np.array_equal(yrelu, np.maximum(y, 0))
            if switch == 0 and first is None:
                first = (y, dx, df)
            elif switch == 0:
                assert all(np.array_equal(a, c) for a, c in zip(first, (y, dx, df)))      # run to run identical
    finally:
        ctx.check(lib.vlb_ctx_set_test_switch(ctx.handle, 0))
        ctx.set_precision(0)
