"""CUDA kernels, called through the C ABI, against the CPU checker on the same seeded inputs
and against the golden vectors of the reference's compiled CPU backend.

Bars: bit-exact for max-pool routing, pooling values, ROI bin geometry and (with
integer-valued gradients, whose sums are exact in any order) ROI / sampler scatter;
relative L2 <= 1e-5 for convolution, fully-connected and batch-norm results in the default
(3xTF32) arithmetic and for the CUDA-core fp32 path; <= 2e-3 for the plain-TF32 fast path.
"""
import numpy as np
import pytest

from conftest import bit_equal, cases_of, load_golden, rel_l2

pytestmark = pytest.mark.gpu

TOL_FAITHFUL = 1e-5     # 3xTF32 and fp32 paths
TOL_TF32 = 2e-3         # single-pass TF32 path


def _up(mat, *arrays):
    return [None if a is None else mat.from_numpy(a) for a in arrays]


# ------------------------------------------------------------------ pooling
def test_pool_golden(gpu):
    nn, mat, _ = gpu
    g = load_golden("pool")
    for c in cases_of(g):
        if c == "ties":
            continue
        prm = g[c + ".prm"]
        kw = dict(stride=tuple(prm[2:4]), pad=tuple(prm[4:8]))
        (x,) = _up(mat, g[c + ".x"])
        for m in ("max", "avg"):
            y = nn.vl_nnpool(x, tuple(prm[0:2]), method=m, **kw)
            assert bit_equal(mat.to_numpy(y), g["%s.%s.y" % (c, m)]), (c, m, "y")
            (dy,) = _up(mat, g["%s.%s.dy" % (c, m)])
            dx = nn.vl_nnpool(x, tuple(prm[0:2]), dy, method=m, **kw)
            assert bit_equal(mat.to_numpy(dx), g["%s.%s.dx" % (c, m)]), (c, m, "dx")
    x, dy = _up(mat, g["ties.x"], g["ties.dy"])
    assert bit_equal(mat.to_numpy(nn.vl_nnpool(x, (2, 2), stride=2)), g["ties.max.y"])
    assert bit_equal(mat.to_numpy(nn.vl_nnpool(x, (2, 2), dy, stride=2)), g["ties.max.dx"])


@pytest.mark.parametrize("shape,pool,stride,pad", [
    ((224, 224, 4, 2), (2, 2), (2, 2), (0, 0, 0, 0)),       # VGG pool1 geometry
    ((14, 14, 64, 3), (2, 2), (2, 2), (0, 0, 0, 0)),        # VGG pool5 geometry (H % 4 != 0)
    ((32, 32, 8, 5), (3, 3), (2, 2), (0, 1, 0, 1)),         # CIFAR overlapping, asymmetric pad
    ((24, 24, 20, 10), (2, 2), (2, 2), (0, 0, 0, 0)),       # LeNet
    ((13, 17, 3, 2), (4, 3), (3, 2), (1, 2, 2, 0)),
    ((5, 5, 2, 2), (5, 5), (1, 1), (0, 0, 0, 0)),           # one window = whole map
])
@pytest.mark.parametrize("method", ["max", "avg"])
def test_pool_vs_oracle(gpu, oracle, shape, pool, stride, pad, method):
    nn, mat, _ = gpu
    rng = np.random.default_rng(11)
    x = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
    y_ref = oracle.pool_forward(x, pool, stride, pad, method)
    dy = np.asfortranarray(rng.standard_normal(y_ref.shape).astype(np.float32))
    xd, dyd = _up(mat, x, dy)
    assert bit_equal(mat.to_numpy(nn.vl_nnpool(xd, pool, stride=stride, pad=pad, method=method)), y_ref)
    dx = nn.vl_nnpool(xd, pool, dyd, stride=stride, pad=pad, method=method)
    assert bit_equal(mat.to_numpy(dx), oracle.pool_backward(x, dy, pool, stride, pad, method))


def test_pool_rejects_bad_arguments(gpu):
    nn, mat, _ = gpu
    from matconvnet_b200.capi import VlbError
    x = mat.zeros((8, 8, 1, 1))
    with pytest.raises(VlbError):
        nn.vl_nnpool(x, (2, 2), pad=2)            # padding >= window
    with pytest.raises(VlbError):
        nn.vl_nnpool(x, (9, 9))                   # window larger than input


# ------------------------------------------------------------------ batch normalisation
def test_bnorm_golden(gpu):
    nn, mat, _ = gpu
    g = load_golden("bnorm")
    for c in cases_of(g):
        x, gg, b, dy = _up(mat, g[c + ".x"], g[c + ".g"], g[c + ".b"], g[c + ".dy"])
        eps = float(g[c + ".eps"])
        y, mom = nn.vl_nnbnorm(x, gg, b, epsilon=eps)
        assert rel_l2(mat.to_numpy(y), g[c + ".y64"]) < TOL_FAITHFUL, c
        assert rel_l2(mat.to_numpy(mom), g[c + ".mom64"]) < TOL_FAITHFUL, c
        assert rel_l2(mat.to_numpy(y), g[c + ".y"]) < TOL_FAITHFUL, c
        dx, dg, db, mom2 = nn.vl_nnbnorm(x, gg, b, dy, epsilon=eps)
        for got, name in ((dx, "dx"), (dg, "dg"), (db, "db")):
            assert rel_l2(mat.to_numpy(got).ravel(), g[c + "." + name + "64"].ravel()) < TOL_FAITHFUL, (c, name)
            assert rel_l2(mat.to_numpy(got).ravel(), g[c + "." + name].ravel()) < TOL_FAITHFUL, (c, name)
        assert rel_l2(mat.to_numpy(mom2), g[c + ".mom64"]) < TOL_FAITHFUL, c
        (momd,) = _up(mat, g[c + ".mom"])
        dxm, dgm, dbm, _ = nn.vl_nnbnorm(x, gg, b, dy, epsilon=eps, moments=momd)
        for got, name in ((dxm, "dxm"), (dgm, "dgm"), (dbm, "dbm")):
            assert rel_l2(mat.to_numpy(got).ravel(), g[c + "." + name].ravel()) < TOL_FAITHFUL, (c, name)
        ym, _ = nn.vl_nnbnorm(x, gg, b, epsilon=eps, moments=momd)
        assert bit_equal(mat.to_numpy(ym), g[c + ".ym"]), c       # same arithmetic, element-wise


@pytest.mark.parametrize("shape", [(28, 28, 128, 8), (28, 28, 512, 2), (7, 7, 33, 5), (1, 1, 10, 3), (64, 64, 32, 4)])
def test_bnorm_vs_oracle(gpu, oracle, shape):
    nn, mat, _ = gpu
    rng = np.random.default_rng(12)
    x = np.asfortranarray((rng.standard_normal(shape) * 1.5 + 0.3).astype(np.float32))
    dy = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
    g = (rng.standard_normal(shape[2]) + 1).astype(np.float32)
    b = rng.standard_normal(shape[2]).astype(np.float32)
    x64, dy64, g64, b64 = (a.astype(np.float64) for a in (x, dy, g, b))
    ref = oracle.bnorm_backward(x64, g64, b64, dy64, 1e-5)          # double instantiation
    xd, dyd, gd, bd = _up(mat, x, dy, g, b)
    got = nn.vl_nnbnorm(xd, gd, bd, dyd, epsilon=1e-5)
    for a, r, name in zip(got, ref, ("dx", "dg", "db", "moments")):
        assert rel_l2(mat.to_numpy(a).ravel(), r.ravel()) < TOL_FAITHFUL, name
    # given moments == computed moments (reference xtest/suite/nnbnorm.m:53-79)
    got2 = nn.vl_nnbnorm(xd, gd, bd, dyd, epsilon=1e-5, moments=got[3])
    for a, r in zip(got2[:3], got[:3]):
        assert rel_l2(mat.to_numpy(a).ravel(), mat.to_numpy(r).ravel()) < 1e-6
    # run-to-run determinism: no atomics anywhere in this block
    again = nn.vl_nnbnorm(xd, gd, bd, dyd, epsilon=1e-5)
    for a, r in zip(again, got):
        assert bit_equal(mat.to_numpy(a), mat.to_numpy(r))
    y, mom = nn.vl_nnbnorm(xd, gd, bd, epsilon=1e-5)
    yr, momr = oracle.bnorm_forward(x64, g64, b64, 1e-5)
    assert rel_l2(mat.to_numpy(y), yr) < TOL_FAITHFUL and rel_l2(mat.to_numpy(mom), momr) < TOL_FAITHFUL


# ------------------------------------------------------------------ bias, relu, loss
def test_bias_golden(gpu):
    nn, mat, ctx = gpu
    g = load_golden("bias")
    H, W, K, N = g["y0"].shape
    lib = ctx.lib
    for i, (ym, hx, xm, hb, bm) in enumerate(g["fwd_args"]):
        y, x, b = _up(mat, g["y0"], g["x"] if hx else None, g["b"] if hb else None)
        ctx.check(lib.vlb_bias_forward(ctx.handle, mat.ptr(y), ym, mat.ptr(x), xm, mat.ptr(b), bm, H, W, K, N))
        assert bit_equal(mat.to_numpy(y), g["fwd%d" % i]), i
    for i, (dxm, dbm, xm, bm) in enumerate(g["bwd_args"]):
        dx, db, dy = _up(mat, g["dx0"], g["db0"], g["dy"])
        ctx.check(lib.vlb_bias_backward(ctx.handle, mat.ptr(dx), dxm, mat.ptr(db), dbm, xm, bm, mat.ptr(dy), H, W, K, N))
        assert bit_equal(mat.to_numpy(dx), g["bwd%d.dx" % i]), i
        assert rel_l2(mat.to_numpy(db), g["bwd%d.db" % i]) < 1e-6, i


def test_relu_and_loss(gpu, oracle):
    nn, mat, _ = gpu
    rng = np.random.default_rng(13)
    for shape in [(7, 5, 3, 2), (16, 16, 8, 4), (1, 1, 1000, 64)]:
        x = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
        x.reshape(-1, order="F")[::7] = 0.0
        dy = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
        xd, dyd = _up(mat, x, dy)
        assert bit_equal(mat.to_numpy(nn.vl_nnrelu(xd)), oracle.relu_forward(x))
        assert bit_equal(mat.to_numpy(nn.vl_nnrelu(xd, dyd)), oracle.relu_backward(x, dy))
    for shape in [(1, 1, 1000, 64), (1, 1, 10, 100), (3, 2, 5, 4)]:
        x = np.asfortranarray((rng.standard_normal(shape) * 3).astype(np.float32))
        lab = rng.integers(1, shape[2] + 1, size=shape[3]).astype(np.float32)
        xd, labd = _up(mat, x, lab)
        loss = float(nn.vl_nnsoftmaxloss(xd, labd).cpu()[0])
        ref = float(oracle.softmaxloss_forward(x.astype(np.float64), lab.astype(np.float64)))
        assert abs(loss - ref) <= 1e-5 * abs(ref)
        dx = nn.vl_nnsoftmaxloss(xd, labd, 1.0)
        assert rel_l2(mat.to_numpy(dx), oracle.softmaxloss_backward(x.astype(np.float64), lab.astype(np.float64), 1.0)) < TOL_FAITHFUL
    # class 0 skips an image, first image included (matlab/vl_nnsoftmaxloss.m:55-67)
    x = np.asfortranarray((rng.standard_normal((2, 2, 7, 5)) * 3).astype(np.float32))
    lab = np.array([0, 3, 7, 0, 1], np.float32)
    xd, labd = _up(mat, x, lab)
    loss = float(nn.vl_nnsoftmaxloss(xd, labd).cpu()[0])
    ref = float(oracle.softmaxloss_forward(x.astype(np.float64), lab.astype(np.float64)))
    assert abs(loss - ref) <= 1e-5 * abs(ref)
    dx = mat.to_numpy(nn.vl_nnsoftmaxloss(xd, labd, 0.5))
    assert rel_l2(dx, oracle.softmaxloss_backward(x.astype(np.float64), lab.astype(np.float64), 0.5)) < TOL_FAITHFUL
    assert np.all(dx[:, :, :, 0] == 0) and np.all(dx[:, :, :, 3] == 0)


def test_softmaxloss_label_above_the_class_count_is_reported(gpu):
    """An indexing error in the reference (x(c_) out of range); here the image is skipped, nothing is read out of range,
    and the context's status word makes the next vlb_ctx_device_status return VLE_IllegalArgument."""
    from matconvnet_b200 import capi
    nn, mat, ctx = gpu
    x = mat.from_numpy(np.zeros((1, 1, 4, 3), np.float32))
    lab = mat.from_numpy(np.array([1, 9, 2], np.float32))
    nn.vl_nnsoftmaxloss(x, lab)
    with pytest.raises(capi.VlbError) as err:
        ctx.device_status()
    assert err.value.code == capi.ERROR_NAMES.index("VLE_IllegalArgument")
    assert ctx.device_status() == 0          # the word was cleared


# ------------------------------------------------------------------ ROI pooling
def test_roipool_golden(gpu):
    nn, mat, _ = gpu
    g = load_golden("roipool")
    (x,) = _up(mat, g["x"])
    keys = sorted({k[:-2] for k in g if k.endswith(".y")})
    for key in keys:
        tname, sub, method = key.split(".")
        sub = tuple(int(v) for v in sub.split("x"))
        (rois,) = _up(mat, g["rois." + tname])
        tf = g["tf." + tname]
        y = nn.vl_nnroipool(x, rois, subdivisions=sub, transform=tf, method=method)
        assert bit_equal(mat.to_numpy(y), g[key + ".y"]), key
        (dyi,) = _up(mat, g[key + ".dyi"])
        dxi = nn.vl_nnroipool(x, rois, dyi, subdivisions=sub, transform=tf, method=method)
        # the backward pass gathers in the CPU loop's order (ROI, bin column, bin row): bit for bit, integer-valued or not
        assert bit_equal(mat.to_numpy(dxi), g[key + ".dxi"]), key
        (dy,) = _up(mat, g[key + ".dy"])
        dx = nn.vl_nnroipool(x, rois, dy, subdivisions=sub, transform=tf, method=method)
        assert bit_equal(mat.to_numpy(dx), g[key + ".dx"]), key


def test_roipool_bins_bit_exact(gpu, oracle):
    """Every (roi, ph, pw) bin of the Fast R-CNN head geometry, feature-map and image coordinates."""
    nn, mat, _ = gpu
    rng = np.random.default_rng(14)
    H, W, N, K = 38, 50, 2, 256
    for transform, scale in ((1.0, 1.0), (1.0 / 16, 16.0), ([0.97, 0.02, -0.03, 1.04, 0.4, -0.6], 1.0)):
        u1 = rng.uniform(1, W - 2, K); v1 = rng.uniform(1, H - 2, K)
        u2 = u1 + rng.uniform(2, W, K); v2 = v1 + rng.uniform(2, H, K)
        rois = np.stack([rng.integers(1, N + 1, K), u1 * scale, v1 * scale, np.minimum(u2, W) * scale,
                         np.minimum(v2, H) * scale]).astype(np.float32)
        rois = np.asfortranarray(rois)
        for sub in [(7, 7), (6, 6), (1, 1), (16, 16)]:
            bref, iref = oracle.roipool_bounds(rois, (H, W, 512, N), sub, transform)
            (rd,) = _up(mat, rois)
            b, im = nn.roipool_bounds(rd, (H, W, 512, N), sub, transform)
            assert np.array_equal(mat.to_numpy(b), bref), (transform, sub)
            assert np.array_equal(im.cpu().numpy(), iref)


def test_roipool_identity(gpu):
    nn, mat, _ = gpu
    x = np.asfortranarray((np.arange(2, 11)[:, None] * np.arange(1, 11)[None, :]).astype(np.float32)).reshape(9, 10, 1, 1, order="F")
    rois = np.array([[1, 1, 1, 9, 10]], np.float32).T
    xd, rd = _up(mat, x, rois)
    for m in ("max", "avg"):
        y = nn.vl_nnroipool(xd, rd, subdivisions=(9, 10), transform=np.array([[0, 1, 0], [1, 0, 0]], float), method=m)
        assert np.array_equal(mat.to_numpy(y), x)


# ------------------------------------------------------------------ bilinear sampler
def test_sampler_golden(gpu):
    nn, mat, _ = gpu
    g = load_golden("sampler")
    for c in cases_of(g):
        x, grid, dy = _up(mat, g[c + ".x"], g[c + ".grid"], g[c + ".dy"])
        assert bit_equal(mat.to_numpy(nn.vl_nnbilinearsampler(x, grid)), g[c + ".y"]), c
        dx, dgrid = nn.vl_nnbilinearsampler(x, grid, dy)
        assert bit_equal(mat.to_numpy(dgrid), g[c + ".dgrid"]), c
        assert rel_l2(mat.to_numpy(dx), g[c + ".dx"]) < 1e-6, c


def test_sampler_affine_vs_oracle(gpu, oracle):
    """Small rotations and scales through the affine-grid formula of the reference
    (matlab/+dagnn/AffineGridGenerator.m:36-57,106-118), two grids per image."""
    nn, mat, _ = gpu
    rng = np.random.default_rng(15)
    H = W = 16; C = 5; N = 3; Ng = 6
    xi = np.linspace(-1, 1, H); yi = np.linspace(-1, 1, W)
    yy, xx = np.meshgrid(xi, yi)
    base = np.stack([yy.ravel(), xx.ravel()], 1)                    # (Wo*Ho) x 2
    grid = np.zeros((2, H, W, Ng), np.float32, order="F")
    for n in range(Ng):
        th, s = rng.uniform(-0.2, 0.2), rng.uniform(0.8, 1.2)
        A = s * np.array([[np.cos(th), -np.sin(th)], [np.sin(th), np.cos(th)]])
        t = rng.uniform(-0.1, 0.1, 2)
        gpts = base @ A + t
        grid[:, :, :, n] = gpts.reshape(W, H, 2).transpose(2, 1, 0)
    x = np.asfortranarray(rng.standard_normal((H, W, C, N)).astype(np.float32))
    y_ref = oracle.sampler_forward(x, grid)
    dy = np.asfortranarray(rng.integers(-4, 5, y_ref.shape).astype(np.float32))
    xd, gd, dyd = _up(mat, x, grid, dy)
    assert bit_equal(mat.to_numpy(nn.vl_nnbilinearsampler(xd, gd)), y_ref)
    dx, dgrid = nn.vl_nnbilinearsampler(xd, gd, dyd)
    dxr, dgr = oracle.sampler_backward(x, grid, dy)
    assert bit_equal(mat.to_numpy(dgrid), dgr)
    assert rel_l2(mat.to_numpy(dx), dxr) < 1e-6


def test_sampler_backward_gather_paths(gpu, oracle):
    """The data gradient's three routes against the checker: the shared-memory gather with the channels of an image
    shared out among several CTAs (few images; channel count not a multiple of the inner block; two grids per image) --
    bit for bit, real-valued derivatives; a grid that piles every tap on a few input pixels (lists too long: atomic
    scatter inside the gather kernel); planes too large for the lists (the scatter kernel).  The last two with
    integer-valued derivatives, whose sums are exact in any order."""
    import torch
    nn, mat, _ = gpu
    rng = np.random.default_rng(17)
    # 1: gather, chunked channels, grouped grids
    H, W, C, N, Ng, Ho, Wo = 12, 20, 13, 3, 6, 16, 8
    x = np.asfortranarray(rng.standard_normal((H, W, C, N)).astype(np.float32))
    grid = np.asfortranarray(rng.uniform(-1.1, 1.1, (2, Ho, Wo, Ng)).astype(np.float32))
    dy = np.asfortranarray(rng.standard_normal((Ho, Wo, C, Ng)).astype(np.float32))
    xd, gd, dyd = _up(mat, x, grid, dy)
    dx, dgrid = nn.vl_nnbilinearsampler(xd, gd, dyd)
    dxr, dgr = oracle.sampler_backward(x, grid, dy)
    assert bit_equal(mat.to_numpy(dx), dxr) and bit_equal(mat.to_numpy(dgrid), dgr)
    dx2, _ = nn.vl_nnbilinearsampler(xd, gd, dyd)
    assert torch.equal(dx, dx2)
    # 1b: planes whose sizes are not multiples of four (the stages are filled with 4-byte copies), five channels (a full
    # stage of four and a stage of one for the data gradient; two stages of two and one of one for the grid derivative),
    # more input than output pixels
    H, W, C, N, Ng, Ho, Wo = 7, 9, 5, 150, 150, 5, 7
    xb = np.asfortranarray(rng.standard_normal((H, W, C, N)).astype(np.float32))
    gridb = np.asfortranarray(rng.uniform(-1.05, 1.05, (2, Ho, Wo, Ng)).astype(np.float32))
    dyb = np.asfortranarray(rng.standard_normal((Ho, Wo, C, Ng)).astype(np.float32))
    dx, dgrid = nn.vl_nnbilinearsampler(*_up(mat, xb, gridb, dyb))
    dxr, dgr = oracle.sampler_backward(xb, gridb, dyb)
    assert bit_equal(mat.to_numpy(dx), dxr) and bit_equal(mat.to_numpy(dgrid), dgr)
    H, W, C, N, Ng, Ho, Wo = 12, 20, 13, 3, 6, 16, 8
    # 2: every output pixel samples around one point
    grid2 = np.asfortranarray((0.013 * rng.standard_normal((2, Ho, Wo, Ng)) + 0.2).astype(np.float32))
    dyi = np.asfortranarray(rng.integers(-3, 4, (Ho, Wo, C, Ng)).astype(np.float32))
    x1 = np.ones_like(x)
    dx, dgrid = nn.vl_nnbilinearsampler(*_up(mat, x1, grid2, dyi))
    dxr, dgr = oracle.sampler_backward(x1, grid2, dyi)
    assert rel_l2(mat.to_numpy(dx), dxr) < 1e-6 and bit_equal(mat.to_numpy(dgrid), dgr)
    # 3: planes of 150 x 150
    x3 = np.asfortranarray(rng.standard_normal((150, 150, 2, 1)).astype(np.float32))
    grid3 = np.asfortranarray(rng.uniform(-1, 1, (2, 150, 150, 1)).astype(np.float32))
    dy3 = np.asfortranarray(rng.integers(-3, 4, (150, 150, 2, 1)).astype(np.float32))
    dx, dgrid = nn.vl_nnbilinearsampler(*_up(mat, x3, grid3, dy3))
    dxr, dgr = oracle.sampler_backward(x3, grid3, dy3)
    assert rel_l2(mat.to_numpy(dx), dxr) < 1e-6 and bit_equal(mat.to_numpy(dgrid), dgr)


def test_roipool_backward_batches_and_fallback(gpu, oracle):
    """ROI pooling backward beyond one shared-memory batch (many ROIs on one image, processed in several batches with the
    partial sums carried in dX), with an image that no ROI names (its slab is zero), and on a map too large for a slab
    (atomic scatter, integer-valued derivatives)."""
    nn, mat, _ = gpu
    rng = np.random.default_rng(18)
    H, W, C, N, K = 20, 30, 24, 3, 3000
    x = np.asfortranarray(rng.standard_normal((H, W, C, N)).astype(np.float32))
    u1, v1 = rng.uniform(1, W - 2, K), rng.uniform(1, H - 2, K)
    u2, v2 = np.minimum(u1 + rng.uniform(0, W, K), W), np.minimum(v1 + rng.uniform(0, H, K), H)
    image = np.where(rng.uniform(size=K) < 0.9, 1, 3)            # image 2 has no ROI
    rois = np.asfortranarray(np.stack([image, u1, v1, u2, v2]).astype(np.float32))
    for method in ("max", "avg"):
        y = oracle.roipool_forward(x, rois, (7, 7), 1.0, method)
        dy = np.asfortranarray(rng.standard_normal(y.shape).astype(np.float32))
        dx = nn.vl_nnroipool(*_up(mat, x, rois, dy), subdivisions=(7, 7), method=method)
        want = oracle.roipool_backward(x, rois, dy, (7, 7), 1.0, method)
        assert bit_equal(mat.to_numpy(dx), want), method
        assert np.all(mat.to_numpy(dx)[:, :, :, 1] == 0)
    xb = np.asfortranarray(rng.standard_normal((300, 260, 2, 1)).astype(np.float32))
    rb = np.asfortranarray(np.array([[1, 5, 9, 200, 250], [1, 100, 50, 260, 300], [1, 1, 1, 20, 20]], np.float32).T)
    yb = oracle.roipool_forward(xb, rb, (6, 5), 1.0, "max")
    dyb = np.asfortranarray(rng.integers(-3, 4, yb.shape).astype(np.float32))
    dxb = nn.vl_nnroipool(*_up(mat, xb, rb, dyb), subdivisions=(6, 5), method="max")
    assert bit_equal(mat.to_numpy(dxb), oracle.roipool_backward(xb, rb, dyb, (6, 5), 1.0, "max"))


# ------------------------------------------------------------------ LRN, softmax, dropout
@pytest.mark.parametrize("prm", [[5, 2.0, 1e-4, 0.75], [4, 1.0, 0.1, 0.5], [1, 1.5, 0.5, 1.0], [9, 2.0, 1e-2, 0.6]])
def test_lrn_vs_oracle(gpu, oracle, reference_backend, prm):
    """vl_nnnormalize forward and backward on AlexNet's first LRN shape (55x55x96, reduced batch) and a ragged one: within
    1e-5 of the double-precision checker; within the error of the reference CPU code's approximate power (5e-3) of the
    compiled reference."""
    nn, mat, _ = gpu
    rng = np.random.default_rng(40)
    for shape in [(55, 55, 96, 2), (7, 5, 13, 3)]:
        x = np.asfortranarray(rng.standard_normal(shape).astype(np.float32) * 3)
        dy = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
        xd, dyd = _up(mat, x, dy)
        y = mat.to_numpy(nn.vl_nnnormalize(xd, prm))
        dx = mat.to_numpy(nn.vl_nnnormalize(xd, prm, dyd))
        assert rel_l2(y, oracle.lrn_forward(x.astype(np.float64), prm)) < TOL_FAITHFUL
        assert rel_l2(dx, oracle.lrn_backward(x.astype(np.float64), prm, dy.astype(np.float64))) < TOL_FAITHFUL
        if reference_backend is not None:
            assert rel_l2(y, reference_backend.lrn_forward(x, prm)) < 5e-3
            assert rel_l2(dx, reference_backend.lrn_backward(x, prm, dy)) < 5e-3


def test_softmax_and_dropout(gpu, oracle):
    import torch
    nn, mat, _ = gpu
    rng = np.random.default_rng(41)
    for shape in [(1, 1, 1000, 16), (6, 5, 21, 3)]:
        x = np.asfortranarray((rng.standard_normal(shape) * 4).astype(np.float32))
        dy = np.asfortranarray(rng.standard_normal(shape).astype(np.float32))
        xd, dyd = _up(mat, x, dy)
        assert rel_l2(mat.to_numpy(nn.vl_nnsoftmax(xd)), oracle.softmax(x.astype(np.float64))) < 1e-6
        assert rel_l2(mat.to_numpy(nn.vl_nnsoftmax(xd, dyd)), oracle.softmax(x.astype(np.float64), dy.astype(np.float64))) < TOL_FAITHFUL
    # dropout (matlab/vl_nndropout.m): mask = 1/(1-rate) * (rand >= rate); y = mask .* x; backward = mask .* dzdy
    x = mat.as_mat(torch.randn(64, 64, 32, 8, device="cuda"))
    for rate in (0.5, 0.2, 0.0):
        y, mask = nn.vl_nndropout(x, rate=rate, seed=3)
        scale = np.float32(1.0 / (1.0 - rate))
        assert bool(((mask == 0) | (mask == float(scale))).all())
        kept = float((mask != 0).float().mean())
        assert abs(kept - (1.0 - rate)) < 4e-3                      # 1M draws: 4e-3 is eight standard deviations
        assert torch.equal(y, mask * x)
        y2, mask2 = nn.vl_nndropout(x, rate=rate, seed=3)
        assert torch.equal(mask, mask2)                             # the same seed gives the same mask
        if rate > 0:
            _, mask3 = nn.vl_nndropout(x, rate=rate, seed=4)
            assert not torch.equal(mask, mask3)
            agree = float(((mask != 0) == (mask3 != 0)).float().mean())
            assert abs(agree - (rate ** 2 + (1 - rate) ** 2)) < 6e-3    # independent streams
        dz = mat.as_mat(torch.randn(64, 64, 32, 8, device="cuda"))
        dx, _ = nn.vl_nndropout(x, dz, mask=mask)
        assert torch.equal(dx, mask * dz)


def test_alexnet_style_chain_with_lrn_and_dropout(gpu, oracle):
    """conv -> relu -> LRN -> max-pool -> conv-as-FC -> dropout -> conv-as-FC -> softmax loss through vl_simplenn; every
    layer replayed from the GPU's own tensors (the dropout layer with the mask the forward pass drew)."""
    import torch
    import cpu_net
    from matconvnet_b200 import models, simplenn
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    rng = np.random.default_rng(42)
    layers = [models._conv(rng, 3, 3, 3, 16, 1, 1), models._relu(), {"type": "normalize", "param": [5, 2.0, 1e-4, 0.75]},
              models._pool("max", 2, 2), models._conv(rng, 8, 8, 16, 24, 1, 0), models._relu(),
              {"type": "dropout", "rate": 0.5, "seed": 7}, models._conv(rng, 1, 1, 24, 5, 1, 0),
              {"type": "softmaxloss", "class": torch.tensor([1, 5, 2, 3], device="cuda").float()}]
    net = {"layers": layers}
    x = mat.from_numpy(np.asfortranarray(rng.standard_normal((16, 16, 3, 4)).astype(np.float32)))
    res = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
    host = []
    for l in layers:
        m = dict(l)
        if "weights" in l:
            m["weights"] = [mat.to_numpy(w).astype(np.float64) for w in l["weights"]]
        if l.get("class") is not None:
            m["class"] = l["class"].cpu().numpy().astype(np.float64)
        host.append(m)
    f64 = lambda t: np.asfortranarray(mat.to_numpy(t), dtype=np.float64)
    for i, l in enumerate(host):
        d = res[i + 1]["dzdx"]
        d = np.float64(d) if np.isscalar(d) else f64(d)
        if l["type"] == "dropout":
            mask = f64(res[i]["aux"])
            assert bit_equal(mat.to_numpy(res[i + 1]["x"]), (mask * f64(res[i]["x"])).astype(np.float32))
            assert bit_equal(mat.to_numpy(res[i]["dzdx"]), (mask * d).astype(np.float32))
            continue
        y = cpu_net.layer_forward(oracle, oracle, l, f64(res[i]["x"]))
        got = res[i + 1]["x"].cpu().numpy() if l["type"] == "softmaxloss" else mat.to_numpy(res[i + 1]["x"])
        assert rel_l2(got, y) < TOL_FAITHFUL, (i, l["type"])
        dx, _ = cpu_net.layer_backward(oracle, oracle, l, f64(res[i]["x"]), d)
        assert rel_l2(mat.to_numpy(res[i]["dzdx"]), dx) < TOL_FAITHFUL, (i, l["type"])


def test_bnorm_relu_fused_forward_is_bit_identical(gpu):
    """vl_nnbnorm(..., relu=True) against vl_nnrelu(vl_nnbnorm(...)), vector and scalar paths, and a small network with
    conv -> bnorm -> relu blocks under fuse_relu against the plain schedule: same outputs and gradients bit for bit."""
    import torch
    from matconvnet_b200 import models, simplenn
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    g = torch.Generator(device="cuda").manual_seed(50)
    for shape in [(28, 28, 128, 8), (7, 5, 6, 3)]:
        x = mat.as_mat(torch.randn(*shape, device="cuda", generator=g))
        gam = mat.as_mat(torch.rand(shape[2], 1, device="cuda", generator=g) + 0.5)
        bet = mat.as_mat(torch.randn(shape[2], 1, device="cuda", generator=g))
        y, mom = nn.vl_nnbnorm(x, gam, bet, epsilon=1e-5)
        yr, momr = nn.vl_nnbnorm(x, gam, bet, epsilon=1e-5, relu=True)
        assert torch.equal(yr, nn.vl_nnrelu(y)) and torch.equal(mom, momr)
        yg, _ = nn.vl_nnbnorm(x, gam, bet, epsilon=1e-5, moments=mom, relu=True)
        assert torch.equal(yg, nn.vl_nnrelu(nn.vl_nnbnorm(x, gam, bet, epsilon=1e-5, moments=mom)[0]))
    rng = np.random.default_rng(51)
    bn = lambda c: {"type": "bnorm", "weights": [mat.from_numpy(np.ones((c, 1), np.float32)), mat.from_numpy(np.zeros((c, 1), np.float32))],
                    "epsilon": 1e-5}
    layers = [models._conv(rng, 3, 3, 3, 32, 1, 1), bn(32), models._relu(), models._conv(rng, 3, 3, 32, 32, 1, 1), bn(32),
              models._relu(), models._pool("max", 2, 2), models._conv(rng, 8, 8, 32, 4, 1, 0),
              {"type": "softmaxloss", "class": torch.tensor([1, 2, 3, 4, 1], device="cuda").float()}]
    net = {"layers": layers}
    x = mat.as_mat(torch.randn(16, 16, 3, 5, device="cuda", generator=g))
    plain = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
    fused = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx, fuse_relu=True)
    assert torch.equal(plain[-1]["x"], fused[-1]["x"]) and torch.equal(plain[0]["dzdx"], fused[0]["dzdx"])
    for a, c in zip(plain, fused):
        for u, v in zip(a["dzdw"] or [], c["dzdw"] or []):
            assert (u is None and v is None) or torch.equal(u, v)
