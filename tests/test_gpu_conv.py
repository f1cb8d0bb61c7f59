"""Convolution and fully-connected kernels through the C ABI against the CPU checker.

Every case runs in the three arithmetic modes of the engine:
  3xTF32 (default, tensor cores, fp32-faithful)  -> rel. L2 <= 1e-5
  FP32   (CUDA cores)                            -> rel. L2 <= 1e-5
  TF32   (tensor cores, single pass)             -> rel. L2 <= 2e-3
The comparison target is the double-precision instantiation of the checker, so the bound
measures our error alone, plus the golden single-precision vectors of the reference itself.
"""
import zlib

import numpy as np
import pytest

from conftest import cases_of, load_golden, rel_l2

pytestmark = pytest.mark.gpu

MODES = [("3xtf32", 0, 1e-5), ("fp32", 2, 1e-5), ("tf32", 1, 2e-3)]


def _up(mat, *arrays):
    return [None if a is None else mat.from_numpy(a) for a in arrays]


@pytest.fixture
def precision(gpu):
    _, _, ctx = gpu
    yield ctx
    ctx.set_precision(0)
    assert ctx.device_status() == 0      # no tensor-core kernel gave up a pipeline wait


@pytest.mark.parametrize("mode,prec,tol", MODES)
def test_conv_golden(gpu, precision, mode, prec, tol):
    nn, mat, ctx = gpu
    ctx.set_precision(prec)
    g = load_golden("conv")
    for c in cases_of(g):
        prm = g[c + ".prm"]
        kw = dict(stride=tuple(prm[0:2]), pad=tuple(prm[2:6]), dilate=tuple(prm[6:8]))
        x, f, b, dy = _up(mat, g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"])
        y = nn.vl_nnconv(x, f, b, **kw)
        dx, df, db = nn.vl_nnconv(x, f, b, dy, **kw)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            got = mat.to_numpy(got)
            assert rel_l2(got.ravel(), g[c + "." + name + "64"].ravel()) < tol, (c, name, mode)
            assert rel_l2(got.ravel(), g[c + "." + name].ravel()) < tol + 2e-6, (c, name, mode)


@pytest.mark.parametrize("mode,prec,tol", MODES)
def test_fc_golden(gpu, precision, mode, prec, tol):
    nn, mat, ctx = gpu
    ctx.set_precision(prec)
    g = load_golden("fc")
    for c in cases_of(g):
        x, f, b, dy = _up(mat, g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"])
        y = nn.vl_nnconv(x, f, b)
        dx, df, db = nn.vl_nnconv(x, f, b, dy)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(mat.to_numpy(got).ravel(), g[c + "." + name].ravel()) < tol + 2e-6, (c, name, mode)


# (x shape, f shape, stride, pad, dilate): the layer geometries of the five configurations, scaled
# down in batch/extent so the scalar CPU checker finishes in seconds.
LAYERS = {
    "lenet_conv1": ((28, 28, 1, 6), (5, 5, 1, 20), 1, 0, 1),
    "lenet_conv2": ((12, 12, 20, 6), (5, 5, 20, 50), 1, 0, 1),
    "cifar_conv1": ((32, 32, 3, 4), (5, 5, 3, 32), 1, 2, 1),
    "cifar_conv2": ((16, 16, 32, 4), (5, 5, 32, 32), 1, 2, 1),
    "cifar_conv3": ((8, 8, 32, 4), (5, 5, 32, 64), 1, 2, 1),
    "cifar_fc4": ((4, 4, 64, 10), (4, 4, 64, 64), 1, 0, 1),
    "cifar_fc5": ((1, 1, 64, 10), (1, 1, 64, 10), 1, 0, 1),
    "resnet_1x1_a": ((28, 28, 512, 2), (1, 1, 512, 128), 1, 0, 1),
    "resnet_3x3": ((28, 28, 128, 2), (3, 3, 128, 128), 1, 1, 1),
    "resnet_1x1_b": ((28, 28, 128, 2), (1, 1, 128, 512), 1, 0, 1),
    "vgg_conv1_1": ((64, 48, 3, 2), (3, 3, 3, 64), 1, 1, 1),
    "vgg_conv1_2": ((48, 40, 64, 2), (3, 3, 64, 64), 1, 1, 1),
    "vgg_conv3_1": ((28, 28, 128, 2), (3, 3, 128, 256), 1, 1, 1),
    "vgg_conv5": ((14, 14, 512, 2), (3, 3, 512, 512), 1, 1, 1),
    "vgg_fc6": ((7, 7, 512, 4), (7, 7, 512, 256), 1, 0, 1),
    "vgg_fc7": ((1, 1, 4096, 8), (1, 1, 4096, 512), 1, 0, 1),
    "vgg_fc8": ((1, 1, 4096, 8), (1, 1, 4096, 1000), 1, 0, 1),
    "odd_stride2": ((17, 15, 6, 3), (3, 3, 6, 10), 2, (1, 0, 1, 1), 1),
    "odd_dilate2": ((15, 13, 4, 2), (3, 3, 4, 8), 1, 2, 2),
    "odd_groups": ((10, 10, 8, 2), (3, 3, 2, 12), 1, 1, 1),
    "odd_nobias_ragged": ((9, 11, 5, 3), (2, 4, 5, 7), (1, 2), (0, 1, 2, 0), 1),
    # channel counts that are multiples of 32 (one filter tap per 32-deep reduction block) with strides, dilation,
    # asymmetric padding, a ragged last row tile, and 96 = 3 x 32 channels (not a multiple of 64)
    "c32_stride2_pad": ((19, 17, 32, 3), (3, 3, 32, 40), 2, (1, 0, 2, 1), 1),
    "c96_dilate2": ((15, 14, 96, 2), (3, 2, 96, 72), 1, (2, 2, 1, 1), (2, 1)),
    "c64_5x5_stride_1_2": ((13, 21, 64, 2), (5, 5, 64, 33), (1, 2), 2, 1),
    # image-end shapes served by the direct CUDA-core kernels: few inputs per pixel (forward), few channels (dgrad)
    "small_r_stride": ((41, 37, 2, 5), (3, 5, 2, 20), (2, 1), (1, 0, 2, 1), 1),
    "small_r_dilate_c1": ((50, 47, 1, 3), (3, 3, 1, 70), 1, (2, 1, 0, 2), 2),
    "small_n_4ch_5x5": ((36, 40, 4, 4), (5, 5, 4, 24), 1, 2, 1),
    "small_n_rgb_3x3": ((40, 36, 3, 3), (3, 3, 3, 20), 1, 1, 1),
    "small_n_3x3_pad_dilate_y": ((33, 38, 2, 4), (3, 3, 2, 9), 1, (2, 2, 0, 2), (2, 1)),
}


def _he(rng, shape):
    # dagnn.Conv.initParams (reference matlab/+dagnn/Conv.m:38-46)
    return np.asfortranarray((rng.standard_normal(shape) * np.sqrt(2.0 / np.prod(shape[:3]))).astype(np.float32))


@pytest.mark.parametrize("mode,prec,tol", MODES)
@pytest.mark.parametrize("layer", sorted(LAYERS))
def test_conv_layers_vs_oracle(gpu, oracle, precision, layer, mode, prec, tol):
    nn, mat, ctx = gpu
    ctx.set_precision(prec)
    xs, fs, stride, pad, dilate = LAYERS[layer]
    as2 = lambda v: (v, v) if np.isscalar(v) else tuple(v)
    as4 = lambda v: (v,) * 4 if np.isscalar(v) else tuple(v)
    rng = np.random.default_rng(zlib.crc32(layer.encode()))
    x = np.asfortranarray(rng.standard_normal(xs).astype(np.float32))
    f = _he(rng, fs)
    b = None if "nobias" in layer else (rng.standard_normal(fs[3]) * 0.1).astype(np.float32)
    kw = dict(stride=as2(stride), pad=as4(pad), dilate=as2(dilate))
    x64, f64 = x.astype(np.float64), f.astype(np.float64)
    b64 = None if b is None else b.astype(np.float64)
    y_ref = oracle.conv_forward(x64, f64, b64, **kw)
    dy = np.asfortranarray(rng.standard_normal(y_ref.shape).astype(np.float32))
    dx_ref, df_ref, db_ref = oracle.conv_backward(x64, f64, dy.astype(np.float64), **kw)
    xd, fd, bd, dyd = _up(mat, x, f, b, dy)
    y = nn.vl_nnconv(xd, fd, bd, **kw)
    assert tuple(y.shape) == y_ref.shape
    assert rel_l2(mat.to_numpy(y), y_ref) < tol, "y"
    dx, df, db = nn.vl_nnconv(xd, fd, bd, dyd, **kw)
    assert rel_l2(mat.to_numpy(dx), dx_ref) < tol, "dx"
    assert rel_l2(mat.to_numpy(df), df_ref) < tol, "df"
    if b is not None:
        assert rel_l2(mat.to_numpy(db).ravel(), db_ref) < tol, "db"
    else:
        assert db is None
    # skipping outputs (NoDerData / NoDerFilters) leaves the others unchanged
    dx2, df2, _ = nn.vl_nnconv(xd, fd, bd, dyd, no_der_filters=True, **kw)
    assert df2 is None and np.array_equal(mat.to_numpy(dx2), mat.to_numpy(dx))
    dx3, df3, _ = nn.vl_nnconv(xd, fd, bd, dyd, no_der_data=True, **kw)
    assert dx3 is None and np.array_equal(mat.to_numpy(df3), mat.to_numpy(df))


def test_fused_bias_gradient_is_deterministic_and_matches_the_separate_kernel(gpu):
    """When the output plane is a multiple of four pixels the bias gradient is summed by the kernel that writes the
    dY tile images of the filter gradient (per-block partials finished by the last block, in block order): the
    result must not depend on the scheduling, and must agree with the stand-alone reduction used when only the bias
    gradient is asked for (reference bits/nnconv.cu:229-244)."""
    nn, mat, ctx = gpu
    import torch
    ctx.set_precision(0)
    x = mat.as_mat(torch.randn(40, 36, 32, 6, device="cuda"))
    f = mat.as_mat(torch.randn(3, 3, 32, 48, device="cuda") * 0.05)
    b = mat.zeros((1, 48))
    dy = mat.as_mat(torch.randn(40, 36, 48, 6, device="cuda"))
    runs = [mat.to_numpy(nn.vl_nnconv(x, f, b, dy, pad=1, no_der_data=True)[2]).ravel() for _ in range(3)]
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    alone = mat.to_numpy(nn.vl_nnconv(x, f, b, dy, pad=1, no_der_data=True, no_der_filters=True)[2]).ravel()
    ref = mat.to_numpy(dy).astype(np.float64).sum(axis=(0, 1, 3))
    assert rel_l2(runs[0], ref) < 1e-6 and rel_l2(alone, ref) < 1e-6


def test_conv_identities_on_device(gpu):
    """stride == subsampling, pad == crop, groups == block-diagonal (reference
    xtest/suite/nnconv.m:88-125,144-161), in the default arithmetic."""
    nn, mat, _ = gpu
    rng = np.random.default_rng(21)
    x = np.asfortranarray(rng.standard_normal((20, 18, 8, 2)).astype(np.float32))
    f = np.asfortranarray(rng.standard_normal((3, 3, 8, 16)).astype(np.float32))
    b = rng.standard_normal(16).astype(np.float32)
    xd, fd, bd = _up(mat, x, f, b)
    y1 = mat.to_numpy(nn.vl_nnconv(xd, fd, bd))
    for s in [(2, 2), (3, 1)]:
        ys = mat.to_numpy(nn.vl_nnconv(xd, fd, bd, stride=s))
        assert rel_l2(ys, y1[::s[0], ::s[1]]) < 1e-5
    yp = mat.to_numpy(nn.vl_nnconv(xd, fd, bd, pad=(2, 1, 0, 2)))
    xp = np.zeros((23, 20, 8, 2), np.float32, order="F")
    xp[2:22, 0:18] = x
    assert rel_l2(yp, mat.to_numpy(nn.vl_nnconv(mat.from_numpy(xp), fd, bd))) < 1e-5
    fg = np.asfortranarray(rng.standard_normal((3, 3, 4, 16)).astype(np.float32))
    fdense = np.zeros((3, 3, 8, 16), np.float32, order="F")
    fdense[:, :, 0:4, 0:8] = fg[:, :, :, 0:8]
    fdense[:, :, 4:8, 8:16] = fg[:, :, :, 8:16]
    yg = mat.to_numpy(nn.vl_nnconv(xd, mat.from_numpy(fg), bd))
    assert rel_l2(yg, mat.to_numpy(nn.vl_nnconv(xd, mat.from_numpy(fdense), bd))) < 1e-5


def test_conv_rejects_bad_arguments(gpu):
    nn, mat, _ = gpu
    from matconvnet_b200.capi import VlbError
    x, f = mat.zeros((8, 8, 6, 1)), mat.zeros((3, 3, 4, 2))
    with pytest.raises(VlbError):
        nn.vl_nnconv(x, f, None)                          # filter depth does not divide data depth
    with pytest.raises(VlbError):
        nn.vl_nnconv(mat.zeros((2, 2, 4, 1)), f, None)    # filters larger than the data
    with pytest.raises(TypeError):
        import torch
        nn.vl_nnconv(torch.zeros(8, 8, 4, 1), f, None)    # host tensor: no CPU path
