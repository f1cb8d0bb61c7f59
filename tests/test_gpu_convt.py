"""Convolution transpose through the C ABI against the CPU checker and the reference's golden vectors
(reference xtest/suite/nnconvt.m: upsampling, crops, filter groups, the identity with vl_nnconv).

Arithmetic modes and bounds as for the convolution (tests/test_gpu_conv.py).
"""
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
    assert ctx.device_status() == 0


@pytest.mark.parametrize("mode,prec,tol", MODES)
def test_convt_golden(gpu, precision, mode, prec, tol):
    nn, mat, ctx = gpu
    ctx.set_precision(prec)
    g = load_golden("convt")
    for c in cases_of(g):
        prm = [int(v) for v in g[c + ".prm"]]
        kw = dict(upsample=tuple(prm[0:2]), crop=tuple(prm[2:6]), num_groups=prm[6])
        x, f, b, dy = _up(mat, g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"])
        y = nn.vl_nnconvt(x, f, b, **kw)
        dx, df, db = nn.vl_nnconvt(x, f, b, dy, **kw)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            got = mat.to_numpy(got)
            assert got.size == g[c + "." + name].size, (c, name)
            assert rel_l2(got.ravel(), g[c + "." + name + "64"].ravel()) < tol, (c, name, mode)
            assert rel_l2(got.ravel(), g[c + "." + name].ravel()) < tol + 2e-6, (c, name, mode)


# shapes that reach the tensor-core kernels: x, filters (FH, FW, FD, C), upsample, crop
LAYERS = {
    "up1_tensor_memory_kernel": ((20, 24, 64, 3), (3, 3, 48, 64), (1, 1), (1, 1, 1, 1)),     # dgrad stride 1; fprop; wgrad
    "fcn32s_like_up4": ((6, 7, 21, 2), (8, 8, 21, 21), (4, 4), (2, 2, 2, 2)),               # strided: CUDA-core data gradient
    "up2_wide": ((12, 10, 96, 2), (4, 4, 40, 96), (2, 2), (1, 1, 1, 1)),
}


@pytest.mark.parametrize("layer", sorted(LAYERS))
@pytest.mark.parametrize("mode,prec,tol", MODES)
def test_convt_layers_vs_oracle(gpu, oracle, precision, layer, mode, prec, tol):
    nn, mat, ctx = gpu
    ctx.set_precision(prec)
    xs, fs, up, crop = LAYERS[layer]
    rng = np.random.default_rng(len(layer) * 131 + xs[2])
    x = np.asfortranarray(rng.standard_normal(xs).astype(np.float32))
    f = np.asfortranarray((rng.standard_normal(fs) * np.sqrt(2.0 / np.prod(fs[:3]))).astype(np.float32))
    b = rng.standard_normal(fs[2]).astype(np.float32)
    x64, f64, b64 = (a.astype(np.float64) for a in (x, f, b))
    y64 = oracle.convt_forward(x64, f64, b64, up, crop)
    dy = np.asfortranarray(rng.standard_normal(y64.shape).astype(np.float32))
    want = (y64,) + tuple(oracle.convt_backward(x64, f64, dy.astype(np.float64), up, crop))
    xd, fd, bd, dyd = _up(mat, x, f, b, dy)
    got = (nn.vl_nnconvt(xd, fd, bd, upsample=up, crop=crop),) + tuple(nn.vl_nnconvt(xd, fd, bd, dyd, upsample=up, crop=crop))
    for g_, w_, name in zip(got, want, ("y", "dx", "df", "db")):
        assert rel_l2(mat.to_numpy(g_).ravel(), w_.ravel()) < tol, (layer, name, mode)


def test_convt_is_adjoint_of_conv_and_skips_null_outputs(gpu):
    """<convt(x; F), dy> == <x, conv(dy; F)> (the transposed convolution is the adjoint of the convolution with stride =
    upsample, pad = crop); derivative switches leave the skipped outputs out."""
    import torch
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = mat.as_mat(torch.randn(9, 8, 32, 2, device="cuda", generator=g))
    f = mat.as_mat(torch.randn(3, 3, 16, 32, device="cuda", generator=g) * 0.1)
    y = nn.vl_nnconvt(x, f, None, upsample=2, crop=(0, 1, 1, 0))
    dy = mat.as_mat(torch.randn(*mat.shape4(y), device="cuda", generator=g))
    back = nn.vl_nnconv(dy, f, None, stride=2, pad=(0, 1, 1, 0))
    lhs = float((y.double() * dy.double()).sum()), float((x.double() * back.double()).sum())
    assert abs(lhs[0] - lhs[1]) <= 1e-5 * max(1.0, abs(lhs[0]))
    dx, df, db = nn.vl_nnconvt(x, f, None, dy, upsample=2, crop=(0, 1, 1, 0), no_der_filters=True)
    assert df is None and db is None and torch.equal(dx, back)


def test_convt_rejects_bad_arguments(gpu):
    import torch
    from matconvnet_b200 import capi
    nn, mat, ctx = gpu
    x = mat.as_mat(torch.zeros(4, 4, 6, 1, device="cuda"))
    f = mat.as_mat(torch.zeros(3, 3, 2, 6, device="cuda"))
    for kw in (dict(upsample=0), dict(crop=(-1, 0, 0, 0)), dict(num_groups=4), dict(crop=(6, 6, 0, 0))):
        with pytest.raises(capi.VlbError):
            nn.vl_nnconvt(x, f, None, **kw)
    with pytest.raises(capi.VlbError):          # the filter bank's fourth dimension is not the data depth
        nn.vl_nnconvt(x, mat.as_mat(torch.zeros(3, 3, 2, 5, device="cuda")), None)
