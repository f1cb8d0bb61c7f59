"""Full-size checks (the layer shapes of the VGG-16 configuration at 64 images per GPU), where the scalar CPU
checker would take minutes per layer: size-independent properties instead.

* Adjointness.  Convolution is bilinear, so <dY, conv(X, F)> = <dgrad(dY, F), X> = <wgrad(X, dY), F>: the three
  tensor-core kernels (forward, data gradient, filter gradient) are checked against one another; the inner products
  are accumulated in float64 on the device.  The bias gradient is checked against a float64 sum of dY.
* Max-pool backward conserves the gradient mass exactly for 2x2/stride-2 windows (every dY lands on one input
  element), and pooling the routed gradient with the same windows returns dY where dY is positive.
* Batch-norm backward: dx sums to zero per channel and is orthogonal to the centred input (reference
  bits/nnbnorm.cu:136-164 subtracts both projections).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LAYERS = [("conv1_1", 224, 3, 64, 3, 1), ("conv1_2", 224, 64, 64, 3, 1), ("conv2_1", 112, 64, 128, 3, 1),
          ("conv3_2", 56, 256, 256, 3, 1), ("conv5_1", 14, 512, 512, 3, 1), ("fc6", 7, 512, 4096, 7, 0)]


def _dot(a, b):
    import torch
    return float((a.double() * b.double()).sum())


@pytest.mark.parametrize("name,hw,cin,cout,fs,pad", LAYERS)
def test_conv_adjointness_full_size(gpu, name, hw, cin, cout, fs, pad):
    import torch
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    ctx.reserve_workspace(3 << 30)
    g = torch.Generator(device="cuda").manual_seed(7)
    B = 64
    x = mat.as_mat(torch.randn(hw, hw, cin, B, device="cuda", generator=g).clamp_(min=0))      # post-ReLU activations
    f = mat.as_mat(torch.randn(fs, fs, cin, cout, device="cuda", generator=g) * (2.0 / (fs * fs * cin)) ** 0.5)
    b = mat.zeros((1, cout))
    y = nn.vl_nnconv(x, f, b, pad=pad)
    dy = mat.as_mat(torch.randn(*y.shape, device="cuda", generator=g))
    dx, df, db = nn.vl_nnconv(x, f, b, dy, pad=pad)
    assert ctx.device_status() == 0
    lhs = _dot(dy, y)
    # the three inner products agree to the accuracy of the arithmetic (each is a sum of ~1e8 products of the results)
    scale = float(dy.double().norm() * y.double().norm())
    assert abs(lhs - _dot(dx, x)) <= 1e-5 * scale, (lhs, _dot(dx, x), scale)
    assert abs(lhs - _dot(df, f)) <= 1e-5 * scale, (lhs, _dot(df, f), scale)
    ref_db = dy.double().sum(dim=(0, 1, 3))
    err = float((db.double().reshape(-1) - ref_db).norm() / ref_db.norm())
    assert err < 1e-5, err
    del x, f, y, dy, dx, df
    torch.cuda.empty_cache()


def test_maxpool_backward_conserves_mass_full_size(gpu):
    import torch
    nn, mat, ctx = gpu
    x = mat.as_mat(torch.randn(224, 224, 64, 64, device="cuda"))
    y = nn.vl_nnpool(x, (2, 2), stride=2)
    dy = mat.as_mat(torch.randint(-8, 9, tuple(y.shape), device="cuda").float())      # integer-valued: sums are exact
    dx = nn.vl_nnpool(x, (2, 2), dy, stride=2)
    assert float(dx.double().sum()) == float(dy.double().sum())
    # every window holds exactly its dy at the arg-max and zeros elsewhere: pooling |dx| returns |dy|
    back = nn.vl_nnpool(mat.as_mat(torch.abs(dx)), (2, 2), stride=2)
    assert torch.equal(back, torch.abs(dy))
    # and the routed element is the window's maximum
    routed = dx != 0
    ymax = y.repeat_interleave(2, 0).repeat_interleave(2, 1)
    assert bool((x[routed] == ymax[routed]).all())


def test_bnorm_backward_projections_full_size(gpu):
    import torch
    nn, mat, ctx = gpu
    shape = (28, 28, 512, 64)
    x = mat.as_mat(torch.randn(*shape, device="cuda") * 2 + 1)
    dy = mat.as_mat(torch.randn(*shape, device="cuda"))
    gm = mat.as_mat(torch.rand(512, 1, device="cuda") + 0.5)
    bt = mat.zeros((512, 1))
    dx, dg, db, mom = nn.vl_nnbnorm(x, gm, bt, dy, epsilon=1e-5)
    xd, dxd = x.double(), dx.double()
    mean = xd.mean(dim=(0, 1, 3), keepdim=True)
    n = 28 * 28 * 64
    scale = dxd.abs().sum(dim=(0, 1, 3))
    assert float((dxd.sum(dim=(0, 1, 3)).abs() / scale).max()) < 1e-5
    assert float(((dxd * (xd - mean)).sum(dim=(0, 1, 3)).abs() / (scale * xd.std())).max()) < 1e-4
    ref_db = dy.double().sum(dim=(0, 1, 3))
    assert float((db.double().reshape(-1) - ref_db).norm() / ref_db.norm()) < 1e-5
    ref_mean = mean.reshape(-1)
    assert float((mom.double()[:, 0] - ref_mean).abs().max()) < 1e-5           # moments: column 0 means, column 1 sigmas
