"""The benchmark specification's configurations at their full sizes, against the reference's own compiled CPU backend.

The compiled backend (the reference's unmodified CPU sources, double-precision instantiation, its GEMMs routed to a
threaded BLAS) finishes these sizes in seconds, so the batch-size-dependent paths of the GPU kernels -- persistent CTAs
walking many tiles, split reductions, 3.2-million-term filter-gradient sums, 256 overlapping ROIs -- are compared with
the reference itself rather than only with size-independent properties:

  C2  CIFAR-10 network, batch 100                   (reference examples/cifar/cnn_cifar_init.m:11-65)
  C3  ResNet-50 stage-3 bottleneck, batch 64, both batch-norm backward modes
                                                    (examples/imagenet/cnn_imagenet_init_resnet.m:16-115)
  C4  VGG-16 conv1_2, conv3_2, conv5_1 backward at batch 64 (data, filter and bias gradients)
  C5  Fast R-CNN head: 256 ROIs on 38x50x512x2, 7x7 max pooling, 4096-wide conv-as-FC layers, identity and 1/16
      transforms; bilinear sampler 64x64x32x256 with 256 affine grids
                                                    (examples/fast_rcnn/fast_rcnn_init.m:53-61,
                                                     matlab/+dagnn/AffineGridGenerator.m:36-57)

Every layer is replayed from the GPU's own input and output derivative (a ReLU or max-pool decision on an activation
within rounding of a tie must not leak into the layers below it).  Bars: relative L2 <= 1e-5 for convolution, fully
connected and batch-norm results against the double-precision instantiation; bit-exact against the single-precision
instantiation for max / average pooling, ROI pooling (forward and backward) and the bilinear sampler (both derivatives).
Synthetic seeded tensors stand in for CIFAR-10, ILSVRC-2012 and VOC07 images.
"""
import os

import numpy as np
import pytest

from conftest import bit_equal, rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-5


@pytest.fixture(scope="module")
def ref_blas():
    """The compiled reference backend with a threaded BLAS behind it; restored to its plain BLAS afterwards."""
    import oracle as O
    ref = O.reference()
    if ref is None or not O.reference_use_openblas(os.cpu_count() or 1):
        pytest.skip("the compiled reference backend or a threaded BLAS for it is not available")
    yield ref
    O.reference_use_plain_blas()


def _f64(mat, t):
    return np.asfortranarray(mat.to_numpy(t), dtype=np.float64)


def _host_layers(layers, mat):
    out = []
    for l in layers:
        m = dict(l)
        if "weights" in l:
            m["weights"] = [None if w is None else _f64(mat, w) for w in l["weights"]]
        if l.get("class") is not None and not isinstance(l["class"], np.ndarray):
            m["class"] = l["class"].cpu().numpy().astype(np.float64)
        out.append(m)
    return out


def _replay(res, mat, ref, glue, layers, tol=TOL):
    """Every layer from the GPU's own input and output derivative: contractions and normalisations against the double
    instantiation, pooling bit for bit against the single-precision one."""
    import cpu_net
    host = _host_layers(layers, mat)
    worst = 0.0
    for i, l in enumerate(host):
        d = res[i + 1]["dzdx"]
        if l["type"] == "pool":
            x32 = mat.to_numpy(res[i]["x"])
            assert bit_equal(mat.to_numpy(res[i + 1]["x"]), cpu_net.layer_forward(ref, glue, l, x32)), ("pool forward", i)
            dx, _ = cpu_net.layer_backward(ref, glue, l, x32, mat.to_numpy(d))
            assert bit_equal(mat.to_numpy(res[i]["dzdx"]), dx), ("pool backward", i)
            continue
        xi = _f64(mat, res[i]["x"])
        y = cpu_net.layer_forward(ref, glue, l, xi)
        got = res[i + 1]["x"].cpu().numpy() if l["type"] == "softmaxloss" else mat.to_numpy(res[i + 1]["x"])
        err = rel_l2(got, y)
        assert err < tol, ("layer %d (%s) forward" % (i, l["type"]), err)
        d = np.float64(d) if np.isscalar(d) else _f64(mat, d)
        dx, dw = cpu_net.layer_backward(ref, glue, l, xi, d)
        err = rel_l2(mat.to_numpy(res[i]["dzdx"]), dx)
        worst = max(worst, err)
        assert err < tol, ("layer %d (%s) dzdx" % (i, l["type"]), err)
        for j, w in enumerate(dw or []):
            if w is not None and res[i]["dzdw"][j] is not None:
                err = rel_l2(mat.to_numpy(res[i]["dzdw"][j]).ravel(), np.asarray(w).ravel())
                worst = max(worst, err)
                assert err < tol, ("layer %d (%s) dzdw[%d]" % (i, l["type"], j), err)
    return worst


def test_c2_cifar_net_batch_100(gpu, oracle, ref_blas):
    import torch
    import cpu_net
    from matconvnet_b200 import models, simplenn
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    rng = np.random.default_rng(202)
    net = models.cifar(seed=2)
    N = 100
    labels = rng.integers(1, 11, size=N).astype(np.float32)
    net["layers"][-1]["class"] = torch.from_numpy(labels).cuda()
    x = np.asfortranarray(rng.standard_normal((32, 32, 3, N)).astype(np.float32))
    res = simplenn.vl_simplenn(net, mat.from_numpy(x), 1.0, ctx=ctx)
    assert ctx.device_status() == 0
    full = cpu_net.simplenn(ref_blas, oracle, _host_layers(net["layers"], mat), np.asfortranarray(x, dtype=np.float64), np.float64(1.0))
    loss, want = float(res[-1]["x"].cpu()[0]), float(full[-1]["x"])
    assert abs(loss - want) <= 1e-5 * abs(want)
    _replay(res, mat, ref_blas, oracle, net["layers"])
    # the benchmark's schedule gives the same numbers bit for bit
    fused = simplenn.vl_simplenn(net, mat.from_numpy(x), 1.0, ctx=ctx, fuse_relu=True, conserve_memory=True)
    assert torch.equal(fused[-1]["x"], res[-1]["x"]) and torch.equal(fused[0]["dzdx"], res[0]["dzdx"])


def test_c3_resnet_bottleneck_batch_64(gpu, oracle, ref_blas):
    from matconvnet_b200 import simplenn
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    rng = np.random.default_rng(203)
    N, eps = 64, 1e-5
    he = lambda *s: np.asfortranarray((rng.standard_normal(s) * np.sqrt(2.0 / np.prod(s[:3]))).astype(np.float32))
    x = np.asfortranarray(rng.standard_normal((28, 28, 512, N), dtype=np.float32))
    dzdy = np.asfortranarray(rng.standard_normal((28, 28, 512, N), dtype=np.float32))
    layers = []
    for k, (fs, pad) in enumerate([((1, 1, 512, 128), 0), ((3, 3, 128, 128), 1), ((1, 1, 128, 512), 0)]):
        layers.append({"type": "conv", "weights": [mat.from_numpy(he(*fs)), None], "stride": 1, "pad": pad, "dilate": 1})
        layers.append({"type": "bnorm", "weights": [mat.from_numpy(np.ones((fs[3], 1), np.float32)),
                                                    mat.from_numpy(np.zeros((fs[3], 1), np.float32))], "epsilon": eps})
        if k < 2:
            layers.append({"type": "relu"})
    net = {"layers": layers}
    res = simplenn.vl_simplenn(net, mat.from_numpy(x), mat.from_numpy(dzdy), ctx=ctx)
    assert ctx.device_status() == 0
    _replay(res, mat, ref_blas, oracle, layers)
    # the identity branch (matlab/+dagnn/Sum.m:11-23): y = block(x) + x
    y = mat.empty((28, 28, 512, N))
    ctx.check(ctx.lib.vlb_sum(ctx.handle, mat.ptr(y), mat.ptr(res[-1]["x"]), mat.ptr(res[0]["x"]), y.numel()))
    assert bit_equal(mat.to_numpy(y), mat.to_numpy(res[-1]["x"]) + x)
    # backwardWithMoment: the moments handed back by the forward pass, given to the backward pass
    for i, l in enumerate(layers):
        if l["type"] != "bnorm":
            continue
        mom = res[i]["aux"]
        dx, dg, db, _ = nn.vl_nnbnorm(res[i]["x"], l["weights"][0], l["weights"][1], res[i + 1]["dzdx"], epsilon=eps,
                                      moments=mom, ctx=ctx)
        rdx, rdg, rdb, _ = ref_blas.bnorm_backward(_f64(mat, res[i]["x"]), _f64(mat, l["weights"][0]).ravel(),
                                                   _f64(mat, l["weights"][1]).ravel(), _f64(mat, res[i + 1]["dzdx"]), eps,
                                                   moments=_f64(mat, mom))
        assert rel_l2(mat.to_numpy(dx), rdx) < TOL, i
        assert rel_l2(mat.to_numpy(dg).ravel(), rdg.ravel()) < TOL and rel_l2(mat.to_numpy(db).ravel(), rdb.ravel()) < TOL, i


@pytest.mark.parametrize("name,hw,cin,cout", [("conv1_2", 224, 64, 64), ("conv3_2", 56, 256, 256), ("conv5_1", 14, 512, 512)])
def test_c4_vgg16_layers_backward_batch_64(gpu, ref_blas, name, hw, cin, cout):
    """Data, filter and bias gradients of three VGG-16 layers at the benchmark's batch: the longest filter-gradient sums
    (3.2 million terms per element on conv1_2), the persistent kernels' full tile walks, the 14x14 maps' ragged tiles."""
    import torch
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    ctx.reserve_workspace(3 << 30)
    g = torch.Generator(device="cuda").manual_seed(hw)
    x = mat.as_mat(torch.randn(hw, hw, cin, 64, device="cuda", generator=g))
    f = mat.as_mat(torch.randn(3, 3, cin, cout, device="cuda", generator=g) * (2.0 / (9 * cin)) ** 0.5)
    b = mat.zeros((1, cout))
    dy = mat.as_mat(torch.randn(hw, hw, cout, 64, device="cuda", generator=g))
    dx, df, db = nn.vl_nnconv(x, f, b, dy, pad=1, ctx=ctx)
    assert ctx.device_status() == 0
    rdx, rdf, rdb = ref_blas.conv_backward(_f64(mat, x), _f64(mat, f), _f64(mat, dy), (1, 1), (1, 1, 1, 1), (1, 1))
    assert rel_l2(mat.to_numpy(df), rdf) < TOL, name
    assert rel_l2(mat.to_numpy(db).ravel(), rdb.ravel()) < TOL, name
    assert rel_l2(mat.to_numpy(dx), rdx) < TOL, name
    # through the ReLU in front of the layer, as the benchmark runs it: bit for bit the two separate calls
    xr = nn.vl_nnrelu(x, ctx=ctx)
    dx2, df2, _ = nn.vl_nnconv(xr, f, b, dy, pad=1, through_relu=True, ctx=ctx)
    dx1, df1, _ = nn.vl_nnconv(xr, f, b, dy, pad=1, ctx=ctx)
    assert torch.equal(dx2, nn.vl_nnrelu(xr, dx1, ctx=ctx)) and torch.equal(df2, df1)


def _rois(rng, K, H, W, N, scale=1.0):
    """K boxes [image; u1; v1; u2; v2] (1-based, u along the width) with corners uniform in an H x W map and at least two
    pixels wide and high, K / N per image in random order; scale > 1 gives image coordinates for a 1/scale transform."""
    u1, v1 = rng.uniform(1, W - 2, K), rng.uniform(1, H - 2, K)
    u2, v2 = np.minimum(u1 + rng.uniform(2, W, K), W), np.minimum(v1 + rng.uniform(2, H, K), H)
    image = rng.permutation(np.arange(K) % N) + 1
    if scale != 1.0:
        # image coordinate c maps to feature coordinate s*(c - 1) + 1 under the transform [s 0 0 s 1-s 1-s]
        u1, v1, u2, v2 = [(c - 1) * scale + 1 for c in (u1, v1, u2, v2)]
    return np.asfortranarray(np.stack([image, u1, v1, u2, v2]).astype(np.float32))


def test_c5_fast_rcnn_head_full_size(gpu, oracle, ref_blas):
    import torch
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    ctx.reserve_workspace(3 << 30)
    rng = np.random.default_rng(205)
    H, W, Cc, N, K = 38, 50, 512, 2, 256
    x = np.asfortranarray(rng.standard_normal((H, W, Cc, N), dtype=np.float32))
    xd = mat.from_numpy(x)
    g = torch.Generator(device="cuda").manual_seed(205)
    f6 = mat.as_mat(torch.randn(7, 7, Cc, 4096, device="cuda", generator=g) * (2.0 / (49 * Cc)) ** 0.5)
    f7 = mat.as_mat(torch.randn(1, 1, 4096, 4096, device="cuda", generator=g) * (2.0 / 4096) ** 0.5)
    dz = mat.as_mat(torch.randn(1, 1, 4096, K, device="cuda", generator=g))
    for transform, scale in ((1.0, 1.0), (1.0 / 16, 16.0)):
        rois = _rois(rng, K, H, W, N, scale)
        rd = mat.from_numpy(rois)
        # bin geometry and pooled values: bit for bit
        bounds, images = nn.roipool_bounds(rd, (H, W, Cc, N), (7, 7), transform, ctx=ctx)
        rb, ri = oracle.roipool_bounds(rois, (H, W, Cc, N), (7, 7), transform)
        assert np.array_equal(mat.to_numpy(bounds), rb) and np.array_equal(images.cpu().numpy(), ri)
        p = nn.vl_nnroipool(xd, rd, subdivisions=(7, 7), transform=transform, method="max", ctx=ctx)
        assert bit_equal(mat.to_numpy(p), ref_blas.roipool_forward(x, rois, (7, 7), transform, "max"))
        if scale == 1.0:
            h6 = nn.vl_nnconv(p, f6, None, ctx=ctx)
            r6 = nn.vl_nnrelu(h6, ctx=ctx)
            h7 = nn.vl_nnconv(r6, f7, None, ctx=ctx)
            d6r, df7, _ = nn.vl_nnconv(r6, f7, None, dz, ctx=ctx)
            d6 = nn.vl_nnrelu(h6, d6r, ctx=ctx)
            dp, df6, _ = nn.vl_nnconv(p, f6, None, d6, ctx=ctx)
            assert ctx.device_status() == 0
            f764 = _f64(mat, f7)
            assert rel_l2(mat.to_numpy(h7), ref_blas.fc_forward(_f64(mat, r6), f764, None)) < TOL
            rdx, rdf, _ = ref_blas.fc_backward(_f64(mat, r6), f764, _f64(mat, dz), want=(True, True, False))
            assert rel_l2(mat.to_numpy(d6r), rdx) < TOL and rel_l2(mat.to_numpy(df7), rdf) < TOL
            del f764, rdf
            f664 = _f64(mat, f6)
            assert rel_l2(mat.to_numpy(h6), ref_blas.fc_forward(_f64(mat, p), f664, None)) < TOL
            rdx, rdf, _ = ref_blas.fc_backward(_f64(mat, p), f664, _f64(mat, d6), want=(True, True, False))
            assert rel_l2(mat.to_numpy(dp), rdx) < TOL and rel_l2(mat.to_numpy(df6), rdf) < TOL
            del f664, rdf
        else:
            dp = mat.as_mat(torch.randn(7, 7, Cc, K, device="cuda", generator=g))
        # ROI pooling backward with a real-valued derivative: the gather adds in the CPU loop's order, bit for bit,
        # and twice the same
        dx = nn.vl_nnroipool(xd, rd, dp, subdivisions=(7, 7), transform=transform, method="max", ctx=ctx)
        want = ref_blas.roipool_backward(x, rois, mat.to_numpy(dp), (7, 7), transform, "max")
        assert bit_equal(mat.to_numpy(dx), want)
        dx2 = nn.vl_nnroipool(xd, rd, dp, subdivisions=(7, 7), transform=transform, method="max", ctx=ctx)
        assert torch.equal(dx, dx2)
        dxa = nn.vl_nnroipool(xd, rd, dp, subdivisions=(7, 7), transform=transform, method="avg", ctx=ctx)
        assert bit_equal(mat.to_numpy(dxa), ref_blas.roipool_backward(x, rois, mat.to_numpy(dp), (7, 7), transform, "avg"))


def affine_grid(rng, Ho, Wo, Ng):
    """2 x Ho x Wo x Ng sampling grids of small rotations and scales through the reference's generator formula
    (matlab/+dagnn/AffineGridGenerator.m:36-57,106-118)."""
    xi, yi = np.linspace(-1, 1, Ho), np.linspace(-1, 1, Wo)
    yy, xx = np.meshgrid(xi, yi)
    base = np.stack([yy.ravel(), xx.ravel()], 1)
    grid = np.zeros((2, Ho, Wo, Ng), np.float32, order="F")
    for n in range(Ng):
        th, s = rng.uniform(-0.2, 0.2), rng.uniform(0.8, 1.2)
        A = s * np.array([[np.cos(th), -np.sin(th)], [np.sin(th), np.cos(th)]])
        grid[:, :, :, n] = (base @ A + rng.uniform(-0.1, 0.1, 2)).reshape(Wo, Ho, 2).transpose(2, 1, 0)
    return grid


def test_c5_bilinear_sampler_full_size(gpu, ref_blas):
    import torch
    nn, mat, ctx = gpu
    rng = np.random.default_rng(206)
    grid = affine_grid(rng, 64, 64, 256)
    x = np.asfortranarray(rng.standard_normal((64, 64, 32, 256), dtype=np.float32))
    dy = np.asfortranarray(rng.standard_normal((64, 64, 32, 256), dtype=np.float32))
    xd, gd, dyd = mat.from_numpy(x), mat.from_numpy(grid), mat.from_numpy(dy)
    assert bit_equal(mat.to_numpy(nn.vl_nnbilinearsampler(xd, gd, ctx=ctx)), ref_blas.sampler_forward(x, grid))
    dx, dgrid = nn.vl_nnbilinearsampler(xd, gd, dyd, ctx=ctx)
    rdx, rdg = ref_blas.sampler_backward(x, grid, dy)
    assert bit_equal(mat.to_numpy(dgrid), rdg)
    assert bit_equal(mat.to_numpy(dx), rdx)             # a gather in the CPU loop's order: no atomics, bit for bit
    dx2, _ = nn.vl_nnbilinearsampler(xd, gd, dyd, ctx=ctx)
    assert torch.equal(dx, dx2)
