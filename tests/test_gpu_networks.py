"""Whole-network forward+backward through the C ABI against the CPU checker: the five
configurations of the benchmark specification, with their layer geometries and value distributions,
at batch sizes / widths the scalar CPU checker finishes in seconds (the full sizes are exercised by
bench.py and the per-layer tests).  Synthetic seeded tensors stand in for MNIST, CIFAR-10, ILSVRC-2012
and VOC07 images.  Gradients are compared with the double-precision instantiation of the checker.
"""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _np_layers(layers, mat):
    """Host copies (float64) of a device layer list."""
    out = []
    for l in layers:
        m = dict(l)
        if "weights" in l:
            m["weights"] = [None if w is None else mat.to_numpy(w).astype(np.float64) for w in l["weights"]]
        if l.get("class") is not None and not isinstance(l["class"], np.ndarray):
            m["class"] = l["class"].cpu().numpy().astype(np.float64)
        out.append(m)
    return out


def _run_both(gpu, oracle, net, x, dzdy):
    import cpu_net
    from matconvnet_b200 import simplenn
    nn, mat, ctx = gpu
    xd = mat.from_numpy(x)
    dz = dzdy if np.isscalar(dzdy) else mat.from_numpy(dzdy)
    res = simplenn.vl_simplenn(net, xd, dz, ctx=ctx)
    assert ctx.device_status() == 0
    ref = cpu_net.simplenn(oracle, oracle, _np_layers(net["layers"], mat), np.asfortranarray(x, dtype=np.float64),
                           np.float64(dzdy) if np.isscalar(dzdy) else np.asfortranarray(dzdy, dtype=np.float64))
    return res, ref


def _compare(res, ref, mat, layers, tol=TOL):
    worst = 0.0
    for i, l in enumerate(layers):
        if res[i]["dzdw"] is not None:
            for j, (a, b) in enumerate(zip(res[i]["dzdw"], ref[i]["dzdw"])):
                if a is None or j > 1:
                    continue
                err = rel_l2(mat.to_numpy(a).ravel(), np.asarray(b).ravel())
                worst = max(worst, err)
                assert err < tol, ("layer %d (%s) dzdw[%d]" % (i, l["type"], j), err)
    err = rel_l2(mat.to_numpy(res[0]["dzdx"]), ref[0]["dzdx"])
    assert err < tol, ("dzdx of the input", err)
    return max(worst, err)


def _replay(res, mat, oracle, layers, tol=TOL):
    """Layer-by-layer check inside the network: the checker recomputes every layer from the GPU's own input
    and output derivative of that layer, so a ReLU or max-pool decision that flips on a near-zero activation
    cannot leak into the comparison of the layers below it."""
    import cpu_net
    host = _np_layers(layers, mat)
    f64 = lambda t: np.asfortranarray(mat.to_numpy(t), dtype=np.float64)
    for i, l in enumerate(host):
        xi = f64(res[i]["x"])
        y = cpu_net.layer_forward(oracle, oracle, l, xi)
        got = res[i + 1]["x"].cpu().numpy() if l["type"] == "softmaxloss" else mat.to_numpy(res[i + 1]["x"])
        assert rel_l2(got, y) < tol, ("layer %d (%s) forward" % (i, l["type"]), rel_l2(got, y))
        d = res[i + 1]["dzdx"]
        d = np.float64(d) if np.isscalar(d) else f64(d)
        dx, dw = cpu_net.layer_backward(oracle, oracle, l, xi, d)
        err = rel_l2(mat.to_numpy(res[i]["dzdx"]), dx)
        assert err < tol, ("layer %d (%s) dzdx" % (i, l["type"]), err)
        for j, w in enumerate(dw or []):
            if w is not None and res[i]["dzdw"][j] is not None:
                err = rel_l2(mat.to_numpy(res[i]["dzdw"][j]).ravel(), np.asarray(w).ravel())
                assert err < tol, ("layer %d (%s) dzdw[%d]" % (i, l["type"], j), err)


def test_c1_lenet_block_backward(gpu, oracle):
    """conv 5x5x1x20 -> maxpool 2 -> conv 5x5x20x50 -> maxpool 2 on 28x28x1x100, U(0,1) input, N(0,0.01^2)
    filters, zero biases, dzdy N(0,1) (reference examples/mnist/cnn_mnist_init.m:10-29)."""
    from matconvnet_b200 import models
    nn, mat, ctx = gpu
    rng = np.random.default_rng(101)
    net = models.lenet_block(seed=1)
    x = np.asfortranarray(rng.uniform(0, 1, (28, 28, 1, 100)).astype(np.float32))
    dzdy = np.asfortranarray(rng.standard_normal((4, 4, 50, 100)).astype(np.float32))
    res, ref = _run_both(gpu, oracle, net, x, dzdy)
    assert tuple(res[-1]["x"].shape) == (4, 4, 50, 100)
    _compare(res, ref, mat, net["layers"])
    # the pooling layers' derivatives as well (arg-max routing through both pools)
    for i in (1, 3):
        assert rel_l2(mat.to_numpy(res[i]["dzdx"]), ref[i]["dzdx"]) < TOL


def test_c2_cifar_net(gpu, oracle):
    """The CIFAR-10 network of the reference (examples/cifar/cnn_cifar_init.m:11-65): 5x5 convolutions with
    pad 2, overlapping max / average pooling with asymmetric padding, conv-as-FC tail, softmax loss."""
    from matconvnet_b200 import models
    import torch
    nn, mat, ctx = gpu
    rng = np.random.default_rng(102)
    net = models.cifar(seed=2)
    N = 20
    labels = rng.integers(1, 11, size=N).astype(np.float32)
    net["layers"][-1]["class"] = torch.from_numpy(labels).cuda()
    x = np.asfortranarray(rng.standard_normal((32, 32, 3, N)).astype(np.float32))
    res, ref = _run_both(gpu, oracle, net, x, 1.0)
    loss = float(res[-1]["x"].cpu()[0])
    assert abs(loss - float(ref[-1]["x"])) <= 1e-5 * abs(float(ref[-1]["x"]))
    # end to end a ReLU / max-pool decision on an activation within rounding of a tie may flip and change the gradients
    # below it by whole elements: loose bound end to end, the per-layer bound in the replay
    _compare(res, ref, mat, net["layers"], tol=5e-3)
    _replay(res, mat, oracle, net["layers"])


def test_c3_resnet_bottleneck(gpu, oracle):
    """ResNet-50 stage-3 bottleneck on 28x28x512: conv1x1 512->128, bnorm, relu, conv3x3 128->128, bnorm, relu,
    conv1x1 128->512, bnorm, plus the identity (reference examples/imagenet/cnn_imagenet_init_resnet.m:16-115);
    bnorm backward in both modes (computed and given moments)."""
    from matconvnet_b200 import simplenn
    nn, mat, ctx = gpu
    rng = np.random.default_rng(103)
    N, eps = 4, 1e-5
    he = lambda *s: np.asfortranarray((rng.standard_normal(s) * np.sqrt(2.0 / np.prod(s[:3]))).astype(np.float32))
    x = np.asfortranarray(rng.standard_normal((28, 28, 512, N)).astype(np.float32))
    dzdy = np.asfortranarray(rng.standard_normal((28, 28, 512, N)).astype(np.float32))
    specs = [((1, 1, 512, 128), 0), ((3, 3, 128, 128), 1), ((1, 1, 128, 512), 0)]
    layers = []
    for k, (fs, pad) in enumerate(specs):
        layers.append({"type": "conv", "weights": [mat.from_numpy(he(*fs)), None], "stride": 1, "pad": pad, "dilate": 1})
        layers.append({"type": "bnorm", "weights": [mat.from_numpy(np.ones((fs[3], 1), np.float32)),
                                                    mat.from_numpy(np.zeros((fs[3], 1), np.float32))], "epsilon": eps})
        if k < 2:
            layers.append({"type": "relu"})
    net = {"layers": layers}
    res, ref = _run_both(gpu, oracle, net, x, dzdy)
    # sum with the identity branch (reference matlab/+dagnn/Sum.m:11-23): y = block(x) + x, dx = dblock + dzdy
    y = mat.empty((28, 28, 512, N))
    ctx.check(ctx.lib.vlb_sum(ctx.handle, mat.ptr(y), mat.ptr(res[-1]["x"]), mat.ptr(res[0]["x"]), y.numel()))
    assert rel_l2(mat.to_numpy(y), ref[-1]["x"] + x) < TOL
    for i, l in enumerate(layers):
        if l["type"] == "conv":
            assert rel_l2(mat.to_numpy(res[i]["dzdw"][0]), ref[i]["dzdw"][0]) < TOL, i
        if l["type"] == "bnorm":
            for j in range(3):      # dgamma, dbeta, moments
                assert rel_l2(mat.to_numpy(res[i]["dzdw"][j]).ravel(), np.asarray(ref[i]["dzdw"][j]).ravel()) < TOL, (i, j)
    dx_total = mat.to_numpy(res[0]["dzdx"]).astype(np.float64) + dzdy
    assert rel_l2(dx_total, ref[0]["dzdx"] + dzdy) < TOL


def test_c3_bnorm_given_moments_full_size(gpu, oracle):
    """backwardWithMoment at the block's 28x28x128 size agrees with backward (reference xtest/suite/nnbnorm.m:53-79)."""
    nn, mat, ctx = gpu
    import torch
    x = mat.as_mat(torch.randn(28, 28, 128, 64, device="cuda"))
    dy = mat.as_mat(torch.randn(28, 28, 128, 64, device="cuda"))
    g = mat.as_mat(torch.rand(128, 1, device="cuda") + 0.5)
    b = mat.zeros((128, 1))
    dx, dg, db, mom = nn.vl_nnbnorm(x, g, b, dy, epsilon=1e-5)
    dx2, dg2, db2, _ = nn.vl_nnbnorm(x, g, b, dy, epsilon=1e-5, moments=mom)
    for a, r in ((dx2, dx), (dg2, dg), (db2, db)):
        assert rel_l2(mat.to_numpy(a).ravel(), mat.to_numpy(r).ravel()) < 1e-6


def test_c4_vgg16_topology_small(gpu, oracle):
    """VGG-16's layer chain (13 conv 3x3 pad 1 + relu, five 2x2 max-pools, three conv-as-FC layers, softmax
    loss) on 64x64 inputs with the FC widths reduced, batch 2: every filter and bias gradient and the input
    gradient against the checker."""
    import torch
    from matconvnet_b200 import mat as M
    nn, mat, ctx = gpu
    rng = np.random.default_rng(104)
    he = lambda *s: np.asfortranarray((rng.standard_normal(s) * np.sqrt(2.0 / np.prod(s[:3]))).astype(np.float32))
    layers, cin = [], 3
    for cout, reps in [(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]:
        for _ in range(reps):
            layers += [{"type": "conv", "weights": [M.from_numpy(he(3, 3, cin, cout)), M.zeros((1, cout))], "stride": 1, "pad": 1, "dilate": 1},
                       {"type": "relu"}]
            cin = cout
        layers.append({"type": "pool", "method": "max", "pool": [2, 2], "stride": 2, "pad": 0})
    for fs, relu in [((2, 2, 512, 256), True), ((1, 1, 256, 256), True), ((1, 1, 256, 100), False)]:
        layers.append({"type": "conv", "weights": [M.from_numpy(he(*fs)), M.zeros((1, fs[3]))], "stride": 1, "pad": 0, "dilate": 1})
        if relu:
            layers.append({"type": "relu"})
    labels = rng.integers(1, 101, size=2).astype(np.float32)
    layers.append({"type": "softmaxloss", "class": torch.from_numpy(labels).cuda()})
    net = {"layers": layers}
    x = np.asfortranarray(rng.standard_normal((64, 64, 3, 2)).astype(np.float32))
    res, ref = _run_both(gpu, oracle, net, x, 1.0)
    # 16 contractions deep.  End to end the forward error compounds (the loss inherits the absolute error of logits
    # of magnitude ~10) and one ReLU mask that flips on an activation within rounding of zero changes the gradients
    # below it by a whole element, so the end-to-end bound is loose; the per-layer bound holds in the replay.
    assert abs(float(res[-1]["x"].cpu()[0]) - float(ref[-1]["x"])) <= 5e-5 * abs(float(ref[-1]["x"]))
    _compare(res, ref, mat, layers, tol=2e-3)
    _replay(res, mat, oracle, layers)


def test_c4_vgg16_full_size_vs_compiled_reference(gpu, oracle):
    """The real VGG-16 (224x224 inputs, 4096-wide fully connected layers, 1000 classes) at batch 2 against the
    reference's own compiled CPU backend in double precision, its GEMMs routed to a threaded BLAS so that the 62 GFLOP
    finish in seconds: the loss, and every layer replayed from the GPU's own input and output derivative."""
    import os
    import torch
    import cpu_net
    import oracle as O
    from matconvnet_b200 import models, simplenn
    nn, mat, ctx = gpu
    ref = O.reference()
    if ref is None or not O.reference_use_openblas(os.cpu_count() or 1):
        pytest.skip("the compiled reference backend or a threaded BLAS for it is not available")
    try:
        ctx.set_precision(0)
        ctx.reserve_workspace(3 << 30)
        rng = np.random.default_rng(106)
        net = models.vgg16(seed=3)
        labels = rng.integers(1, 1001, size=2).astype(np.float32)
        net["layers"][-1]["class"] = torch.from_numpy(labels).cuda()
        x = np.asfortranarray(rng.standard_normal((224, 224, 3, 2)).astype(np.float32))
        res = simplenn.vl_simplenn(net, mat.from_numpy(x), 1.0, ctx=ctx)
        assert ctx.device_status() == 0
        host = _np_layers(net["layers"], mat)
        f64 = lambda t: np.asfortranarray(mat.to_numpy(t), dtype=np.float64)
        full = cpu_net.simplenn(ref, oracle, host, np.asfortranarray(x, dtype=np.float64), np.float64(1.0), conserve_memory=True)
        loss, loss_ref = float(res[-1]["x"].cpu()[0]), float(full[-1]["x"])
        assert abs(loss - loss_ref) <= 5e-5 * abs(loss_ref), (loss, loss_ref)
        del full
        for i, l in enumerate(host):
            xi = f64(res[i]["x"])
            y = cpu_net.layer_forward(ref, oracle, l, xi)
            got = res[i + 1]["x"].cpu().numpy() if l["type"] == "softmaxloss" else mat.to_numpy(res[i + 1]["x"])
            assert rel_l2(got, y) < TOL, ("layer %d (%s) forward" % (i, l["type"]), rel_l2(got, y))
            d = res[i + 1]["dzdx"]
            d = np.float64(d) if np.isscalar(d) else f64(d)
            dx, dw = cpu_net.layer_backward(ref, oracle, l, xi, d)
            assert rel_l2(mat.to_numpy(res[i]["dzdx"]), dx) < TOL, ("layer %d (%s) dzdx" % (i, l["type"]),)
            for j, w in enumerate(dw or []):
                if w is not None and res[i]["dzdw"][j] is not None:
                    err = rel_l2(mat.to_numpy(res[i]["dzdw"][j]).ravel(), np.asarray(w).ravel())
                    assert err < TOL, ("layer %d (%s) dzdw[%d]" % (i, l["type"], j), err)
        # the benchmark's schedule (ReLU fused into the layers around it, derivatives dropped as they are used) gives the
        # same loss and the same gradients bit for bit
        fused = simplenn.vl_simplenn(net, mat.from_numpy(x), 1.0, ctx=ctx, fuse_relu=True, conserve_memory=True)
        assert torch.equal(fused[-1]["x"], res[-1]["x"]) and torch.equal(fused[0]["dzdx"], res[0]["dzdx"])
        for a, c in zip(res, fused):
            for u, v in zip(a["dzdw"] or [], c["dzdw"] or []):
                assert (u is None and v is None) or torch.equal(u, v)
    finally:
        O.reference_use_plain_blas()


def test_c5_fast_rcnn_head_and_sampler(gpu, oracle):
    """ROI max-pool 7x7 on a 38x50x512x2 map with ROIs in feature-map coordinates, two conv-as-FC layers
    (widths reduced for the CPU checker), backward; and the bilinear sampler backward with an affine grid of
    small rotations and scales (reference examples/fast_rcnn/fast_rcnn_init.m:53-61,
    matlab/+dagnn/AffineGridGenerator.m:36-57)."""
    nn, mat, ctx = gpu
    rng = np.random.default_rng(105)
    H, W, Cc, N, K = 38, 50, 512, 2, 32
    x = np.asfortranarray(rng.standard_normal((H, W, Cc, N)).astype(np.float32))
    u1, v1 = rng.uniform(1, W - 2, K), rng.uniform(1, H - 2, K)
    u2, v2 = np.minimum(u1 + rng.uniform(2, W, K), W), np.minimum(v1 + rng.uniform(2, H, K), H)
    rois = np.asfortranarray(np.stack([np.arange(K) % N + 1, u1, v1, u2, v2]).astype(np.float32))
    f6 = np.asfortranarray((rng.standard_normal((7, 7, Cc, 64)) * np.sqrt(2.0 / (49 * Cc))).astype(np.float32))
    f7 = np.asfortranarray((rng.standard_normal((1, 1, 64, 48)) * np.sqrt(2.0 / 64)).astype(np.float32))
    dz = np.asfortranarray(rng.standard_normal((1, 1, 48, K)).astype(np.float32))
    xd, rd, f6d, f7d, dzd = (mat.from_numpy(a) for a in (x, rois, f6, f7, dz))
    p = nn.vl_nnroipool(xd, rd, subdivisions=(7, 7), method="max")
    h6 = nn.vl_nnconv(p, f6d, None)
    r6 = nn.vl_nnrelu(h6)
    h7 = nn.vl_nnconv(r6, f7d, None)
    d6r, df7, _ = nn.vl_nnconv(r6, f7d, None, dzd)
    d6 = nn.vl_nnrelu(h6, d6r)
    dp, df6, _ = nn.vl_nnconv(p, f6d, None, d6)
    dx = nn.vl_nnroipool(xd, rd, dp, subdivisions=(7, 7), method="max")
    x64, f664, f764 = x.astype(np.float64), f6.astype(np.float64), f7.astype(np.float64)
    pr = oracle.roipool_forward(x64, rois.astype(np.float64), (7, 7), 1.0, "max")
    h6r = oracle.conv_forward(pr, f664, None)
    r6r = oracle.relu_forward(h6r)
    d6rr, df7r, _ = oracle.conv_backward(r6r, f764, dz.astype(np.float64), want=(True, True, False))
    d6ref = oracle.relu_backward(h6r, d6rr)
    dpr, df6r, _ = oracle.conv_backward(pr, f664, d6ref, want=(True, True, False))
    dxr = oracle.roipool_backward(x64, rois.astype(np.float64), dpr, (7, 7), 1.0, "max")
    assert np.array_equal(mat.to_numpy(p), pr.astype(np.float32))          # pooled values: bit-exact routing
    assert rel_l2(mat.to_numpy(h7), oracle.conv_forward(r6r, f764, None)) < TOL
    assert rel_l2(mat.to_numpy(df7), df7r) < TOL and rel_l2(mat.to_numpy(df6), df6r) < TOL
    assert rel_l2(mat.to_numpy(dx), dxr) < TOL
    # sampler: 64x64x8 images, two grids per image
    Hs = Ws = 64
    xi, yi = np.linspace(-1, 1, Hs), np.linspace(-1, 1, Ws)
    yy, xx = np.meshgrid(xi, yi)
    base = np.stack([yy.ravel(), xx.ravel()], 1)
    Ng, Ns = 8, 4
    grid = np.zeros((2, Hs, Ws, Ng), np.float32, order="F")
    for n in range(Ng):
        th, s = rng.uniform(-0.2, 0.2), rng.uniform(0.8, 1.2)
        A = s * np.array([[np.cos(th), -np.sin(th)], [np.sin(th), np.cos(th)]])
        grid[:, :, :, n] = (base @ A + rng.uniform(-0.1, 0.1, 2)).reshape(Ws, Hs, 2).transpose(2, 1, 0)
    xs = np.asfortranarray(rng.standard_normal((Hs, Ws, 8, Ns)).astype(np.float32))
    dys = np.asfortranarray(rng.standard_normal((Hs, Ws, 8, Ng)).astype(np.float32))
    dxs, dgs = nn.vl_nnbilinearsampler(mat.from_numpy(xs), mat.from_numpy(grid), mat.from_numpy(dys))
    dxr, dgr = oracle.sampler_backward(xs, grid, dys)
    assert rel_l2(mat.to_numpy(dxs), dxr) < 1e-6
    assert np.array_equal(mat.to_numpy(dgs), dgr)


def test_fused_relu_is_bit_identical(gpu):
    """vl_nnconv(..., relu=True) against vl_nnrelu(vl_nnconv(...)) for every forward path (tensor-memory kernel, fully
    connected with and without split reduction, image-end kernel, CUDA-core fallback); the backward pass through a ReLU
    before a convolution or pooling layer (through_relu=True) against the two separate calls; and whole networks run
    with fuse_relu against the plain schedule: same loss and same gradients, bit for bit."""
    import torch
    from matconvnet_b200 import models, simplenn
    nn, mat, ctx = gpu
    ctx.set_precision(0)
    g = torch.Generator(device="cuda").manual_seed(5)
    cases = [((20, 24, 32, 3), (3, 3, 32, 48), dict(pad=1)),                 # tensor-memory kernel
             ((64, 48, 3, 2), (3, 3, 3, 64), dict(pad=1)),                   # image-end kernel
             ((7, 7, 64, 5), (7, 7, 64, 40), dict()),                        # fully connected, split reduction
             ((1, 1, 96, 6), (1, 1, 96, 20), dict()),                        # fully connected, one pass
             ((10, 10, 8, 2), (3, 3, 2, 12), dict(pad=1)),                   # filter groups: CUDA-core fallback
             ((17, 15, 6, 3), (3, 3, 6, 10), dict(stride=2, pad=(1, 0, 1, 1))),
             # more tiles than SMs, so that each CTA walks several tiles and the data gradient fetches its ReLU mask as
             # bits while a tile is computed: 32 columns and few chains per tile; 128 columns and 18 chains per tile
             ((48, 48, 32, 16), (3, 3, 32, 48), dict(pad=1)),
             ((56, 56, 128, 8), (3, 3, 128, 256), dict(pad=1)),
             ((52, 50, 72, 9), (3, 3, 72, 40), dict(pad=1))]          # ragged: 72 of 128 columns, last row tile partial
    for xs, fs, kw in cases:
        for prec in (0, 1):                  # 3xTF32 and plain TF32 (one chain per issuer and tile)
            ctx.set_precision(prec)
            x = mat.as_mat(torch.randn(*xs, device="cuda", generator=g))
            f = mat.as_mat(torch.randn(*fs, device="cuda", generator=g) * 0.1)
            b = mat.as_mat(torch.randn(1, fs[3], device="cuda", generator=g))
            want = nn.vl_nnrelu(nn.vl_nnconv(x, f, b, **kw))
            got = nn.vl_nnconv(x, f, b, relu=True, **kw)
            assert torch.equal(got, want), (xs, fs)
            # backward through the ReLU before the convolution: x is that ReLU's output
            xr = nn.vl_nnrelu(x)
            dzdy = mat.as_mat(torch.randn(*mat.shape4(want), device="cuda", generator=g))
            dx, df, db = nn.vl_nnconv(xr, f, b, dzdy, **kw)
            dx2, df2, db2 = nn.vl_nnconv(xr, f, b, dzdy, through_relu=True, **kw)
            assert torch.equal(dx2, nn.vl_nnrelu(xr, dx)), (xs, fs)
            assert torch.equal(df2, df) and torch.equal(db2, db), (xs, fs)
    ctx.set_precision(0)
    pools = [((24, 20, 5, 3), (2, 2), dict(stride=2)),                        # 2x2 kernel, two outputs per thread
             ((10, 6, 4, 2), (2, 2), dict(stride=2)),                         # 2x2 kernel, one output per thread
             ((13, 11, 3, 2), (3, 3), dict(stride=2, pad=(0, 1, 0, 1))),      # generic kernel
             ((9, 9, 2, 2), (3, 2), dict(stride=1, pad=1))]
    for xs, pool, kw in pools:
        for method in ("max", "avg"):
            xr = nn.vl_nnrelu(mat.as_mat(torch.randn(*xs, device="cuda", generator=g)))
            y = nn.vl_nnpool(xr, pool, method=method, **kw)
            dzdy = mat.as_mat(torch.randn(*mat.shape4(y), device="cuda", generator=g))
            want = nn.vl_nnrelu(xr, nn.vl_nnpool(xr, pool, dzdy, method=method, **kw))
            got = nn.vl_nnpool(xr, pool, dzdy, method=method, through_relu=True, **kw)
            assert torch.equal(got, want), (xs, pool, method)
    labels = torch.randint(1, 11, (8,), device="cuda", generator=g).float()
    # a VGG-like chain (conv 3x3 + relu pairs, 2x2 max-pools, conv-as-FC + relu): every ReLU sits before a convolution,
    # a pooling or a fully connected layer
    rng = np.random.default_rng(9)
    cv = lambda fh, cin, cout, pad: models._conv(rng, fh, fh, cin, cout, 1, pad)
    vgg = [cv(3, 3, 32, 1), models._relu(), cv(3, 32, 32, 1), models._relu(), models._pool("max", 2, 2),
           cv(3, 32, 64, 1), models._relu(), cv(3, 64, 64, 1), models._relu(), models._pool("max", 2, 2),
           cv(8, 64, 64, 0), models._relu(), cv(1, 64, 10, 0), {"type": "softmaxloss", "class": None}]
    nets = [(models.cifar(seed=4), (32, 32, 3, 8)), ({"layers": vgg}, (32, 32, 3, 8))]
    for net, xs in nets:
        net["layers"][-1]["class"] = labels
        x = mat.as_mat(torch.randn(*xs, device="cuda", generator=g))
        plain = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx)
        fused = simplenn.vl_simplenn(net, x, 1.0, ctx=ctx, fuse_relu=True)
        assert torch.equal(plain[-1]["x"], fused[-1]["x"])
        assert torch.equal(plain[0]["dzdx"], fused[0]["dzdx"])
        for a, c in zip(plain, fused):
            if torch.is_tensor(c["dzdx"]):      # the fused schedule keeps no derivative between a ReLU and the layer after
                assert torch.equal(a["dzdx"], c["dzdx"])
            if a["dzdw"] is not None:
                for u, v in zip(a["dzdw"], c["dzdw"]):
                    assert (u is None and v is None) or torch.equal(u, v)
