"""Pins the CPU checker (oracle/mcn_oracle.c) before anything is judged against it:

1. against golden vectors computed by the reference's own compiled CPU code
   (tests/golden/*.npz, generator tests/golden/make_golden.py);
2. against the compiled reference directly, where its library is present;
3. against the known-answer identities of the reference's MATLAB test-suite, restated:
   ROI identity (xtest/suite/nnroipool.m:40-49), bnorm closed form (nnbnorm.m:9-31),
   given-moments == computed-moments (nnbnorm.m:53-79), avg-pool == convolution with a
   constant filter (nnpool.m:34-49), stride == subsampling of stride 1 (nnconv.m:88-107),
   pad == crop (nnconv.m:109-125), groups == block-diagonal dense filters (nnconv.m:144-161),
   forward-difference derivative checks (nntest.m:94-108).
"""
import numpy as np
import pytest

from conftest import bit_equal, cases_of, load_golden, rel_l2


def test_conv_golden(oracle):
    g = load_golden("conv")
    for c in cases_of(g):
        prm = g[c + ".prm"]
        kw = dict(stride=tuple(prm[0:2]), pad=tuple(prm[2:6]), dilate=tuple(prm[6:8]))
        y = oracle.conv_forward(g[c + ".x"], g[c + ".f"], g[c + ".b"], **kw)
        dx, df, db = oracle.conv_backward(g[c + ".x"], g[c + ".f"], g[c + ".dy"], **kw)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(got, g[c + "." + name]) < 1e-6, (c, name)
            assert rel_l2(got, g[c + "." + name + "64"]) < 1e-5, (c, name)


def test_convt_golden(oracle):
    g = load_golden("convt")
    for c in cases_of(g):
        prm = [int(v) for v in g[c + ".prm"]]
        kw = dict(upsample=tuple(prm[0:2]), crop=tuple(prm[2:6]), num_groups=prm[6])
        y = oracle.convt_forward(g[c + ".x"], g[c + ".f"], g[c + ".b"], **kw)
        dx, df, db = oracle.convt_backward(g[c + ".x"], g[c + ".f"], g[c + ".dy"], **kw)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(got, g[c + "." + name]) < 1e-6, (c, name)
            assert rel_l2(got, g[c + "." + name + "64"]) < 1e-5, (c, name)
    # upsample 1, no crop: the transposed convolution is the convolution of the zero-padded input with the flipped filters
    # whose last two dimensions are exchanged (matlab/vl_nnconvt.m)
    c = "up1_is_full_correlation"
    x, f, b = g[c + ".x"], g[c + ".f"], g[c + ".b"]
    ft = np.asfortranarray(np.transpose(f[::-1, ::-1], (0, 1, 3, 2)))
    assert rel_l2(oracle.conv_forward(x, ft, b, pad=(2, 2, 2, 2)), g[c + ".y"]) < 1e-6


def test_fc_golden(oracle):
    g = load_golden("fc")
    for c in cases_of(g):
        y = oracle.fc_forward(g[c + ".x"], g[c + ".f"], g[c + ".b"])
        dx, df, db = oracle.fc_backward(g[c + ".x"], g[c + ".f"], g[c + ".dy"])
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(got, g[c + "." + name]) < 1e-6, (c, name)
        # the gateway routes 1x1-output convolutions here: both routes must agree
        assert rel_l2(oracle.conv_forward(g[c + ".x"], g[c + ".f"], g[c + ".b"]), y) < 1e-6


def test_bias_golden(oracle):
    g = load_golden("bias")
    for i, (ym, hx, xm, hb, bm) in enumerate(g["fwd_args"]):
        y = oracle.bias_forward(g["y0"], ym, g["x"] if hx else None, xm, g["b"] if hb else None, bm)
        assert bit_equal(y, g["fwd%d" % i]), i
    for i, (dxm, dbm, xm, bm) in enumerate(g["bwd_args"]):
        dx, db = oracle.bias_backward(g["dx0"], dxm, g["db0"], dbm, xm, bm, g["dy"])
        assert rel_l2(dx, g["bwd%d.dx" % i]) < 1e-7 and rel_l2(db, g["bwd%d.db" % i]) < 1e-6


def test_bnorm_golden(oracle):
    g = load_golden("bnorm")
    for c in cases_of(g):
        x, gg, b, dy, eps = g[c + ".x"], g[c + ".g"], g[c + ".b"], g[c + ".dy"], float(g[c + ".eps"])
        y, mom = oracle.bnorm_forward(x, gg, b, eps)
        assert bit_equal(y, g[c + ".y"]) and bit_equal(mom, g[c + ".mom"]), c
        ym, _ = oracle.bnorm_forward(x, gg, b, eps, moments=g[c + ".mom"])
        assert bit_equal(ym, g[c + ".ym"]), c
        dx, dg, db, mom2 = oracle.bnorm_backward(x, gg, b, dy, eps)
        assert bit_equal(dx, g[c + ".dx"]) and bit_equal(dg, g[c + ".dg"]) and bit_equal(db, g[c + ".db"]), c
        assert bit_equal(mom2, g[c + ".mom"]), c
        dxm, dgm, dbm, _ = oracle.bnorm_backward(x, gg, b, dy, eps, moments=g[c + ".mom"])
        assert bit_equal(dxm, g[c + ".dxm"]) and bit_equal(dgm, g[c + ".dgm"]) and bit_equal(dbm, g[c + ".dbm"]), c


def test_pool_golden(oracle):
    g = load_golden("pool")
    for c in cases_of(g):
        if c == "ties":
            continue
        prm = g[c + ".prm"]
        kw = dict(pool=tuple(prm[0:2]), stride=tuple(prm[2:4]), pad=tuple(prm[4:8]))
        for m in ("max", "avg"):
            assert bit_equal(oracle.pool_forward(g[c + ".x"], method=m, **kw), g["%s.%s.y" % (c, m)]), (c, m)
            assert bit_equal(oracle.pool_backward(g[c + ".x"], g["%s.%s.dy" % (c, m)], method=m, **kw),
                             g["%s.%s.dx" % (c, m)]), (c, m)
    kw = dict(pool=(2, 2), stride=(2, 2), pad=(0, 0, 0, 0), method="max")
    assert bit_equal(oracle.pool_forward(g["ties.x"], **kw), g["ties.max.y"])
    dx = oracle.pool_backward(g["ties.x"], g["ties.dy"], **kw)
    assert bit_equal(dx, g["ties.max.dx"])
    # first of equal maxima (column-major scan) gets the gradient; the all -inf window routes nowhere
    assert dx[0, 0, 0, 0] == 1.0 and dx[2:, :2].sum() == 0.0 and dx[1, 2, 0, 0] == 3.0


def _roi_keys(g):
    return sorted({k[:-2] for k in g if k.endswith(".y")})


def test_roipool_golden(oracle):
    g = load_golden("roipool")
    x = g["x"]
    for key in _roi_keys(g):
        tname, sub, method = key.split(".")
        sub = tuple(int(v) for v in sub.split("x"))
        rois, tf = g["rois." + tname], g["tf." + tname]
        assert bit_equal(oracle.roipool_forward(x, rois, sub, tf, method), g[key + ".y"]), key
        assert bit_equal(oracle.roipool_backward(x, rois, g[key + ".dy"], sub, tf, method), g[key + ".dx"]), key
        assert bit_equal(oracle.roipool_backward(x, rois, g[key + ".dyi"], sub, tf, method), g[key + ".dxi"]), key


def test_sampler_golden(oracle):
    g = load_golden("sampler")
    for c in cases_of(g):
        assert bit_equal(oracle.sampler_forward(g[c + ".x"], g[c + ".grid"]), g[c + ".y"]), c
        dx, dgrid = oracle.sampler_backward(g[c + ".x"], g[c + ".grid"], g[c + ".dy"])
        assert bit_equal(dx, g[c + ".dx"]) and bit_equal(dgrid, g[c + ".dgrid"]), c


def test_against_compiled_reference(oracle, reference_backend):
    """Fresh seeded inputs through both CPU backends, when the reference library exists."""
    ref = reference_backend
    if ref is None:
        pytest.skip("oracle/_ref/libmcn_ref.so not built on this machine")
    rng = np.random.default_rng(7)
    rn = lambda *s: np.asfortranarray(rng.standard_normal(s).astype(np.float32))
    x, f, b = rn(10, 9, 6, 2), rn(3, 3, 3, 4), rn(4)
    kw = dict(stride=(2, 1), pad=(1, 0, 2, 1), dilate=(1, 2))
    y = ref.conv_forward(x, f, b, **kw)
    assert rel_l2(oracle.conv_forward(x, f, b, **kw), y) < 1e-6
    dy = rn(*y.shape)
    for a, r in zip(oracle.conv_backward(x, f, dy, **kw), ref.conv_backward(x, f, dy, **kw)):
        assert rel_l2(a, r) < 1e-6
    xb, g, bb, dyb = rn(5, 6, 3, 4), rn(3), rn(3), rn(5, 6, 3, 4)
    for a, r in zip(oracle.bnorm_backward(xb, g, bb, dyb), ref.bnorm_backward(xb, g, bb, dyb)):
        assert bit_equal(a, r)
    xs = rn(8, 7, 3, 2)
    grid = np.asfortranarray(rng.uniform(-1.2, 1.2, (2, 5, 6, 4)).astype(np.float32))
    assert bit_equal(oracle.sampler_forward(xs, grid), ref.sampler_forward(xs, grid))


# ----------------------------------------------------------------- known-answer identities
def test_roipool_identity(oracle):
    x = np.asfortranarray((np.arange(2, 11)[:, None] * np.arange(1, 11)[None, :]).astype(np.float32)).reshape(9, 10, 1, 1, order="F")
    rois = np.array([[1, 1, 1, 9, 10]], np.float32).T
    T = np.array([[0, 1, 0], [1, 0, 0]], np.float64)
    for m in ("max", "avg"):
        y = oracle.roipool_forward(x, rois, (9, 10), T, m)
        assert np.array_equal(y, x), m


def test_bnorm_closed_form(oracle):
    rng = np.random.default_rng(3)
    for shape in [(2, 2, 1, 2), (8, 17, 3, 7), (13, 8, 4, 2)]:
        x = np.asfortranarray(rng.standard_normal(shape)) * 3 + 1
        g, b = rng.standard_normal(shape[2]), rng.standard_normal(shape[2])
        eps = 1e-3
        y, m = oracle.bnorm_forward(x, g, b, eps)          # float64 instantiation
        mu = x.mean(axis=(0, 1, 3))
        sigma = np.sqrt(((x - mu[None, None, :, None]) ** 2).mean(axis=(0, 1, 3)) + eps)
        assert np.allclose(m[:, 0], mu, rtol=1e-9, atol=1e-12) and np.allclose(m[:, 1], sigma, rtol=1e-9)
        y_ = g[None, None, :, None] * (x - mu[None, None, :, None]) / sigma[None, None, :, None] + b[None, None, :, None]
        assert np.allclose(y, y_, rtol=1e-9, atol=1e-11)
        dy = np.asfortranarray(rng.standard_normal(shape))
        a = oracle.bnorm_backward(x, g, b, dy, eps)
        c = oracle.bnorm_backward(x, g, b, dy, eps, moments=m)
        for u, v in zip(a[:3], c[:3]):
            assert np.allclose(u, v, rtol=1e-12, atol=1e-12)


def test_avgpool_is_convolution(oracle):
    rng = np.random.default_rng(4)
    x = np.asfortranarray(rng.standard_normal((9, 8, 3, 2)))
    for pool, stride in [((2, 2), (2, 2)), ((3, 2), (1, 2)), ((1, 3), (3, 1))]:
        y = oracle.pool_forward(x, pool, stride, (0, 0, 0, 0), "avg")
        f = np.zeros((pool[0], pool[1], 1, 3), order="F")
        f[:] = 1.0 / (pool[0] * pool[1])
        y_ = oracle.conv_forward(x, f, None, stride)           # 3 groups of one channel
        assert np.allclose(y, y_, rtol=1e-12, atol=1e-12)


def test_conv_identities(oracle):
    rng = np.random.default_rng(5)
    x = np.asfortranarray(rng.standard_normal((11, 10, 4, 2)))
    f = np.asfortranarray(rng.standard_normal((3, 3, 4, 5)))
    b = rng.standard_normal(5)
    y1 = oracle.conv_forward(x, f, b)
    for s in [(2, 2), (3, 1), (1, 3)]:
        assert np.allclose(oracle.conv_forward(x, f, b, stride=s), y1[::s[0], ::s[1]], rtol=1e-12, atol=1e-12)
    pad = (2, 1, 0, 2)
    yp = oracle.conv_forward(x, f, b, pad=pad)
    xp = np.zeros((11 + 3, 10 + 2, 4, 2), order="F")
    xp[2:2 + 11, 0:10] = x
    assert np.allclose(yp, oracle.conv_forward(xp, f, b), rtol=1e-12, atol=1e-12)
    # two groups == dense filters with zero off-diagonal blocks
    fg = np.asfortranarray(rng.standard_normal((3, 3, 2, 6)))
    fd = np.zeros((3, 3, 4, 6), order="F")
    fd[:, :, 0:2, 0:3] = fg[:, :, :, 0:3]
    fd[:, :, 2:4, 3:6] = fg[:, :, :, 3:6]
    b6 = rng.standard_normal(6)
    assert np.allclose(oracle.conv_forward(x, fg, b6), oracle.conv_forward(x, fd, b6), rtol=1e-12, atol=1e-12)


def _numder(fn, x, dzdy, delta=1e-6):
    """Forward-difference derivative of <dzdy, fn(x)> (reference xtest/suite/nntest.m:94-108)."""
    y0 = fn(x)
    d = np.zeros(x.shape, order="F")
    flat = x.reshape(-1, order="F")
    for i in range(flat.size):
        xp = flat.copy()
        xp[i] += delta
        d.reshape(-1, order="F")[i] = ((fn(xp.reshape(x.shape, order="F")) - y0) * dzdy).sum() / delta
    return d


def test_numeric_derivatives(oracle):
    rng = np.random.default_rng(6)
    x = np.asfortranarray(rng.standard_normal((5, 4, 2, 2)))
    f = np.asfortranarray(rng.standard_normal((3, 2, 2, 3)))
    b = rng.standard_normal(3)
    kw = dict(stride=(1, 2), pad=(1, 0, 1, 1))
    dy = np.asfortranarray(rng.standard_normal(oracle.conv_forward(x, f, b, **kw).shape))
    dx, df, db = oracle.conv_backward(x, f, dy, **kw)
    assert np.allclose(dx, _numder(lambda v: oracle.conv_forward(v, f, b, **kw), x, dy), atol=1e-4)
    assert np.allclose(df, _numder(lambda v: oracle.conv_forward(x, v, b, **kw), f, dy), atol=1e-4)
    g, bb = rng.standard_normal(2) + 2, rng.standard_normal(2)
    dyb = np.asfortranarray(rng.standard_normal(x.shape))
    dxb, dg, dbb, _ = oracle.bnorm_backward(x, g, bb, dyb, 1e-3)
    assert np.allclose(dxb, _numder(lambda v: oracle.bnorm_forward(v, g, bb, 1e-3)[0], x, dyb), atol=1e-4)
    grid = np.asfortranarray(rng.uniform(-0.9, 0.9, (2, 3, 3, 2)))
    dys = np.asfortranarray(rng.standard_normal((3, 3, 2, 2)))
    dxs, dgr = oracle.sampler_backward(x, grid, dys)
    assert np.allclose(dxs, _numder(lambda v: oracle.sampler_forward(v, grid), x, dys), atol=1e-4)
    assert np.allclose(dgr, _numder(lambda v: oracle.sampler_forward(x, v), grid, dys), atol=1e-3)
    lab = np.array([1.0, 3.0])
    xl = np.asfortranarray(rng.standard_normal((1, 1, 4, 2)))
    dl = oracle.softmaxloss_backward(xl, lab, 1.0)
    nd = _numder(lambda v: np.array(oracle.softmaxloss_forward(v, lab)), xl, np.array(1.0))
    assert np.allclose(dl, nd, atol=1e-4)


def test_softmaxloss_class_zero_skips_the_image(oracle):
    # matlab/vl_nnsoftmaxloss.m:55-67: mass = (c > 0), index max(c - 1, 0); a float64 closed form of those lines
    rng = np.random.default_rng(16)
    x = np.asfortranarray(rng.standard_normal((2, 3, 5, 4)) * 2)
    lab = np.array([2.0, 0.0, 5.0, 0.0])
    mass = (lab > 0).astype(np.float64)
    idx = np.maximum(lab.astype(int) - 1, 0)
    xmax = x.max(axis=2, keepdims=True)
    ex = np.exp(x - xmax)
    picked = np.stack([x[:, :, idx[n], n] for n in range(4)], axis=-1)
    t = xmax[:, :, 0, :] + np.log(ex.sum(axis=2)) - picked
    want = (t * mass).sum() / 4
    assert abs(float(oracle.softmaxloss_forward(x, lab)) - want) < 1e-12
    y = ex / ex.sum(axis=2, keepdims=True)
    for n in range(4):
        y[:, :, idx[n], n] -= 1
    want_dx = y * mass[None, None, None, :] * 0.7 / 4
    assert np.allclose(oracle.softmaxloss_backward(x, lab, 0.7), want_dx, atol=1e-13)
    assert np.all(oracle.softmaxloss_backward(x, lab, 0.7)[:, :, :, 1] == 0)


def _lrn_closed_form(x, prm):
    n, kappa, alpha, beta = int(prm[0]), prm[1], prm[2], prm[3]
    m1 = (n - 1) // 2
    m2 = n - m1 - 1
    L = np.zeros_like(x)
    for t in range(x.shape[2]):
        L[:, :, t, :] = kappa + alpha * (x[:, :, max(t - m1, 0):min(t + m2, x.shape[2] - 1) + 1, :] ** 2).sum(axis=2)
    return x * L ** (-beta)


@pytest.mark.parametrize("prm", [[5, 2.0, 1e-3, 0.75], [4, 1.0, 0.1, 0.5], [1, 1.5, 0.5, 1.0], [9, 2.0, 1e-2, 0.6]])
def test_lrn_restatement_closed_form_and_compiled_reference(oracle, reference_backend, prm):
    """vl::nn::LRN: the restatement against the definition in double precision (forward) and a numeric derivative
    (backward); and against the reference's compiled CPU code, which evaluates the power with a cubic approximation of
    log2 and exp2 (bits/nnnormalize.cu:49-125) and therefore agrees to a few parts in a thousand only (measured: 4e-4 to
    2e-3, depending on the parameters)."""
    rng = np.random.default_rng(31)
    x = np.asfortranarray(rng.standard_normal((4, 3, 7, 2)))
    dy = np.asfortranarray(rng.standard_normal(x.shape))
    y = oracle.lrn_forward(x, prm)
    assert rel_l2(y, _lrn_closed_form(x, prm)) < 1e-14
    dx = oracle.lrn_backward(x, prm, dy)
    assert np.allclose(dx, _numder(lambda v: oracle.lrn_forward(v, prm), x, dy), atol=1e-5)
    if reference_backend is not None:
        for dt in (np.float32, np.float64):
            assert rel_l2(reference_backend.lrn_forward(x.astype(dt), prm), y) < 5e-3
            assert rel_l2(reference_backend.lrn_backward(x.astype(dt), prm, dy.astype(dt)), dx) < 5e-3


def test_softmax_restatement(oracle):
    """matlab/vl_nnsoftmax.m:24-29 in numpy, and its derivative numerically."""
    rng = np.random.default_rng(32)
    x = np.asfortranarray(rng.standard_normal((3, 2, 6, 2)) * 3)
    dy = np.asfortranarray(rng.standard_normal(x.shape))
    e = np.exp(x - x.max(axis=2, keepdims=True))
    y = e / e.sum(axis=2, keepdims=True)
    assert np.allclose(oracle.softmax(x), y, atol=1e-15)
    assert np.allclose(oracle.softmax(x, dy), y * (dy - (dy * y).sum(axis=2, keepdims=True)), atol=1e-14)
    assert np.allclose(oracle.softmax(x, dy), _numder(lambda v: oracle.softmax(v), x, dy), atol=1e-5)
