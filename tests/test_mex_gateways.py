"""The reference's own MEX gateways, compiled unmodified over the vlb engine, driven without MATLAB.

tests/mexdouble/ builds matlab/src/vl_nnconv.cu, vl_nnbnorm.cu, vl_nnpool.cu, vl_nnroipool.cu and
vl_nnbilinearsampler.cu (plus the reference's data layer) against a stand-in for the MEX API and against
tests/mexdouble/vlb_functors.cpp, which defines the reference's operator classes over the C ABI -- the binding a
maintainer would add.  So what runs here is the reference's option parsing (vlmxNextOption, 'Stride', 'Pad', 'Method',
'Moments', ...), its shape checks and error messages, its output allocation (MexTensor), and then this repository's
kernels.  Without a GPU: the libraries load, export mexFunction, and refuse bad arguments with MATLAB's messages.  On a
B200: forward and backward of every gateway against the golden vectors of the reference's CPU backend.
"""
import ctypes
import os
import sys

import numpy as np
import pytest

from conftest import bit_equal, cases_of, load_golden, rel_l2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "mexdouble"))

import build_mexdouble  # noqa: E402
import mexdriver        # noqa: E402
from mexdriver import MexError, gpu as G  # noqa: E402

TOL = 1e-5


@pytest.fixture(scope="module")
def mex():
    libs = build_mexdouble.build()
    if libs is None:
        pytest.skip("the MEX test double is built where the reference checkout is; no prebuilt libraries here")
    m = mexdriver.MexDouble()
    yield m
    m.close()


def same(got, want):
    """Bit-equal after MATLAB's treatment of shapes: trailing singleton dimensions are dropped."""
    shape = tuple(want.shape)
    while len(shape) > 2 and shape[-1] == 1:
        shape = shape[:-1]
    return tuple(got.shape) == shape and bit_equal(got.ravel(order="F"), np.asarray(want).ravel(order="F"))


def f32(*shape, seed=0):
    return np.asfortranarray(np.random.default_rng(seed).standard_normal(shape).astype(np.float32))


# ------------------------------------------------------------------ without a GPU
def test_every_gateway_exports_mexFunction(mex):
    for name in build_mexdouble.GATEWAYS:
        lib = ctypes.CDLL(os.path.join(build_mexdouble.OUT, name + ".so"))
        assert hasattr(lib, "mexFunction"), name


@pytest.mark.parametrize("name,args,message", [
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4), "Stride", [1, 2, 3]), "STRIDE has neither one nor two elements"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4), "Stride", 0), "STRIDE is smaller than one"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4), "Pad", [1, 2, 3]), "PAD has neither one nor four elements"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4), "Pad", -1), "PAD is negative"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4), "Whatever", 1), "Unknown option 'Whatever'"),
    ("vl_nnconv", (f32(8, 8, 3, 2),), "less than three arguments"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 2, 4), f32(1, 4)), "FILTERS depth does not divide the DATA depth"),
    ("vl_nnconv", (f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 5)), "BIASES"),
    ("vl_nnconv", (f32(2, 2, 3, 2), f32(3, 3, 3, 4), f32(1, 4)), "FILTERS are larger than the DATA"),
    ("vl_nnpool", (f32(8, 8, 3, 2), [2, 2, 2]), "SIZE has neither one nor two elements"),
    ("vl_nnpool", (f32(8, 8, 3, 2), 2, "Method", "median"), "METHOD is not a supported method"),
    ("vl_nnpool", (f32(8, 8, 3, 2), 2, "Pad", 2), "pad"),
    ("vl_nnbnorm", (f32(8, 8, 3, 2), f32(4, 1), f32(3, 1)), "MULTIPLIERS"),
    ("vl_nnbnorm", (f32(8, 8, 3, 2), f32(3, 1), f32(3, 1), "Moments", f32(3, 3)), "MOMENTS"),
    ("vl_nnroipool", (f32(8, 8, 3, 2), f32(4, 2)), "ROI is not a 5 x K array"),
    ("vl_nnroipool", (f32(8, 8, 3, 2), f32(5, 2), "Subdivisions", [1, 2, 3]), "SUBDIVISIONS does not have one or two elements"),
    ("vl_nnroipool", (f32(8, 8, 3, 2), f32(5, 2), "Transform", [1, 2, 3]), "TRANSFORM is neither"),
    ("vl_nnbilinearsampler", (f32(8, 8, 3, 2), f32(3, 4, 4, 2)), "GRID"),
    ("vl_nnbilinearsampler", (f32(8, 8, 3, 2), f32(2, 4, 4, 3)), "GRID"),
])
def test_bad_arguments_get_the_gateways_own_messages(mex, name, args, message):
    with pytest.raises(MexError) as err:
        mex.call(name, 1, *args)
    assert message.lower() in str(err.value).lower()


def test_host_arrays_are_refused_by_the_engine_not_computed_on_the_cpu(mex):
    before = mex.launches()
    with pytest.raises(MexError) as err:
        mex.call("vl_nnconv", 1, f32(8, 8, 3, 2), f32(3, 3, 3, 4), f32(1, 4))
    assert "single-precision gpuArrays only" in str(err.value)
    with pytest.raises(MexError):
        mex.call("vl_nnpool", 1, f32(8, 8, 3, 2), 2)
    assert mex.launches() == before


# ------------------------------------------------------------------ on a B200
@pytest.mark.gpu
def test_vl_nnconv_gateway_golden(mex, gpu):
    nn, mat, ctx = gpu
    g = load_golden("conv")
    before = mex.launches()
    for c in cases_of(g):
        prm = [int(v) for v in g[c + ".prm"]]
        opts = ("Stride", prm[0:2], "Pad", prm[2:6], "Dilate", prm[6:8])
        x, f, b, dy = g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"]
        y, placement = mex.call("vl_nnconv", 1, G(x), G(f), G(b), *opts, with_placement=True)
        assert placement == [True] and y.dtype == np.float32 and y.shape == g[c + ".y"].shape, c
        dx, df, db = mex.call("vl_nnconv", 3, G(x), G(f), G(b), G(dy), *opts)
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(got.ravel(), g[c + "." + name + "64"].ravel()) < TOL, (c, name)
        # the same kernels as the Python wrappers reach: bit for bit
        kw = dict(stride=tuple(prm[0:2]), pad=tuple(prm[2:6]), dilate=tuple(prm[6:8]))
        xd, fd, bd, dyd = (mat.from_numpy(a) for a in (x, f, b, dy))
        assert bit_equal(y, mat.to_numpy(nn.vl_nnconv(xd, fd, bd, ctx=ctx, **kw))), c
        for got, want in zip((dx, df, db), nn.vl_nnconv(xd, fd, bd, dyd, ctx=ctx, **kw)):
            assert bit_equal(got.ravel(), mat.to_numpy(want).ravel()), c
    assert mex.launches() > before


@pytest.mark.gpu
def test_vl_nnconv_gateway_options(mex):
    g = load_golden("conv")
    c = "basic3x3"
    prm = [int(v) for v in g[c + ".prm"]]
    opts = ("stride", prm[0:2], "pad", prm[2:6])          # option names are case-insensitive
    x, f, b, dy = g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"]
    dx, df, db = mex.call("vl_nnconv", 3, G(x), G(f), G(b), G(dy), *opts, "NoDerData")
    assert dx.size == 0 and rel_l2(df, g[c + ".df64"]) < TOL and rel_l2(db.ravel(), g[c + ".db64"].ravel()) < TOL
    dx, df, db = mex.call("vl_nnconv", 3, G(x), G(f), G(b), G(dy), *opts, "NoDerFilters", "NoDerBiases")
    assert df.size == 0 and db.size == 0 and rel_l2(dx, g[c + ".dx64"]) < TOL
    # no biases: an empty third argument
    empty = np.zeros((0, 0), np.float32)
    y0 = mex.call("vl_nnconv", 1, G(x), G(f), G(empty), *opts)
    yb = mex.call("vl_nnconv", 1, G(x), G(f), G(b), *opts)
    assert rel_l2(yb - y0, np.broadcast_to(b.reshape(1, 1, -1, 1), yb.shape)) < 1e-5
    # a derivative of the wrong shape is refused by the gateway before anything is launched
    with pytest.raises(MexError) as err:
        mex.call("vl_nnconv", 3, G(x), G(f), G(b), G(dy[:-1]), *opts)
    assert "DEROUTPUT" in str(err.value)


@pytest.mark.gpu
def test_vl_nnconv_gateway_fully_connected_shortcut(mex):
    g = load_golden("fc")
    for c in cases_of(g):
        x, f, b, dy = g[c + ".x"], g[c + ".f"], g[c + ".b"], g[c + ".dy"]
        y = mex.call("vl_nnconv", 1, G(x), G(f), G(b))
        dx, df, db = mex.call("vl_nnconv", 3, G(x), G(f), G(b), G(dy))
        for got, name in ((y, "y"), (dx, "dx"), (df, "df"), (db, "db")):
            assert rel_l2(got.ravel(), g[c + "." + name].ravel()) < TOL + 2e-6, (c, name)


@pytest.mark.gpu
def test_vl_nnconv_gateway_without_filters_is_refused(mex):
    x = f32(8, 8, 3, 2)
    empty = np.zeros((0, 0), np.float32)
    with pytest.raises(MexError) as err:
        mex.call("vl_nnconv", 1, G(x), G(empty), G(empty), "Stride", 2)
    assert "not covered by the B200 engine" in str(err.value)


@pytest.mark.gpu
def test_vl_nnbnorm_gateway_golden(mex):
    g = load_golden("bnorm")
    for c in cases_of(g):
        x, gg, b, dy = g[c + ".x"], g[c + ".g"], g[c + ".b"], g[c + ".dy"]
        eps = float(g[c + ".eps"])
        y, mom = mex.call("vl_nnbnorm", 2, G(x), G(gg), G(b), "Epsilon", eps)
        assert mom.shape == g[c + ".mom64"].shape, c
        assert rel_l2(y, g[c + ".y64"]) < TOL and rel_l2(mom, g[c + ".mom64"]) < TOL, c
        dx, dg, db, mom2 = mex.call("vl_nnbnorm", 4, G(x), G(gg), G(b), G(dy), "Epsilon", eps)
        for got, name in ((dx, "dx"), (dg, "dg"), (db, "db"), (mom2, "mom")):
            assert rel_l2(got.ravel(), g[c + "." + name + "64"].ravel()) < TOL, (c, name)
        ym = mex.call("vl_nnbnorm", 1, G(x), G(gg), G(b), "Epsilon", eps, "Moments", G(g[c + ".mom"]))
        assert same(ym, g[c + ".ym"]), c
        dxm, dgm, dbm = mex.call("vl_nnbnorm", 3, G(x), G(gg), G(b), G(dy), "Epsilon", eps, "Moments", G(g[c + ".mom"]))
        for got, name in ((dxm, "dxm"), (dgm, "dgm"), (dbm, "dbm")):
            assert rel_l2(got.ravel(), g[c + "." + name].ravel()) < TOL, (c, name)


@pytest.mark.gpu
def test_vl_nnpool_gateway_golden(mex):
    g = load_golden("pool")
    for c in cases_of(g):
        if c == "ties":
            continue
        prm = [int(v) for v in g[c + ".prm"]]
        x = g[c + ".x"]
        for method in ("max", "avg"):
            opts = ("Stride", prm[2:4], "Pad", prm[4:8], "Method", method)
            y = mex.call("vl_nnpool", 1, G(x), prm[0:2], *opts)
            assert same(y, g["%s.%s.y" % (c, method)]), (c, method)
            dx = mex.call("vl_nnpool", 1, G(x), prm[0:2], G(g["%s.%s.dy" % (c, method)]), *opts)
            assert rel_l2(dx, g["%s.%s.dx" % (c, method)]) < 1e-6, (c, method)
    # the default method is max; the first maximum of a window takes the derivative
    y = mex.call("vl_nnpool", 1, G(g["ties.x"]), 2, "Stride", 2)
    assert same(y, g["ties.max.y"])
    dx = mex.call("vl_nnpool", 1, G(g["ties.x"]), 2, G(g["ties.dy"]), "Stride", 2)
    assert same(dx, g["ties.max.dx"])


@pytest.mark.gpu
def test_vl_nnroipool_gateway_golden(mex):
    g = load_golden("roipool")
    x = g["x"]
    for key in sorted({k[:-2] for k in g if k.endswith(".y")}):
        tname, sub, method = key.split(".")
        sub = [int(v) for v in sub.split("x")]
        tf = g["tf." + tname].reshape(2, 3, order="F")
        opts = ("Subdivisions", sub, "Transform", tf, "Method", method)
        rois = g["rois." + tname]
        y = mex.call("vl_nnroipool", 1, G(x), G(rois), *opts)
        assert same(y, g[key + ".y"]), key
        dx = mex.call("vl_nnroipool", 1, G(x), G(rois), G(g[key + ".dy"]), *opts)
        assert same(dx, g[key + ".dx"]), key
    # scalar transform = isotropic scale; the default is the identity.  (Subdivisions always with two elements: the
    # gateway's one-element branch falls through into the two-element one and reads past the scalar,
    # matlab/src/vl_nnroipool.cu:125-131.)
    rois = g["rois.id"]
    y1 = mex.call("vl_nnroipool", 1, G(x), G(rois), "Subdivisions", [3, 3])
    y2 = mex.call("vl_nnroipool", 1, G(x), G(rois), "Subdivisions", [3, 3], "Transform", 1.0, "Method", "max")
    assert bit_equal(y1, y2)


@pytest.mark.gpu
def test_vl_nnbilinearsampler_gateway_golden(mex):
    g = load_golden("sampler")
    for c in cases_of(g):
        x, grid, dy = g[c + ".x"], g[c + ".grid"], g[c + ".dy"]
        assert same(mex.call("vl_nnbilinearsampler", 1, G(x), G(grid)), g[c + ".y"]), c
        dx, dgrid = mex.call("vl_nnbilinearsampler", 2, G(x), G(grid), G(dy))
        assert same(dgrid, g[c + ".dgrid"]), c
        assert rel_l2(dx, g[c + ".dx"]) < 1e-6, c
