"""Generates tests/golden/*.npz from the reference's own compiled CPU backend.

Run where the reference checkout is present (it builds oracle/_ref/libmcn_ref.so from the
reference's sources and calls it through oracle/oracle.py):

    python tests/golden/make_golden.py

Each file holds the seeded inputs and the reference's outputs for one block, in single
precision (plus the double-precision instantiation's outputs for the contractions and for
batch normalisation, to tell the reference's own rounding from ours).  The plain BLAS of
oracle/ref_blas.cpp is used so the vectors do not depend on a BLAS library version.
The fixtures pin the C restatement (tests/test_oracle_pinned.py) and are compared
directly with the CUDA kernels (tests/test_gpu_*.py) on machines without the reference.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_oracle  # noqa: E402
import oracle as O  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def randn(rng, *shape):
    return np.asfortranarray(rng.standard_normal(shape).astype(np.float32))


def perm(rng, *shape):
    """All-distinct values (a permutation), as the reference's pooling tests use
    (matlab/xtest/suite/nnpool.m:23-28) so that arg-max is unambiguous."""
    n = int(np.prod(shape))
    return np.asfortranarray((rng.permutation(n).astype(np.float32) + 1).reshape(shape, order="F"))


CONV_CASES = {
    # name: (x shape, f shape, stride, pad, dilate)
    "basic3x3": ((9, 8, 4, 3), (3, 3, 4, 6), (1, 1), (1, 1, 1, 1), (1, 1)),
    "lenet5x5": ((12, 12, 5, 2), (5, 5, 5, 7), (1, 1), (0, 0, 0, 0), (1, 1)),
    "cifar5x5pad2": ((16, 16, 3, 2), (5, 5, 3, 8), (1, 1), (2, 2, 2, 2), (1, 1)),
    "stride_asympad": ((11, 10, 3, 2), (3, 2, 3, 5), (2, 3), (1, 2, 0, 1), (1, 1)),
    "dilate": ((13, 12, 2, 2), (3, 3, 2, 4), (1, 2), (2, 1, 1, 2), (2, 3)),
    "groups": ((8, 7, 6, 2), (3, 3, 2, 9), (1, 1), (1, 0, 0, 1), (1, 1)),
    "pointwise": ((7, 6, 16, 3), (1, 1, 16, 10), (1, 1), (0, 0, 0, 0), (1, 1)),
    "h14": ((14, 14, 8, 2), (3, 3, 8, 16), (1, 1), (1, 1, 1, 1), (1, 1)),
}

FC_CASES = {"fc_4x4": ((4, 4, 6, 5), (4, 4, 6, 9)), "fc_1x1": ((1, 1, 40, 7), (1, 1, 40, 12)),
            "fc_single": ((3, 3, 4, 1), (3, 3, 4, 5))}

POOL_CASES = {
    # name: (x shape, pool, stride, pad)
    "vgg2x2": ((12, 8, 3, 2), (2, 2), (2, 2), (0, 0, 0, 0)),
    "vgg2x2_h14": ((14, 10, 2, 2), (2, 2), (2, 2), (0, 0, 0, 0)),
    "cifar3x3s2": ((16, 16, 4, 2), (3, 3), (2, 2), (0, 1, 0, 1)),
    "odd": ((11, 9, 3, 2), (3, 2), (1, 3), (2, 1, 1, 0)),
    "odd_uncovered": ((7, 5, 2, 2), (2, 2), (2, 2), (0, 0, 0, 0)),
    "overlap_s1": ((6, 7, 2, 1), (3, 3), (1, 1), (1, 1, 1, 1)),
}


# name: x shape, filter shape (FH, FW, FD, FN = C), upsample, crop, groups  (the shapes of xtest/suite/nnconvt.m:
# upsampling 1-3 by 1-3, crops, two filter groups)
CONVT_CASES = {
    "up2_crop": ((5, 6, 4, 2), (3, 3, 5, 4), (2, 2), (1, 0, 1, 1), 1),
    "groups2_up12": ((4, 4, 6, 2), (4, 3, 2, 6), (1, 2), (0, 1, 2, 0), 2),
    "up31_nocrop": ((7, 5, 3, 1), (2, 2, 4, 3), (3, 1), (0, 0, 0, 0), 1),
    "up1_is_full_correlation": ((6, 6, 2, 2), (3, 3, 3, 2), (1, 1), (0, 0, 0, 0), 1),
    "fcn_upsample_4x": ((4, 5, 3, 1), (8, 8, 1, 3), (4, 4), (2, 2, 2, 2), 3),
}


def gen_convt(ref):
    rng = np.random.default_rng(20240608)
    out = {}
    for name, (xs, fs, up, crop, groups) in CONVT_CASES.items():
        x, f, b = randn(rng, *xs), randn(rng, *fs), randn(rng, fs[2] * groups)
        y = ref.convt_forward(x, f, b, up, crop, groups)
        dy = randn(rng, *y.shape)
        dx, df, db = ref.convt_backward(x, f, dy, up, crop, groups)
        x64, f64, b64, dy64 = (a.astype(np.float64) for a in (x, f, b, dy))
        y64 = ref.convt_forward(x64, f64, b64, up, crop, groups)
        dx64, df64, db64 = ref.convt_backward(x64, f64, dy64, up, crop, groups)
        for k, v in dict(x=x, f=f, b=b, y=y, dy=dy, dx=dx, df=df, db=db, y64=y64, dx64=dx64, df64=df64,
                         db64=db64, prm=np.array(list(up) + list(crop) + [groups])).items():
            out[name + "." + k] = v
    np.savez_compressed(os.path.join(OUT, "convt.npz"), **out)


def main():
    build_oracle.build_reference()
    ref = O.reference()
    assert ref is not None, "reference checkout not found: cannot make golden vectors"
    O.reference_use_plain_blas()
    gen_convt(ref)
    if "--only-convt" in sys.argv:          # the other files are left as they are
        return
    rng = np.random.default_rng(20240607)

    out = {}
    for name, (xs, fs, stride, pad, dilate) in CONV_CASES.items():
        x, f, b = randn(rng, *xs), randn(rng, *fs), randn(rng, fs[3])
        y = ref.conv_forward(x, f, b, stride, pad, dilate)
        dy = randn(rng, *y.shape)
        dx, df, db = ref.conv_backward(x, f, dy, stride, pad, dilate)
        x64, f64, b64, dy64 = (a.astype(np.float64) for a in (x, f, b, dy))
        y64 = ref.conv_forward(x64, f64, b64, stride, pad, dilate)
        dx64, df64, db64 = ref.conv_backward(x64, f64, dy64, stride, pad, dilate)
        for k, v in dict(x=x, f=f, b=b, y=y, dy=dy, dx=dx, df=df, db=db, y64=y64, dx64=dx64, df64=df64,
                         db64=db64, prm=np.array(list(stride) + list(pad) + list(dilate))).items():
            out[name + "." + k] = v
    np.savez_compressed(os.path.join(OUT, "conv.npz"), **out)

    out = {}
    for name, (xs, fs) in FC_CASES.items():
        x, f, b = randn(rng, *xs), randn(rng, *fs), randn(rng, fs[3])
        y = ref.fc_forward(x, f, b)
        dy = randn(rng, *y.shape)
        dx, df, db = ref.fc_backward(x, f, dy)
        for k, v in dict(x=x, f=f, b=b, y=y, dy=dy, dx=dx, df=df, db=db).items():
            out[name + "." + k] = v
    np.savez_compressed(os.path.join(OUT, "fc.npz"), **out)

    out = {}
    y0, xin, b = randn(rng, 5, 4, 6, 3), randn(rng, 5, 4, 6, 3), randn(rng, 6)
    dx0, db0, dyb = randn(rng, 5, 4, 6, 3), randn(rng, 6), randn(rng, 5, 4, 6, 3)
    out.update(y0=y0, x=xin, b=b, dx0=dx0, db0=db0, dy=dyb)
    fwd_args = [(0.0, True, 1.0, True, 1.0), (0.5, True, 2.0, True, 3.0), (0.5, False, 0.0, False, 0.0),
                (0.7, True, 1.5, False, 0.0), (0.0, False, 0.0, True, 2.0)]
    out["fwd_args"] = np.array(fwd_args, dtype=np.float64)
    for i, (ym, hx, xm, hb, bm) in enumerate(fwd_args):
        out["fwd%d" % i] = ref.bias_forward(y0, ym, xin if hx else None, xm, b if hb else None, bm)
    bwd_args = [(0.5, 0.25, 2.0, 3.0), (1.0, 0.0, 1.0, 1.0), (2.0, 1.0, 0.5, 0.5)]
    out["bwd_args"] = np.array(bwd_args, dtype=np.float64)
    for i, (dxm, dbm, xm, bm) in enumerate(bwd_args):
        dx, db = ref.bias_backward(dx0, dxm, db0, dbm, xm, bm, dyb)
        out["bwd%d.dx" % i], out["bwd%d.db" % i] = dx, db
    np.savez_compressed(os.path.join(OUT, "bias.npz"), **out)

    out = {}
    for name, shape, eps in [("small", (6, 5, 4, 7), 1e-4), ("vec", (8, 4, 5, 3), 1e-5), ("odd", (7, 7, 3, 2), 1e-3),
                             ("resnet", (28, 28, 8, 4), 1e-5)]:
        x = randn(rng, *shape) * 2 + 0.5
        g, b, dy = randn(rng, shape[2]), randn(rng, shape[2]), randn(rng, *shape)
        y, mom = ref.bnorm_forward(x, g, b, eps)
        dx, dg, db, mom2 = ref.bnorm_backward(x, g, b, dy, eps)
        dxm, dgm, dbm, _ = ref.bnorm_backward(x, g, b, dy, eps, moments=mom)
        ym, _ = ref.bnorm_forward(x, g, b, eps, moments=mom)
        x64, g64, b64, dy64 = (a.astype(np.float64) for a in (x, g, b, dy))
        y64, mom64 = ref.bnorm_forward(x64, g64, b64, eps)
        dx64, dg64, db64, _ = ref.bnorm_backward(x64, g64, b64, dy64, eps)
        for k, v in dict(x=x, g=g, b=b, dy=dy, y=y, mom=mom, dx=dx, dg=dg, db=db, dxm=dxm, dgm=dgm, dbm=dbm, ym=ym,
                         y64=y64, mom64=mom64, dx64=dx64, dg64=dg64, db64=db64, eps=np.array(eps)).items():
            out[name + "." + k] = v
    np.savez_compressed(os.path.join(OUT, "bnorm.npz"), **out)

    out = {}
    for name, (xs, pool, stride, pad) in POOL_CASES.items():
        x = perm(rng, *xs)
        for method in ("max", "avg"):
            y = ref.pool_forward(x, pool, stride, pad, method)
            dy = randn(rng, *y.shape)
            dx = ref.pool_backward(x, dy, pool, stride, pad, method)
            for k, v in dict(y=y, dy=dy, dx=dx).items():
                out["%s.%s.%s" % (name, method, k)] = v
        out[name + ".x"] = x
        out[name + ".prm"] = np.array(list(pool) + list(stride) + list(pad))
    # ties and -inf: first maximal element in column-major window order wins; all -inf routes nowhere
    x = np.zeros((4, 4, 1, 1), np.float32, order="F")
    x[:2, :2] = 3.0
    x[2:, :2] = -np.inf
    x[:2, 2:, 0, 0] = np.array([[1, 5], [5, 5]], np.float32)
    dy = np.asfortranarray(np.arange(1, 5, dtype=np.float32).reshape(2, 2, 1, 1, order="F"))
    out["ties.x"], out["ties.dy"] = x, dy
    out["ties.max.y"] = ref.pool_forward(x, (2, 2), (2, 2), (0, 0, 0, 0), "max")
    out["ties.max.dx"] = ref.pool_backward(x, dy, (2, 2), (2, 2), (0, 0, 0, 0), "max")
    np.savez_compressed(os.path.join(OUT, "pool.npz"), **out)

    out = {}
    x = perm(rng, 15, 14, 3, 2)
    # whole map, interior, overhanging, degenerate (reversed corners), image index out of range, fractional
    rois = np.asfortranarray(np.array([
        [1, 1, 1, 14, 15], [2, 3.4, 2.2, 7.7, 9.1], [1, -3, -2, 20, 30], [2, 5, 5, 5, 5], [3, 9, 11, 10, 12],
        [0, 2.5, 3.5, 4.5, 6.5], [1, 8, 9, 3, 2], [2, 13.5, 14.5, 14.49, 15.5], [1, 0.5, 0.5, 1.5, 1.5]],
        dtype=np.float32).T)
    out["x"], out["rois"] = x, rois
    tfs = {"id": [1, 0, 0, 1, 0, 0], "half": [0.5, 0, 0, 0.5, 0.5, 0.5], "sixteenth": [1 / 16., 0, 0, 1 / 16., 15 / 16., 15 / 16.],
           "affine": [0.9, 0.1, -0.2, 1.1, 0.3, -0.4]}
    for tname, tf in tfs.items():
        out["tf." + tname] = np.array(tf, dtype=np.float64)
        r = rois.copy(order="F")
        if tname == "sixteenth":
            r[1:, :] = r[1:, :] * 16 - 7
        out["rois." + tname] = r
        for sub in [(1, 1), (2, 1), (1, 2), (3, 7), (7, 7), (16, 16)]:
            for method in ("max", "avg"):
                y = ref.roipool_forward(x, r, sub, tf, method)
                dy = randn(rng, *y.shape)
                dyi = np.asfortranarray(rng.integers(-8, 9, size=y.shape).astype(np.float32))
                key = "%s.%dx%d.%s" % (tname, sub[0], sub[1], method)
                out[key + ".y"] = y
                out[key + ".dy"], out[key + ".dx"] = dy, ref.roipool_backward(x, r, dy, sub, tf, method)
                out[key + ".dyi"], out[key + ".dxi"] = dyi, ref.roipool_backward(x, r, dyi, sub, tf, method)
    np.savez_compressed(os.path.join(OUT, "roipool.npz"), **out)

    out = {}
    for name, xs, gs, lim in [("inrange", (8, 7, 3, 2), (2, 5, 6, 4), 1.0), ("overhang", (9, 6, 2, 3), (2, 7, 4, 3), 1.3),
                              ("same", (10, 10, 4, 2), (2, 10, 10, 2), 0.95)]:
        x = randn(rng, *xs)
        grid = np.asfortranarray(rng.uniform(-lim, lim, gs).astype(np.float32))
        y = ref.sampler_forward(x, grid)
        dy = randn(rng, *y.shape)
        dx, dgrid = ref.sampler_backward(x, grid, dy)
        for k, v in dict(x=x, grid=grid, y=y, dy=dy, dx=dx, dgrid=dgrid).items():
            out[name + "." + k] = v
    np.savez_compressed(os.path.join(OUT, "sampler.npz"), **out)
    total = sum(os.path.getsize(os.path.join(OUT, f)) for f in os.listdir(OUT) if f.endswith(".npz"))
    print("golden vectors written: %.1f KB" % (total / 1024.0))


if __name__ == "__main__":
    main()
