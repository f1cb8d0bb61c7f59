"""Per-layer timing of the hot-path kernels through the C ABI.

    python layerbench.py [--net vgg16] [--batch 64] [--precision 3xtf32] [--layers conv3_1,fc6]
    python layerbench.py --kind bnorm|pool|roipool|sampler|update

A measuring tool beside bench.py (which imports its bandwidth rows for the bench line's `kernels` list); not part of
the library.

Each row is one block of the network at the given batch: forward, data-gradient and
filter-gradient times from CUDA events on the launching stream (median of --iters after warm-up, the
L2 flushed between iterations by writing a 256 MB buffer), and the algorithmic rate they imply:
2*M*N*K flops for contractions, the compulsory bytes for the bandwidth-bound blocks.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from matconvnet_b200 import mat, nn  # noqa: E402

VGG = [("conv1_1", 224, 3, 64, 3, 1), ("conv1_2", 224, 64, 64, 3, 1), ("conv2_1", 112, 64, 128, 3, 1),
       ("conv2_2", 112, 128, 128, 3, 1), ("conv3_1", 56, 128, 256, 3, 1), ("conv3_2", 56, 256, 256, 3, 1),
       ("conv4_1", 28, 256, 512, 3, 1), ("conv4_2", 28, 512, 512, 3, 1), ("conv5_1", 14, 512, 512, 3, 1),
       ("fc6", 7, 512, 4096, 7, 0), ("fc7", 1, 4096, 4096, 1, 0), ("fc8", 1, 4096, 1000, 1, 0)]
RESNET = [("res_1x1_a", 28, 512, 128, 1, 0), ("res_3x3", 28, 128, 128, 3, 1), ("res_1x1_b", 28, 128, 512, 1, 0)]


def timed(fn, iters, flush):
    times = []
    for it in range(iters + 2):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            times.append(e0.elapsed_time(e1))
    return float(np.median(times))


def timed_queued(fns, reps):
    """Kernels of tens of microseconds: the host cannot enqueue as fast as they run, so events around a single call
    measure the host.  Here the GPU is kept busy (a spin kernel of about a millisecond) while the host enqueues `reps`
    calls, which then run back to back; the callables rotate over independent inputs that together exceed the L2, so
    every call finds its operands in DRAM.  Returns milliseconds per call."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(4_000_000)
    e0.record()
    for i in range(reps):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def conv_rows(layers, batch, iters, flush, which):
    rows = []
    for name, hw, cin, cout, fs, pad in layers:
        if which and name not in which:
            continue
        x = mat.as_mat(torch.randn(hw, hw, cin, batch, device="cuda"))
        f = mat.as_mat(torch.randn(fs, fs, cin, cout, device="cuda") * (2.0 / (fs * fs * cin)) ** 0.5)
        b = mat.zeros((1, cout))
        y = nn.vl_nnconv(x, f, b, pad=pad)
        dy = mat.as_mat(torch.randn(*y.shape, device="cuda"))
        flops = 2.0 * y.shape[0] * y.shape[1] * batch * cout * fs * fs * cin
        t_f = timed(lambda: nn.vl_nnconv(x, f, b, pad=pad), iters, flush)
        t_d = timed(lambda: nn.vl_nnconv(x, f, b, dy, pad=pad, no_der_filters=True, no_der_biases=True), iters, flush)
        t_w = timed(lambda: nn.vl_nnconv(x, f, b, dy, pad=pad, no_der_data=True), iters, flush)
        rows.append({"layer": name, "gflop": flops / 1e9, "fprop_ms": t_f, "dgrad_ms": t_d, "wgrad_dbias_ms": t_w,
                     "fprop_tflops": flops / t_f / 1e9, "dgrad_tflops": flops / t_d / 1e9,
                     "wgrad_tflops": flops / t_w / 1e9})
    return rows


def bandwidth_rows(kind, iters, flush):
    rows = []
    if kind == "bnorm":
        for shape in [(28, 28, 128, 64), (28, 28, 512, 64), (56, 56, 64, 64)]:
            n = float(np.prod(shape))
            sets = max(2, int(400e6 / (8 * n)) + 1)          # x and dy of all sets together: well above the 126 MB L2
            xs = [mat.as_mat(torch.randn(*shape, device="cuda")) for _ in range(sets)]
            dys = [mat.as_mat(torch.randn(*shape, device="cuda")) for _ in range(sets)]
            g, b = mat.as_mat(torch.rand(shape[2], 1, device="cuda") + 0.5), mat.zeros((shape[2], 1))
            t_b = timed_queued([lambda x=x, dy=dy: nn.vl_nnbnorm(x, g, b, dy, epsilon=1e-5) for x, dy in zip(xs, dys)], 2 * sets)
            t_f = timed_queued([lambda x=x: nn.vl_nnbnorm(x, g, b, epsilon=1e-5) for x in xs], 2 * sets)
            rows.append({"block": "bnorm %s" % (shape,), "bwd_ms": t_b, "bwd_GBs_20B": 20 * n / t_b / 1e6,
                         "bwd_GBs_12B": 12 * n / t_b / 1e6, "fwd_ms": t_f, "fwd_GBs_16B": 16 * n / t_f / 1e6,
                         "fwd_GBs_8B": 8 * n / t_f / 1e6})
    elif kind == "pool":
        for hw, c in [(224, 64), (112, 128), (56, 256), (28, 512), (14, 512)]:
            x = mat.as_mat(torch.randn(hw, hw, c, 64, device="cuda"))
            y = nn.vl_nnpool(x, (2, 2), stride=2)
            dy = mat.as_mat(torch.randn(*y.shape, device="cuda"))
            nin, nout = float(x.numel()), float(y.numel())
            t_f = timed(lambda: nn.vl_nnpool(x, (2, 2), stride=2), iters, flush)
            t_b = timed(lambda: nn.vl_nnpool(x, (2, 2), dy, stride=2), iters, flush)
            rows.append({"block": "maxpool2x2 %dx%dx%dx64" % (hw, hw, c), "fwd_ms": t_f, "fwd_GBs": 4 * (nin + nout) / t_f / 1e6,
                         "bwd_ms": t_b, "bwd_GBs": 4 * (2 * nin + nout) / t_b / 1e6})
    elif kind == "roipool":
        g = torch.Generator(device="cuda").manual_seed(0)
        H, W, Cc, N, K = 38, 50, 512, 2, 256
        x = mat.as_mat(torch.randn(H, W, Cc, N, device="cuda", generator=g))
        u1 = torch.rand(K, device="cuda", generator=g) * (W - 3) + 1
        v1 = torch.rand(K, device="cuda", generator=g) * (H - 3) + 1
        u2 = torch.minimum(u1 + 2 + torch.rand(K, device="cuda", generator=g) * W, torch.tensor(float(W), device="cuda"))
        v2 = torch.minimum(v1 + 2 + torch.rand(K, device="cuda", generator=g) * H, torch.tensor(float(H), device="cuda"))
        rois = mat.as_mat(torch.stack([torch.arange(K, device="cuda") % N + 1.0, u1, v1, u2, v2]))
        y = nn.vl_nnroipool(x, rois, subdivisions=(7, 7))
        # four rotating sets (165 MB together, above the L2), launches queued back to back: the kernels take tens of microseconds
        xs = [x] + [mat.as_mat(torch.randn(H, W, Cc, N, device="cuda", generator=g)) for _ in range(3)]
        dys = [mat.as_mat(torch.randn(*y.shape, device="cuda", generator=g)) for _ in range(4)]
        t_f = timed_queued([lambda a=a: nn.vl_nnroipool(a, rois, subdivisions=(7, 7)) for a in xs], 8)
        t_b = timed_queued([lambda a=a, d=d: nn.vl_nnroipool(a, rois, d, subdivisions=(7, 7)) for a, d in zip(xs, dys)], 8)
        nbytes = 4.0 * (2 * x.numel() + y.numel())
        rows.append({"block": "roipool 38x50x512x2, 256 rois, 7x7", "fwd_ms": t_f, "bwd_ms": t_b, "bwd_bytes": nbytes,
                     "bwd_GBs": nbytes / t_b / 1e6})
    elif kind == "sampler":
        # 256 affine grids of small rotations and scales (matlab/+dagnn/AffineGridGenerator.m:36-57): grid = [yy xx] * A + t
        g = torch.Generator(device="cuda").manual_seed(0)
        x = mat.as_mat(torch.randn(64, 64, 32, 256, device="cuda", generator=g))
        lin = torch.linspace(-1, 1, 64, device="cuda")
        yy = lin.view(64, 1, 1).expand(64, 64, 256)           # (ho, wo, n): row coordinate
        xx = lin.view(1, 64, 1).expand(64, 64, 256)
        th = (torch.rand(256, device="cuda", generator=g) - 0.5) * 0.4
        sc = 0.8 + 0.4 * torch.rand(256, device="cuda", generator=g)
        t = (torch.rand(2, 256, device="cuda", generator=g) - 0.5) * 0.2
        gy = sc * (torch.cos(th) * yy + torch.sin(th) * xx) + t[0]
        gx = sc * (-torch.sin(th) * yy + torch.cos(th) * xx) + t[1]
        grid = mat.as_mat(torch.stack([gy, gx]))
        dy = mat.as_mat(torch.randn(64, 64, 32, 256, device="cuda", generator=g))
        x2, dy2 = (mat.as_mat(torch.randn(64, 64, 32, 256, device="cuda", generator=g)) for _ in range(2))
        t_f = timed_queued([lambda: nn.vl_nnbilinearsampler(x, grid), lambda: nn.vl_nnbilinearsampler(x2, grid)], 4)
        t_b = timed_queued([lambda: nn.vl_nnbilinearsampler(x, grid, dy), lambda: nn.vl_nnbilinearsampler(x2, grid, dy2)], 4)
        nbytes = 4.0 * (3 * x.numel() + 2 * grid.numel())
        rows.append({"block": "sampler 64x64x32x256, 256 affine grids", "fwd_ms": t_f, "bwd_ms": t_b, "bwd_bytes": nbytes,
                     "bwd_GBs": nbytes / t_b / 1e6})
    elif kind == "update":
        # the trainer's SGD step on VGG-16's largest parameter tensors (fc6 filters 102.8M, fc7 16.8M, conv5 2.4M floats):
        # the fused kernel (reads W, M, G; writes W, M) against the reference's four vl_taccum passes
        for name, n in (("fc6 filters", 7 * 7 * 512 * 4096), ("fc7 filters", 4096 * 4096), ("conv5 filters", 3 * 3 * 512 * 512)):
            w, m, g = (torch.randn(n, device="cuda") for _ in range(3))

            def four():
                par = nn.vl_taccum(0.5, g, 0.0005, w)
                nn.vl_taccum(0.9, m, -1.0, par, out=m)
                nn.vl_taccum(1.0, w, 0.01, m, out=w)
            t_f = timed(lambda: nn.sgd_update_(w, m, g, 0.5, 0.0005, 0.9, 0.01), iters, flush)
            t_4 = timed(four, iters, flush)
            rows.append({"block": "sgd update, " + name, "fused_ms": t_f, "fused_GBs": 20.0 * n / t_f / 1e6, "taccum_x3_ms": t_4})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--net", default="vgg16", choices=["vgg16", "resnet"])
    ap.add_argument("--kind", default="conv", choices=["conv", "bnorm", "pool", "roipool", "sampler", "update"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32", "fp32"])
    ap.add_argument("--layers", default="")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--test-switch", type=int, default=0, help="vlb_ctx_set_test_switch bits (2: no tensor-map windows, 4: filter gradient on the shared-memory kernel)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    ctx = nn.default_context()
    ctx.set_precision({"3xtf32": 0, "tf32": 1, "fp32": 2}[args.precision])
    ctx.reserve_workspace(3 << 30)
    ctx.check(ctx.lib.vlb_ctx_set_test_switch(ctx.handle, args.test_switch))
    flush = None if args.no_flush else torch.empty(64 << 20, device="cuda")
    if args.kind == "conv":
        which = [s for s in args.layers.split(",") if s]
        rows = conv_rows(VGG if args.net == "vgg16" else RESNET, args.batch, args.iters, flush, which)
    else:
        rows = bandwidth_rows(args.kind, args.iters, flush)
    ctx.device_status()
    for r in rows:
        print(json.dumps({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}))


if __name__ == "__main__":
    main()
