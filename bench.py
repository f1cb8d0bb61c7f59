"""VGG-16 fp32 forward+backward throughput (images/s), data parallel over 1..8 B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torch.distributed.run)
    python bench.py --impl reference --steps K --warmup W    (the reference's CPU backend on the host cores)

A step is one pass of the hot path over one batch of synthetic input: forward, backward and the
gradient exchange (every parameter derivative summed over the workers and divided by their number)
of VGG-16 at 64 images of 224x224x3 per GPU, weights He-normal, labels uniform over 1..1000.
Every block is a call through the C ABI (libvlb.so); torch supplies device memory, streams and
torch.distributed.  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "vgg16_fp32_fwd_bwd_images_per_sec"
UNIT = "images/s"
PER_GPU_BATCH = 64
GFLOP_PER_IMAGE = 92.82          # 3 x 30.94 algorithmic GFLOP: forward, data gradient, filter gradient


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi during the timed region (index, SM clock, max SM clock, power, reasons)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smmax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smmax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smmax) if smmax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_vgg16(batch, steps, warmup, threads):
    """The reference's CPU backend (oracle/_ref when built, else the C restatement) on VGG-16."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_net
    import oracle as O
    glue = O.restatement()
    ref = O.reference()
    kind = "reference" if ref is not None else "port"
    backend = ref if ref is not None else glue
    blas = "plain"
    if ref is not None and O.reference_use_openblas(threads):
        blas = "openblas(ilp64, numpy-bundled), %d threads" % threads
    else:
        threads = 1
    rng = np.random.default_rng(0)
    layers = []
    cin = 3
    for cout, reps in [(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]:
        for _ in range(reps):
            f = np.asfortranarray((rng.standard_normal((3, 3, cin, cout)) * np.sqrt(2.0 / (9 * cin))).astype(np.float32))
            layers += [dict(type="conv", weights=[f, np.zeros(cout, np.float32)], stride=1, pad=1), dict(type="relu")]
            cin = cout
        layers.append(dict(type="pool", method="max", pool=[2, 2], stride=2, pad=0))
    for fh, ci, co, relu in [(7, 512, 4096, True), (1, 4096, 4096, True), (1, 4096, 1000, False)]:
        f = np.asfortranarray((rng.standard_normal((fh, fh, ci, co)) * np.sqrt(2.0 / (fh * fh * ci))).astype(np.float32))
        layers.append(dict(type="conv", weights=[f, np.zeros(co, np.float32)], stride=1, pad=0))
        if relu:
            layers.append(dict(type="relu"))
    labels = rng.integers(1, 1001, size=batch).astype(np.float32)
    layers.append(dict(type="softmaxloss", **{"class": labels}))
    x = np.asfortranarray(rng.standard_normal((224, 224, 3, batch)).astype(np.float32))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        res = cpu_net.simplenn(backend, glue, layers, x, np.float32(1.0), conserve_memory=True)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        del res
    sec = float(np.mean(times))
    return {"value": batch / sec, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": "VGG-16 fwd+bwd, batch %d, %d step(s) of %.1f s; BLAS: %s; im2row/pool/relu single-threaded as in "
                      "the reference" % (batch, steps, sec, blas)}, sec


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    base, sec = cpu_vgg16(args.cpu_batch, args.steps, min(args.warmup, 1), cores)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "VGG-16 fwd+bwd fp32, 224x224x3, bounded sample of %d images per step on the "
                                   "host cores" % args.cpu_batch, "per_gpu_batch": PER_GPU_BATCH},
            "cpu_baseline": base, "gpu_launches": 0,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        pk = json.load(open(path))
        return (pk["bf16_tflops_sustained"] / 2.0, pk["hbm_gbs"],
                "of measured: MEASURED_PEAKS.json bf16_tflops_sustained / 2 (kind::tf32 runs at half the bf16 rate); hbm_gbs")
    return 1400.0 / 2.0, 6650.0, "of fallback: 1.4 PFLOP/s sustained bf16 / 2; 6.65 TB/s"


def contraction_kernels(ctx, passes, peak_tf32):
    """The per-kind sums of the last profile as entries of the bench line's `kernels` list."""
    names = ["conv fprop (conv_ts_kernel; conv1_1 runs on CUDA cores and is not in this sum)",
             "conv dgrad (conv_ts_kernel, ReLU mask fused)",
             "conv wgrad + dbias (dY tile images + conv_ts_kernel in its row mode + sum of the reduction ranges; conv1_1 on CUDA cores)",
             "fully connected fprop/dgrad/wgrad (fc6 on conv_ts_kernel: weights read or written once; fc7, fc8 on tc_gemm_kernel)"]
    out = []
    for kind, name in enumerate(names):
        ms, fl, n = ctx.profile_kind(kind)
        if n == 0:
            continue
        tf = fl / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        out.append({"name": name, "bound": "tensor", "ms_per_step": ms, "contractions": n, "gflop": fl / 1e9, "tflops": tf,
                    "frac": tf / peak_tf32, "tensor_work_frac": passes * tf / peak_tf32})
    return out


def bandwidth_kernels(hbm_gbs):
    """The HBM-bound blocks at the sizes of the specification's configurations C3-C5, timed alone with CUDA events
    (layerbench.py): bytes as the algorithmic figure of each block, fraction of the measured copy bandwidth."""
    import layerbench
    import torch
    out = []
    flush = torch.empty(64 << 20, device="cuda")
    for r in layerbench.bandwidth_rows("bnorm", 5, flush)[:2]:
        out.append({"name": r["block"] + " backward", "bound": "hbm", "us": r["bwd_ms"] * 1e3, "bytes_per_element": 20,
                    "GBs": r["bwd_GBs_20B"], "frac": r["bwd_GBs_20B"] / hbm_gbs, "frac_12_bytes": r["bwd_GBs_12B"] / hbm_gbs})
    for r in layerbench.bandwidth_rows("pool", 5, flush)[:1]:
        out.append({"name": r["block"] + " backward", "bound": "hbm", "us": r["bwd_ms"] * 1e3, "GBs": r["bwd_GBs"],
                    "frac": r["bwd_GBs"] / hbm_gbs})
    for kind in ("roipool", "sampler"):
        for r in layerbench.bandwidth_rows(kind, 5, flush):
            out.append({"name": r["block"] + " backward", "bound": "hbm", "us": r["bwd_ms"] * 1e3, "bytes": r["bwd_bytes"],
                        "GBs": r["bwd_GBs"], "frac": r["bwd_GBs"] / hbm_gbs})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=PER_GPU_BATCH, help="images per GPU")
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32", "fp32"])
    ap.add_argument("--cpu-batch", type=int, default=2, help="images per step of the CPU arm (bounded sample)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel list and the plain-TF32 figure")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from matconvnet_b200 import dataparallel, mat, models, nn, simplenn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path in this engine)"
    torch.cuda.set_device(local)
    stdout_fd = None
    if world > 1:
        # NCCL prints its version banner on stdout when its first communicator comes up; only the JSON line
        # belongs there, so stdout points at stderr until the line is printed.
        sys.stdout.flush()
        stdout_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)
    precision = {"3xtf32": 0, "tf32": 1, "fp32": 2}[args.precision]

    ctx = nn.default_context()
    ctx.set_precision(precision)
    ctx.reserve_workspace(3 << 30)          # operand tile images and split-K partials; grown once, up front

    net = models.vgg16(seed=0)              # identical replica on every rank
    B = args.batch
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)      # a different shard per rank
    xs = [mat.as_mat(torch.randn(224, 224, 3, B, device="cuda", generator=gen)), mat.empty((224, 224, 3, B))]
    x = xs[0]
    labels = torch.randint(1, 1001, (B,), device="cuda", generator=gen).float()
    net["layers"][-1]["class"] = labels
    x_host = torch.empty(x.permute(3, 2, 1, 0).shape, pin_memory=True).copy_(x.permute(3, 2, 1, 0))
    labels_host = labels.cpu().pin_memory()
    loss_host = torch.zeros(2, pin_memory=True)
    one = 1.0

    # every parameter derivative is written straight into a flat bucket of the gradient exchange; one all-reduce per
    # bucket, started when its last member exists, averaging inside the reduction
    exchange = dataparallel.GradientExchange(world, average=True, scale_fn=lambda t, a: nn.scale_(t, a, ctx=ctx))
    views = exchange.plan(simplenn.gradient_specs(net), "cuda")
    key = {simplenn.grad_name(i, j): (i, j) for i in range(len(net["layers"])) for j in range(2)}
    grad_out = {key[n]: v for n, v in views.items()}

    def backward_pass(xin):
        return simplenn.vl_simplenn(net, xin, one, on_dzdw=lambda i, j, w: exchange.push(simplenn.grad_name(i, j), w), ctx=ctx,
                                    conserve_memory=True, fuse_relu=True, grad_out=grad_out)

    def step(xin=x):
        res = backward_pass(xin)
        exchange.pull_all()
        return res

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    for _ in range(warmup):
        res = step()
    ctx.device_status()
    loss0 = float(res[-1]["x"].cpu()[0])
    del res

    # ---- device-resident throughput (inputs already in HBM) ----
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    launches0 = ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    launches = (ctx.launches - launches0) // max(args.steps, 1)
    clocks = sampler.stop()

    # ---- end to end: host buffers in, loss out, copies inside the timed region ----
    # The batch of step i+1 travels from pinned host memory into the second device buffer on a copy stream while step i
    # computes; the loss of every step is copied to pinned host memory behind the step and read by the host one step later.
    compute = torch.cuda.current_stream()
    copy = torch.cuda.Stream()
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    done = [torch.cuda.Event(), torch.cuda.Event()]
    got = [torch.cuda.Event(), torch.cuda.Event()]
    lab2 = [labels, labels.clone()]

    def upload(slot):
        with torch.cuda.stream(copy):
            xs[slot].permute(3, 2, 1, 0).copy_(x_host, non_blocking=True)
            lab2[slot].copy_(labels_host, non_blocking=True)
            ready[slot].record(copy)

    barrier()
    loss = None
    e0.record()
    upload(0)
    for i in range(args.steps):
        slot = i & 1
        compute.wait_event(ready[slot])
        net["layers"][-1]["class"] = lab2[slot]
        res = step(xs[slot])
        loss_host[slot:slot + 1].copy_(res[-1]["x"], non_blocking=True)
        got[slot].record(compute)
        done[slot].record(compute)
        if i + 1 < args.steps:
            if i >= 1:
                copy.wait_event(done[slot ^ 1])     # the other buffer's last reader (step i-1) has finished
            upload(slot ^ 1)
        if i >= 1:
            got[slot ^ 1].synchronize()
            loss = float(loss_host[slot ^ 1])
    got[(args.steps - 1) & 1].synchronize()
    loss = float(loss_host[(args.steps - 1) & 1])
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    net["layers"][-1]["class"] = labels
    h2d = x_host.numel() * 4 + labels_host.numel() * 4

    # ---- where a step's time goes: the contractions by kind, and the tail of the gradient exchange ----
    exchange.bytes = 0
    exchange.collectives = 0
    barrier()
    ctx.profile_begin()
    t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    t0.record()
    backward_pass(x)
    t1.record()
    exchange.pull_all()
    t2.record()
    grad_bytes, collectives = exchange.bytes, exchange.collectives
    tc_ms, tc_flops, tc_count = ctx.profile_end()
    ctx.device_status()
    backward_ms = max_over_ranks(t0.elapsed_time(t1))
    tail_ms = max_over_ranks(t1.elapsed_time(t2))
    peak, hbm, peak_src = _peaks()
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    passes = 3 if args.precision == "3xtf32" else 1
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": None,
                "traffic_note": "DRAM bytes are captured per kernel on single layers (one kernel, a few launches) and kept under "
                                "profiles/; no whole-step counter capture is made",
                "kernel": "conv_ts_kernel (conv fprop / dgrad / wgrad, fc6) + tc_gemm_kernel (fc7, fc8), operand "
                          "preparation and the sums over reduction ranges included",
                "contractions_per_step": tc_count, "ms_per_step": tc_ms, "mma_passes": passes,
                "tensor_work_frac": passes * achieved / peak, "peak_source": peak_src,
                "note": "achieved counts each contraction's 2*M*N*K once; the 3xTF32 arithmetic issues 3 MMAs per product"}
    kernels = contraction_kernels(ctx, passes, peak)

    # ---- the plain-TF32 fast path, reported separately (one MMA per product, about 1e-3 relative error) ----
    tf32 = None
    if args.precision == "3xtf32" and not args.no_kernels:
        ctx.set_precision(1)
        for _ in range(2):
            step()
        barrier()
        e0.record()
        for _ in range(5):
            step()
        e1.record()
        barrier()
        ms_tf32 = max_over_ranks(e0.elapsed_time(e1) / 5)
        ctx.profile_begin()
        step()
        t_ms, t_fl, _ = ctx.profile_end()
        ctx.set_precision(precision)
        t_ach = t_fl / (t_ms * 1e-3) / 1e12 if t_ms > 0 else 0.0
        tf32 = {"metric": METRIC, "value": world * B / (ms_tf32 * 1e-3), "unit": UNIT, "ms_per_step": ms_tf32, "steps": 5,
                "dtype": "tf32", "arithmetic": "plain TF32: one MMA per product, parity bound 2e-3 relative L2",
                "roofline": {"bound": "tensor", "achieved": t_ach, "peak": peak, "unit": "TFLOP/s", "frac": t_ach / peak,
                             "ms_per_step": t_ms, "mma_passes": 1}}

    if world > 1:
        dist.barrier()
    if rank == 0:
        value = world * B / (ms * 1e-3)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32" if args.precision != "tf32" else "tf32", "data": "synthetic",
                "config": {"workload": "VGG-16 fwd+bwd fp32 (13 conv 3x3 + 3 conv-as-FC, relu, 5 max-pool, softmaxloss), "
                                       "224x224x3 N(0,1), He-normal weights, labels U{1..1000}",
                           "per_gpu_batch": B, "global_batch": world * B, "arithmetic": args.precision,
                           "parallelism": "dp%d" % world, "gradient_exchange_bytes": grad_bytes,
                           "gradient_exchange_collectives": collectives,
                           "l2": "inputs and activations of one step (about 15 GB) far exceed the 126 MB L2; no explicit flush",
                           "loss_first_step": loss0},
                "clocks": clocks, "gpu_launches": int(launches),
                "e2e": {"value": world * B / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e, "loss": loss,
                        "note": "input of step i+1 copied from pinned host memory on a copy stream while step i computes; "
                                "every step's loss copied back and read by the host"},
                "roofline": roofline,
                "exchange": {"backward_ms": backward_ms, "tail_after_backward_ms": tail_ms,
                             "note": "one instrumented step, max over ranks: forward+backward enqueue to completion, then the "
                                     "wait for the last all-reduce"},
                "gflop_per_image": GFLOP_PER_IMAGE,
                "step_tflops": GFLOP_PER_IMAGE * value / 1e3}
        if tf32 is not None:
            line["tf32"] = tf32
        if world == 1 and not args.no_kernels:
            try:
                del xs
                torch.cuda.empty_cache()
                kernels += bandwidth_kernels(hbm)
            except Exception as exc:      # a measuring aid: report, do not fail the bench
                kernels.append({"name": "bandwidth blocks", "error": repr(exc)})
        line["kernels"] = kernels
        if world == 1 and not args.no_cpu_baseline:
            try:
                base, _ = cpu_vgg16(4 * args.cpu_batch, 3, 1, os.cpu_count() or 1)     # about 10-15 s of host work
                line["cpu_baseline"] = base
            except Exception as exc:      # the checker is not part of the product: report, do not fail the bench
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": "failed: %r" % (exc,)}
        if stdout_fd is not None:
            sys.stdout.flush()
            os.dup2(stdout_fd, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
