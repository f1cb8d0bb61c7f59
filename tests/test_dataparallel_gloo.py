"""The gradient exchange on two CPU ranks over gloo: the host logic of the multi-GPU path.

Closed form of the reference's own transport test (matlab/xtest/suite/tmovemex.m:42-75): every
worker starts a tensor at its 1-based rank and pushes it; pull returns the SUM over the workers,
L(L+1)/2 per element, as ParameterServer.pull does.  With average=True the exchange returns the mean
instead (sum / workers, the trainer's own normalisation, examples/cnn_train.m:482), and a rank that
averages its own value again stays at the fixed point (L+1)/2.  Also covered: buckets (several
tensors, one collective), the trainer's single normalisation, and a wait that times out because a
worker never joined.
"""
import os
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _worker(rank, world, port, out):
    _init(rank, world, port)
    from matconvnet_b200.dataparallel import GradientExchange
    total = world * (world + 1) / 2.0
    mean = (world + 1) / 2.0
    # sums, as ParameterServer.pull: two tensors pushed in reverse-layer order, one a column-major view
    ex = GradientExchange(world)
    a = torch.full((3, 5), float(rank + 1))
    b = torch.arange(24, dtype=torch.float32).reshape(4, 3, 2).permute(2, 1, 0) * (rank + 1)
    ex.push("l2_0", a)
    ex.push("l1_0", b)
    got = ex.pull_all()
    ok = torch.allclose(got["l2_0"], torch.full((3, 5), total))
    ok &= torch.allclose(got["l1_0"], torch.arange(24, dtype=torch.float32).reshape(4, 3, 2).permute(2, 1, 0) * total)
    ok &= got["l1_0"].data_ptr() == b.data_ptr()            # in place, like vl_tmove's 'inplace' push
    ok &= ex.bytes == (15 + 24) * 4 and ex.pending == [] and ex.collectives == 2
    # means: further rounds stay at the fixed point
    exa = GradientExchange(world, average=True)
    a = torch.full((3, 5), float(rank + 1))
    for _ in range(3):
        exa.push("l2_0", a)
        exa.pull_all()
    ok &= torch.allclose(a, torch.full((3, 5), mean))
    # buckets: four tensors, planned into two buckets, one collective each, results in the planned views
    exb = GradientExchange(world, bucket_bytes=700)
    specs = [("l3_0", (5, 4, 3, 2)), ("l3_1", (1, 2)), ("l1_0", (3, 3, 1, 7)), ("l1_1", (1, 7))]
    views = exb.plan(specs, "cpu")
    ok &= all(tuple(views[n].shape) == s for n, s in specs)
    ok &= all(views[n].permute(*range(views[n].dim() - 1, -1, -1)).is_contiguous() for n, _ in specs)   # column-major
    ok &= len(exb._buckets) == 2
    for n, s in specs:
        views[n].fill_(float(rank + 1) * (1 + len(s)))
        exb.push(n, views[n])
    got = exb.pull_all()
    ok &= exb.collectives == 2
    ok &= all(torch.allclose(got[n], torch.full(s, total * (1 + len(s)))) for n, s in specs)
    # a partly filled bucket is sent by pull_all
    views["l3_0"].fill_(1.0)
    exb.push("l3_0", views["l3_0"])
    ok &= torch.allclose(exb.pull_all()["l3_0"], torch.full((5, 4, 3, 2), float(world)))
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_gradient_exchange_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def _timeout_worker(rank, world, port, out):
    _init(rank, world, port)
    from matconvnet_b200.dataparallel import ExchangeError, GradientExchange
    ex = GradientExchange(world)
    a = torch.ones(8)
    ex.push("first", a)                      # both workers join this one
    ex.pull_all(timeout=20)
    ok = torch.allclose(a, torch.full((8,), float(world)))
    if rank == 0:
        ex.push("second", a)                 # worker 1 never joins: it left between two steps
        t0 = time.time()
        try:
            ex.pull_all(timeout=2)
            ok = False
        except ExchangeError:
            ok &= time.time() - t0 < 15 and ex.pending == []
    else:
        time.sleep(4)
    out[rank] = bool(ok)
    os._exit(0)                              # no orderly shutdown of a group whose collective failed


def test_a_worker_that_never_joins_surfaces_as_an_error_on_the_host():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_timeout_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    assert dict(out) == {0: True, 1: True}


def test_single_worker_is_identity():
    sys.path.insert(0, ROOT)
    from matconvnet_b200.dataparallel import GradientExchange
    ex = GradientExchange(1)
    t = torch.randn(7)
    ref = t.clone()
    ex.push("w", t)
    assert torch.equal(ex.pull_all()["w"], ref)
    exa = GradientExchange(1, average=True)
    exa.push("w", t)
    assert torch.equal(exa.pull_all()["w"], ref)


def test_the_last_bucket_is_kept_small():
    """The collective of the last bucket starts when the backward pass ends and is waited for in full, so the planner
    splits the trailing small tensors (at most tail_bytes) off a last bucket that would hold more."""
    sys.path.insert(0, ROOT)
    from matconvnet_b200.dataparallel import GradientExchange
    specs = [("a", (1000,)), ("b", (1000,)), ("c", (300,)), ("d", (40,)), ("e", (10,))]
    ex = GradientExchange(1, bucket_bytes=6000, tail_bytes=1600)
    views = ex.plan(specs, "cpu")
    assert [b["names"] for b in ex._buckets] == [["a", "b"], ["c"], ["d", "e"]]
    assert all(tuple(views[n].shape) == s for n, s in specs)
    # a last bucket that is small enough stays whole; one whose last member alone is too large is not split
    ex = GradientExchange(1, bucket_bytes=6000, tail_bytes=4000)
    ex.plan(specs, "cpu")
    assert [b["names"] for b in ex._buckets] == [["a", "b"], ["c", "d", "e"]]
    ex = GradientExchange(1, bucket_bytes=1 << 20, tail_bytes=100)
    ex.plan(specs, "cpu")
    assert [b["names"] for b in ex._buckets] == [["a", "b", "c", "d", "e"]]
    # every tensor still lands where it was planned and comes back from pull_all
    ex = GradientExchange(1, bucket_bytes=6000, tail_bytes=1600)
    views = ex.plan(specs, "cpu")
    for i, (n, s) in enumerate(specs):
        views[n].fill_(float(i + 1))
        ex.push(n, views[n])
    got = ex.pull_all()
    assert all(torch.equal(got[n], torch.full(s, float(i + 1))) for i, (n, s) in enumerate(specs))


def test_vgg16_gradients_are_planned_into_five_buckets_with_a_small_last_one():
    """The benchmark's network: filters and biases of fc8 ... conv1_1 in the order the backward pass produces them."""
    sys.path.insert(0, ROOT)
    from matconvnet_b200.dataparallel import GradientExchange
    convs = [(3, 64), (64, 64), (64, 128), (128, 128), (128, 256), (256, 256), (256, 256), (256, 512), (512, 512), (512, 512),
             (512, 512), (512, 512), (512, 512)]
    fcs = [((7, 7, 512, 4096), 4096), ((1, 1, 4096, 4096), 4096), ((1, 1, 4096, 1000), 1000)]
    specs = []
    for i, (shape, k) in enumerate(reversed(fcs)):
        specs += [("fc%d_f" % i, shape), ("fc%d_b" % i, (1, k))]
    for i, (c, k) in enumerate(reversed(convs)):
        specs += [("conv%d_f" % i, (3, 3, c, k)), ("conv%d_b" % i, (1, k))]
    ex = GradientExchange(2, average=True)
    ex.plan(specs, "meta")
    sizes = [b["flat"].numel() * 4 for b in ex._buckets]
    assert len(sizes) == 5
    assert sizes[-1] <= 2 << 20 and sizes[-2] > 8 << 20          # the tail is small; what was cut off it goes out earlier
    assert sum(len(b["names"]) for b in ex._buckets) == len(specs)
    assert ex._buckets[-1]["names"][-1] == "conv12_b"            # the first layer's bias is produced last
