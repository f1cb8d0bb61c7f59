"""The gradient exchange on two CPU ranks over gloo: the host logic of the multi-GPU path.

Closed form of the reference's own transport test (matlab/xtest/suite/tmovemex.m:42-75): every
worker starts a tensor at its 1-based rank and repeats push/pull T times accumulating the pulled SUM;
here pull returns the AVERAGE (sum / workers, examples/cnn_train.m:482), so after each round every
element equals the mean of the workers' values, and a rank that averages its own value again stays
at the fixed point (L+1)/2.
"""
import os
import socket
import sys

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


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from matconvnet_b200.dataparallel import GradientExchange
    ex = GradientExchange(world)
    # two tensors pushed in reverse-layer order, as the backward pass does; one is a column-major view
    a = torch.full((3, 5), float(rank + 1))
    b = torch.arange(24, dtype=torch.float32).reshape(4, 3, 2).permute(2, 1, 0) * (rank + 1)
    ex.push("l2_0", a)
    ex.push("l1_0", b)
    got = ex.pull_all()
    mean = (world + 1) / 2.0
    ok = torch.allclose(got["l2_0"], torch.full((3, 5), mean))
    ok &= torch.allclose(got["l1_0"], torch.arange(24, dtype=torch.float32).reshape(4, 3, 2).permute(2, 1, 0) * mean)
    ok &= got["l1_0"].data_ptr() == b.data_ptr()            # in place, like vl_tmove's 'inplace' push
    ok &= ex.bytes == (15 + 24) * 4 and ex.pending == []
    for _ in range(3):                                      # further rounds stay at the fixed point
        ex.push("l2_0", a)
        ex.pull_all()
    ok &= torch.allclose(a, torch.full((3, 5), mean))
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_gradient_exchange_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def test_single_worker_is_identity():
    sys.path.insert(0, ROOT)
    from matconvnet_b200.dataparallel import GradientExchange
    ex = GradientExchange(1)
    t = torch.randn(7)
    ref = t.clone()
    ex.push("w", t)
    assert torch.equal(ex.pull_all()["w"], ref)
