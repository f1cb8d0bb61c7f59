"""Gradient exchange for batch-sharded data parallelism: one process per GPU.

Replaces the reference's parameter server (matlab/ParameterServer.m:76-121 over
matlab/src/vl_tmove.cu, a host-staged shared-memory reduction tree): ``push`` starts an
asynchronous all-reduce (sum) of one parameter derivative on the communication backend's own
stream as soon as the backward pass has produced it (the reference's push-as-you-go schedule,
matlab/simplenn/vl_simplenn.m:504-509); ``pull_all`` waits for all of them and divides by the
number of workers, as the reference's trainer does (examples/cnn_train.m:455,482).
Backend: NCCL over NVLink on GPUs; gloo on CPU for tests of the host logic.
"""
import torch
import torch.distributed as dist


class GradientExchange:
    def __init__(self, world_size=None, scale_fn=None):
        self.world = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.pending = []
        self.scale_fn = scale_fn      # (tensor, alpha) -> None, in place; defaults to tensor.mul_
        self.bytes = 0

    def push(self, name, tensor):
        """Start summing `tensor` over all workers, in place."""
        self.bytes += tensor.numel() * tensor.element_size()
        if self.world > 1:
            # the all-reduce needs the dense buffer; a column-major view shares storage with it
            flat = tensor.permute(*range(tensor.dim() - 1, -1, -1)) if not tensor.is_contiguous() else tensor
            work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, async_op=True)
        else:
            work = None
        self.pending.append((name, tensor, work))

    def pull_all(self):
        """Wait for every pushed tensor and average it; returns {name: tensor}."""
        out = {}
        for name, tensor, work in self.pending:
            if work is not None:
                work.wait()
            if self.world > 1:
                if self.scale_fn is not None:
                    self.scale_fn(tensor, 1.0 / self.world)
                else:
                    tensor.mul_(1.0 / self.world)
            out[name] = tensor
        self.pending = []
        return out
