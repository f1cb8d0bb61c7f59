"""Gradient exchange for batch-sharded data parallelism: one process per GPU.

Replaces the reference's parameter server (matlab/ParameterServer.m:76-121 over
matlab/src/vl_tmove.cu, a host-staged shared-memory reduction tree).  ``push`` hands over one
parameter derivative as soon as the backward pass has produced it (the reference's push-as-you-go
schedule, matlab/simplenn/vl_simplenn.m:504-509); the all-reduce (sum) runs on the communication
backend's own stream and overlaps the remaining layers.  ``pull_all`` waits for all of them and
returns the SUMS over the workers, exactly what ``ParameterServer.pull`` returns
(ParameterServer.m:106-121): the division by the number of workers belongs to the trainer
(examples/cnn_train.m:455,482; ``train.accumulate_gradients(..., num_workers=...)`` here).
``average=True`` is for a caller that wants the mean in place instead and applies no further
normalisation (the benchmark's step): the division is then folded into the reduction itself where
the backend can do that (NCCL's averaging reduction), so no extra pass over the gradients runs.

Buckets.  Launching one collective per tensor costs a fixed latency each, and half of a network's
parameter tensors are bias vectors of a few KB.  ``plan`` therefore lays the derivatives out in a
few flat buffers, in push order, and returns views into them for the backward pass to write its
results to directly (``vl_simplenn(..., grad_out=...)``): no copies, and one collective per bucket,
issued when the bucket's last member has been pushed.

Failure detection without a GPU fault (reference: the bounded waits of vl_tmove.cu:1344-1359, which
return VLE_Timeout): ``pull_all(timeout=seconds)`` bounds each wait; a worker that never joined a
collective, or a backend error, surfaces as ``ExchangeError`` on the host, the pending list is
dropped and the exchange can be torn down between steps.

Backend: NCCL over NVLink on GPUs; gloo on CPU for tests of the host logic.
"""
import datetime

import torch
import torch.distributed as dist


class ExchangeError(RuntimeError):
    """A collective did not complete: timeout (a worker never joined) or a backend error."""


def _dense(tensor):
    """The dense buffer behind a tensor or its column-major view (the all-reduce needs contiguous memory)."""
    if tensor.is_contiguous():
        return tensor
    rev = tensor.permute(*range(tensor.dim() - 1, -1, -1))
    if not rev.is_contiguous():
        raise ValueError("gradient tensors must be dense (row- or column-major)")
    return rev


class GradientExchange:
    def __init__(self, world_size=None, average=False, scale_fn=None, bucket_bytes=32 << 20, tail_bytes=2 << 20):
        self.world = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.average = bool(average)
        self.scale_fn = scale_fn      # (tensor, alpha) -> None, in place; defaults to tensor.mul_
        self.bucket_bytes = int(bucket_bytes)
        self.tail_bytes = int(tail_bytes)      # the most the last bucket may hold (its collective cannot overlap anything)
        self.pending = []             # (names, tensors, flat buffer or None, work)
        self.bytes = 0                # bytes handed to push since the counter was last reset
        self.collectives = 0          # all-reduce calls issued since the counter was last reset
        self._bucket_of = {}          # name -> bucket index
        self._buckets = []            # dicts: flat, names, missing (set of names not yet pushed in this step)
        self._native_avg = None

    # ------------------------------------------------------------------ planning
    def plan(self, specs, device, dtype=torch.float32):
        """specs: [(name, MATLAB shape)] in the order the backward pass will push them.  Returns {name: tensor}, each a
        column-major tensor of its shape that lives inside a flat bucket; consecutive tensors share a bucket until it
        holds bucket_bytes.  Pushing exactly these tensors triggers one collective per bucket.

        The last bucket's collective starts when the backward pass ends, so all of it is waited for.  It is therefore
        kept small: if it would hold more than tail_bytes, its trailing members that fit in tail_bytes (the first layers'
        small filters, produced last) become a bucket of their own and the rest is reduced while those layers are still
        being computed."""
        self._bucket_of, self._buckets = {}, []
        out = {}
        sized = []
        for name, shape in specs:
            numel = 1
            for s in shape:
                numel *= int(s)
            sized.append((name, shape, numel, (numel + 63) // 64 * 64))     # members start on 256-byte boundaries (vector accesses)
        groups, group, size = [], [], 0
        for item in sized:
            group.append(item)
            size += item[3]
            if size * 4 >= self.bucket_bytes:
                groups.append(group)
                group, size = [], 0
        if group:
            groups.append(group)
        if groups and sum(i[3] for i in groups[-1]) * 4 > self.tail_bytes and len(groups[-1]) > 1:
            last, tail, tsize = groups[-1], [], 0
            while len(last) > 1 and (tsize + last[-1][3]) * 4 <= self.tail_bytes:
                tsize += last[-1][3]
                tail.insert(0, last.pop())
            if tail:
                groups.append(tail)
        for group in groups:
            size = sum(i[3] for i in group)
            flat = torch.zeros(size, device=device, dtype=dtype)
            names, off = [], 0
            for name, shape, numel, padded in group:
                shape = tuple(int(s) for s in shape)
                view = flat.narrow(0, off, numel).view(shape[::-1]).permute(*range(len(shape) - 1, -1, -1))
                out[name] = view
                self._bucket_of[name] = len(self._buckets)
                names.append(name)
                off += padded
            self._buckets.append(dict(flat=flat, names=names, missing=set(names), tensors={n: out[n] for n in names}))
        return out

    # ------------------------------------------------------------------ push / pull
    def _reduce_op(self, flat):
        if not self.average:
            return dist.ReduceOp.SUM, False
        if self._native_avg is None:
            self._native_avg = dist.get_backend() == "nccl" and flat.is_cuda
        return (dist.ReduceOp.AVG, False) if self._native_avg else (dist.ReduceOp.SUM, True)

    def _start(self, names, tensors, flat):
        work, scale_after = None, False
        if self.world > 1:
            op, scale_after = self._reduce_op(flat)
            try:
                work = dist.all_reduce(flat, op=op, async_op=True)
            except RuntimeError as exc:
                self.pending = []
                raise ExchangeError("all_reduce could not be started: %s" % (exc,)) from exc
            self.collectives += 1
        self.pending.append((names, tensors, flat, work, scale_after))

    def push(self, name, tensor):
        """Start summing `tensor` over all workers, in place (at once, or when its bucket is complete)."""
        self.bytes += tensor.numel() * tensor.element_size()
        b = self._bucket_of.get(name)
        if b is not None:
            bucket = self._buckets[b]
            if bucket["tensors"][name].data_ptr() != tensor.data_ptr():
                raise ValueError("'%s' was planned into a bucket: push the tensor plan() returned" % name)
            bucket["missing"].discard(name)
            if not bucket["missing"]:
                bucket["missing"] = set(bucket["names"])
                self._start(list(bucket["names"]), [bucket["tensors"][n] for n in bucket["names"]], bucket["flat"])
            return
        self._start([name], [tensor], _dense(tensor))

    def flush(self):
        """Start the collective of every bucket that has received some but not all of its members."""
        for bucket in self._buckets:
            if len(bucket["missing"]) != len(bucket["names"]):
                bucket["missing"] = set(bucket["names"])
                self._start(list(bucket["names"]), [bucket["tensors"][n] for n in bucket["names"]], bucket["flat"])

    def pull_all(self, timeout=None):
        """Wait for every pushed tensor; returns {name: tensor} holding the sums over the workers (the means when the
        exchange was built with average=True).  timeout: seconds per wait, None = the process group's own."""
        self.flush()
        out = {}
        pending, self.pending = self.pending, []
        for names, tensors, flat, work, scale_after in pending:
            if work is not None:
                try:
                    ok = work.wait() if timeout is None else work.wait(datetime.timedelta(seconds=float(timeout)))
                except RuntimeError as exc:
                    raise ExchangeError("gradient exchange of %s failed: %s" % (names, exc)) from exc
                if ok is False:
                    raise ExchangeError("gradient exchange of %s did not complete" % (names,))
            if scale_after:
                if self.scale_fn is not None:
                    self.scale_fn(flat, 1.0 / self.world)
                else:
                    flat.mul_(1.0 / self.world)
            for n, t in zip(names, tensors):
                out[n] = t
        return out
