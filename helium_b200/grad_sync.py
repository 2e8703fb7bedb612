"""Data-parallel gradient reduction for the training-step configurations.

The hot path shards by batch / tokens: every kernel works on its own rank's rows, and the only
cross-rank dependency is the sum of the weight and bias gradients (the reference has no multi-GPU
code at all; its optimiser consumes whatever gradient tensor it is handed, helium/src/optimizer/sgd.rs:35-62).
`GradReducer` is that one exchange step: gradients are grouped into buckets in the order the
backward pass produces them, each bucket is all-reduced (NCCL on GPUs, gloo on CPU for the host-logic
tests) on a side stream as soon as its producer kernel has been enqueued, and `finish()` joins the
side stream back before the optimiser would read the gradients.

Reduction is the MEAN over ranks (sum / world): helium's cross-entropy divides by the local batch
(helium/src/loss.rs:5-8), so the mean of per-rank gradients is the gradient of the mean loss over the
global batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


class GradReducer:
    def __init__(self, process_group=None, mean: bool = True):
        import torch.distributed as dist

        self.dist = dist
        self.group = process_group
        self.enabled = dist.is_available() and dist.is_initialized() and dist.get_world_size(process_group) > 1
        self.world = dist.get_world_size(process_group) if self.enabled else 1
        self.mean = mean
        self._pending = []
        self._stream = None
        self.bytes_reduced = 0
        self.collectives = 0

    def _side_stream(self, device):
        import torch

        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        return self._stream

    def reduce_bucket(self, tensors: Sequence, after_event=None) -> None:
        """Starts the all-reduce of one bucket.  `tensors` must be views of memory that stays untouched
        until finish(); on CUDA the collective is ordered after `after_event` (or after everything
        enqueued so far on the current stream when no event is given)."""
        import torch

        if not tensors:
            return
        for t in tensors:
            self.bytes_reduced += t.numel() * t.element_size()
        if not self.enabled:
            return
        op = self.dist.ReduceOp.SUM
        on_cuda = tensors[0].is_cuda
        if on_cuda:
            side = self._side_stream(tensors[0].device)
            ev = after_event
            if ev is None:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
            side.wait_event(ev)
            with torch.cuda.stream(side):
                for t in tensors:
                    if self.mean and self.dist.get_backend(self.group) == "nccl":
                        w = self.dist.all_reduce(t, op=self.dist.ReduceOp.AVG, group=self.group, async_op=True)
                        self._pending.append((w, None))
                    else:
                        w = self.dist.all_reduce(t, op=op, group=self.group, async_op=True)
                        self._pending.append((w, t if self.mean else None))
                    self.collectives += 1
        else:
            for t in tensors:
                w = self.dist.all_reduce(t, op=op, group=self.group, async_op=True)
                self._pending.append((w, t if self.mean else None))
                self.collectives += 1

    def finish(self) -> None:
        """Joins every started bucket: afterwards the current stream (or the host, on CPU) sees the
        reduced gradients."""
        import torch

        for w, scale_me in self._pending:
            w.wait()
            if scale_me is not None:
                scale_me.mul_(1.0 / self.world)
        self._pending.clear()
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)


class CommReducer:
    """The same bucket / finish interface over the library's own communicator (he_comm, NCCL behind the C
    ABI) instead of torch.distributed: each bucket is one he_allreduce_grads call on a side stream, ordered
    after the producer kernel by an event.  This is the path a non-Python host takes."""

    def __init__(self, comm, mean: bool = True):
        self.comm = comm
        self.world = comm.world
        self.enabled = comm.world > 1
        self.mean = mean
        self._stream = None
        self._dirty = False
        self.bytes_reduced = 0
        self.collectives = 0

    def reduce_bucket(self, tensors: Sequence, after_event=None) -> None:
        import torch

        if not tensors:
            return
        for t in tensors:
            self.bytes_reduced += t.numel() * t.element_size()
        if not self.enabled:
            return
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=tensors[0].device)
        ev = after_event
        if ev is None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
        self._stream.wait_event(ev)
        self.comm.allreduce(list(tensors), mean=self.mean, stream=self._stream)
        self.collectives += len(tensors)
        self._dirty = True

    def finish(self) -> None:
        import torch

        if self._dirty:
            torch.cuda.current_stream().wait_stream(self._stream)
            self._dirty = False
        self.comm.poll()   # an asynchronous NCCL error surfaces here, once per step


def shard_rows(total_rows: int, world: int, rank: int) -> range:
    """Rows of a batch-sharded tensor owned by `rank`: contiguous blocks, the first `total % world`
    ranks one row longer."""
    base, extra = divmod(total_rows, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def bucket_by_bytes(sizes_bytes: Sequence[int], cap_bytes: int) -> List[List[int]]:
    """Greedy bucketing in production order: a bucket closes once it holds >= cap_bytes.  Large
    buckets amortise launch latency; NVSwitch gives every pair full bandwidth, so nothing is gained
    from more, smaller collectives."""
    buckets: List[List[int]] = []
    cur: List[int] = []
    acc = 0
    for i, s in enumerate(sizes_bytes):
        cur.append(i)
        acc += s
        if acc >= cap_bytes:
            buckets.append(cur)
            cur, acc = [], 0
    if cur:
        buckets.append(cur)
    return buckets


__all__ = ["GradReducer", "CommReducer", "shard_rows", "bucket_by_bytes"]
