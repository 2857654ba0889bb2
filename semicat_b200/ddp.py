"""Data-parallel plumbing for the DiT training measurement: one process per GPU, the batch sharded over
ranks, one gradient all-reduce (SUM, then / world) per optimiser step over NCCL.  This is what the
reference gets from Lightning's ``strategy: ddp`` (configs/trainer/ddp.yaml:4-9); the attention kernels are
oblivious to it, and nothing else is exchanged between ranks.

Gradients live in one flat fp32 buffer (every ``p.grad`` is a view into it), so the exchange needs no packing
copies.  As one message it takes about 1.6 ms over NVSwitch (0.56 GB); with the step down to some 20 ms per GPU that
is worth hiding, so ``FlatGradients.overlap_buckets(n)`` splits the buffer into contiguous buckets and all-reduces
each on a second stream as soon as autograd has accumulated the last gradient in it.  Parameters sit in the buffer in
forward order, so the buckets complete from the back (output head first, embedding last).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_from_env(backend: str | None = None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun).
    Returns (rank, world, local_rank).  With WORLD_SIZE unset or 1 no group is created."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, **kw)
    return rank, world, local


def shard_bounds(global_batch: int, rank: int, world: int):
    """Contiguous, as-even-as-possible split of the global batch (the reference's per-device batch split,
    semicat/data/text8.py:98-103, requires divisibility; this does not)."""
    base, rem = divmod(global_batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class FlatGradients:
    """Owns one flat fp32 gradient buffer and points every parameter's ``.grad`` into it."""

    def __init__(self, params, group=None):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        self.group = group
        dev = self.params[0].device
        total = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        off = 0
        for p in self.params:
            if p.dtype != torch.float32:
                raise TypeError("FlatGradients expects fp32 master parameters (bf16 enters through autocast)")
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()

        self._buckets = None

    def zero(self):
        self.flat.zero_()
        if self._buckets is not None:
            self._pending = [len(b[2]) for b in self._buckets]
            self._sent = [False] * len(self._buckets)

    # ---- overlapped exchange -------------------------------------------------------------------------------------
    def overlap_buckets(self, n_buckets: int = 4):
        """Split the flat buffer into ``n_buckets`` contiguous parts of about equal size (on parameter boundaries) and
        all-reduce each as soon as its last gradient has been accumulated during ``backward()``, on a second stream
        (CUDA) or in place (CPU).  Call :meth:`zero` before every backward and :meth:`all_reduce_mean` after it: it sends
        what the hooks did not (buckets with a parameter that received no gradient) and joins the second stream."""
        if self._buckets is not None:
            raise RuntimeError("overlap_buckets() was already called")
        total, target = self.flat.numel(), self.flat.numel() / max(n_buckets, 1)
        buckets, start, off, members = [], 0, 0, []
        for p in self.params:
            members.append(p)
            off += p.numel()
            if off - start >= target and len(buckets) < n_buckets - 1:
                buckets.append((start, off, members))
                start, members = off, []
        if members:
            buckets.append((start, total, members))
        self._buckets = buckets
        self._comm = torch.cuda.Stream(self.flat.device) if self.flat.is_cuda else None
        for i, (_, _, ps) in enumerate(buckets):
            for p in ps:
                p.register_post_accumulate_grad_hook(lambda _p, i=i: self._accumulated(i))
        self.zero()
        return len(buckets)

    def _active(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def _accumulated(self, i: int):
        self._pending[i] -= 1
        if self._pending[i] < 0:
            raise RuntimeError("FlatGradients.overlap_buckets: a second backward() since the last zero(); buckets of the first "
                               "one have already been exchanged (accumulate over micro-batches without overlap_buckets)")
        if self._pending[i] == 0 and self._active():
            self._send(i)

    def _send(self, i: int):
        lo, hi, _ = self._buckets[i]
        part = self.flat[lo:hi]
        world = dist.get_world_size(self.group)
        self._sent[i] = True
        if self._comm is None:
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            part.div_(world)
            return
        self._comm.wait_stream(torch.cuda.current_stream(self.flat.device))  # the accumulations into this bucket
        with torch.cuda.stream(self._comm):
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            part.div_(world)

    def all_reduce_mean(self, check_finite_on_host: bool = False):
        """Average the gradients over the ranks in place.  No-op without a process group."""
        if not self._active():
            return
        world = dist.get_world_size(self.group)
        if self._buckets is not None:
            for i in range(len(self._buckets)):
                if not self._sent[i]:
                    self._send(i)
            if self._comm is not None:
                torch.cuda.current_stream(self.flat.device).wait_stream(self._comm)
            if check_finite_on_host and not bool(torch.isfinite(self.flat).all()):
                raise FloatingPointError("non-finite gradient after all-reduce")
            return
        for p in self.params:  # autograd may have re-pointed a grad (e.g. after set_to_none); restore the view
            if p.grad is None or p.grad.data_ptr() < self.flat.data_ptr() or \
                    p.grad.data_ptr() >= self.flat.data_ptr() + self.flat.numel() * 4:
                raise RuntimeError("a parameter's .grad left the flat buffer; use FlatGradients.zero(), not zero_grad(set_to_none=True)")
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
        self.flat.div_(world)
        if check_finite_on_host and not bool(torch.isfinite(self.flat).all()):
            raise FloatingPointError("non-finite gradient after all-reduce")

    def nbytes(self) -> int:
        return self.flat.numel() * 4
