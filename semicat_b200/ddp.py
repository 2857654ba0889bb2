"""Data-parallel plumbing for the DiT training measurement: one process per GPU, the batch sharded over
ranks, one gradient all-reduce (SUM, then / world) per optimiser step over NCCL.  This is what the
reference gets from Lightning's ``strategy: ddp`` (configs/trainer/ddp.yaml:4-9); the attention kernels are
oblivious to it, and nothing else is exchanged between ranks.

Gradients live in one flat fp32 buffer (every ``p.grad`` is a view into it), so the exchange is a single
large NCCL all-reduce with no packing copies; over NVSwitch the cost is bandwidth of one 0.4-0.6 GB message,
about 1-2 ms next to a step of hundreds of milliseconds, so it is not split into overlapped buckets.
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

    def zero(self):
        self.flat.zero_()

    def all_reduce_mean(self, check_finite_on_host: bool = False):
        """Average the gradients over the ranks in place.  No-op without a process group."""
        if not dist.is_available() or not dist.is_initialized():
            return
        world = dist.get_world_size(self.group)
        if world == 1:
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
