"""Data parallelism for the sparse-attention training step: one process per GPU.

The reference uses single-process ``nn.DataParallel`` (main_conv_ff.py:423: replicate the
model every step, scatter inputs, gather outputs, reduce gradients onto GPU 0) and stacks the
mask list four times so that scatter hands each replica a copy (:299).  Here every rank owns
its replica and its shard of the batch; the only exchanges are

* one all-reduce per step over a single flat gradient bucket (<= ~1.6 MB for the LRA
  encoders: latency-bound on NVLink, so one call, not one per parameter), and
* one broadcast of each layer's ``nb x nb`` byte mask when the pattern is discovered (rank 0
  discovers from its shard's map, as the reference uses replica 0's, main_conv_ff.py:255).

Everything goes through ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
from datetime import timedelta

import torch
import torch.distributed as dist


def init_from_env(backend: str | None = None, timeout_s: float = 600.0):
    """Join the process group torchrun described (RANK / WORLD_SIZE / MASTER_*).  Returns (rank, world)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world == 1:
        return 0, 1
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kw = {}
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group(backend, rank=rank, world_size=world, timeout=timedelta(seconds=timeout_s), **kw)
    return rank, world


def world_size() -> int:
    """Ranks in the job (1 when no process group was set up)."""
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def shard_range(global_batch: int, rank: int, world: int):
    """Contiguous, even split of the global batch (the benchmark configs divide evenly)."""
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} does not divide over {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


class FlatGradBucket:
    """All parameter gradients as views of one contiguous buffer; one all-reduce per step."""

    def __init__(self, params, dtype=None):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        dev = self.params[0].device
        self.dtype = dtype or self.params[0].dtype
        n = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(n, dtype=self.dtype, device=dev)
        off = 0
        for p in self.params:
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()
        self.nbytes = n * self.flat.element_size()

    def zero(self):
        self.flat.zero_()

    def allreduce_mean(self, async_op: bool = False):
        """Average gradients over ranks.  With async_op the handle is returned (wait before the optimizer)."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return None
        self.flat.div_(dist.get_world_size())
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, async_op=async_op)
        return work


def broadcast_mask(mat: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Every rank ends up with rank ``src``'s [nb, nb] uint8 mask (nb*nb bytes on the wire)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(mat, src=src)
    return mat


def average_map(A: torch.Tensor) -> torch.Tensor:
    """Optional variant: all ranks average their local mean attention maps (4*L*L bytes) before
    discovery, so the mask reflects the global batch rather than rank 0's shard."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(A, op=dist.ReduceOp.SUM)
        A.div_(dist.get_world_size())
    return A


def agree_on_masks(local_maps, discover, average: bool = False):
    """``discover(A) -> uint8 [nb, nb] tensor`` runs on rank 0 only (or on every rank after
    averaging); the result is broadcast.  Returns the list of masks, identical on all ranks."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    masks = []
    for A in local_maps:
        if average:
            A = average_map(A.clone())
        if rank == 0 or average:
            m = discover(A)
        else:
            nb = None
            m = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            shape = torch.tensor(list(m.shape) if m is not None else [0, 0], device=A.device)
            dist.broadcast(shape, src=0)
            if m is None:
                m = torch.empty(int(shape[0]), int(shape[1]), dtype=torch.uint8, device=A.device)
            m = broadcast_mask(m.contiguous(), 0)
        masks.append(m)
    return masks
