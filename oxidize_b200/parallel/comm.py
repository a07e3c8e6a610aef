"""Process-group plumbing and the collective facade the model calls.

One process per GPU; ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks) bootstraps the
job, carries barriers, pipeline p2p and the *baseline* collectives.  The reference has no GPU
collectives at all — its only ones are a TCP ring all-reduce / all-gather
(``oxidize-core/src/mesh/ring.rs:245-365``) — so the NCCL path here is the in-repo baseline
and the fused NVLink kernels (:mod:`oxidize_b200.parallel.fused`) are the product.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelLayout:
    """World = pp × tp ranks; experts are partitioned over the tp ranks of a stage (ep = tp)."""

    world_size: int = 1
    rank: int = 0
    tp_size: int = 1
    pp_size: int = 1

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def pp_rank(self) -> int:
        return self.rank // self.tp_size


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> ParallelLayout:
    """Initialise from torchrun-style env (RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR/PORT)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s),
                                    device_id=torch.device("cuda", torch.cuda.current_device()))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s))
    return ParallelLayout(world, rank, world, 1)


class TorchComm:
    """Collectives through torch.distributed (NCCL / gloo): the unfused baseline."""

    def __init__(self, group=None):
        self.group = group
        self.size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_collectives = 0

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
            self.num_collectives += 1
        return x

    def linear_allreduce(self, x: torch.Tensor, w, residual=None) -> torch.Tensor:
        """Row-parallel projection: local GEMM, then the all-reduce as a separate collective."""
        from .. import ops

        out = self.all_reduce(ops.linear(x, w))
        return out if residual is None else out + residual

    def all_gather_cat(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.size == 1:
            return x
        x = x.contiguous()
        flat = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x, group=self.group)
        out = flat.view((self.size,) + tuple(x.shape))
        self.num_collectives += 1
        if dim in (-1, x.dim() - 1):
            return out.movedim(0, -2).reshape(*x.shape[:-1], self.size * x.shape[-1])
        parts = list(out.unbind(0))
        return torch.cat(parts, dim=dim)

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    def broadcast_object(self, obj, src: int = 0):
        if self.size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]
