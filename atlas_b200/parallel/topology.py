"""Rank topology: one OS process per GPU; world = tp x ep (orthogonal mesh) or tp == ep == world (overlapping).

Reference parity: ``crates/spark-server/src/main_modules/serve_phases/topology.rs:24-160`` and
``docs/adr/0007-tp-ep-composition.md``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..layers.common import ParallelCtx
from .comm import CommBackend, SingleGpuBackend, TorchDistBackend


@dataclass
class Topology:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    tp_size: int = 1
    ep_size: int = 1
    tp_rank: int = 0
    ep_rank: int = 0
    overlapping: bool = False

    @staticmethod
    def resolve(world_size: int, rank: int, tp_size: int = 0, ep_size: int = 0, local_rank: Optional[int] = None) -> "Topology":
        tp = tp_size or (world_size if not ep_size else max(1, world_size // ep_size))
        ep = ep_size or max(1, world_size // tp)
        if tp * ep == world_size:
            overlapping = False
            tp_rank, ep_rank = rank % tp, rank // tp
        elif tp == world_size and ep == world_size:
            overlapping = True
            tp_rank = ep_rank = rank
        else:
            raise ValueError(f"tp_size {tp} x ep_size {ep} does not tile world_size {world_size} "
                             "(use tp*ep == world or tp == ep == world)")
        return Topology(rank, world_size, rank if local_rank is None else local_rank, tp, ep, tp_rank, ep_rank, overlapping)


def init_distributed(tp_size: int = 0, ep_size: int = 0, backend: Optional[str] = None, timeout_s: float = 600.0):
    """Reads RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment (torchrun contract).

    Returns ``(Topology, ParallelCtx, device)``.  World size 1 needs no process group.
    """
    import datetime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local}") if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    topo = Topology.resolve(world, rank, tp_size, ep_size, local)
    if world == 1:
        single = SingleGpuBackend()
        return topo, ParallelCtx(comm=single, ep_comm=single), device
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        kw = {"device_id": device} if use_cuda else {}
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    if topo.overlapping or topo.ep_size == 1 or topo.tp_size == 1:
        world_comm = TorchDistBackend(None)
        tp_comm = world_comm if topo.tp_size > 1 else SingleGpuBackend()
        ep_comm = world_comm if topo.ep_size > 1 else SingleGpuBackend()
    else:
        tp_comm = ep_comm = None
        for e in range(topo.ep_size):
            g = dist.new_group([e * topo.tp_size + t for t in range(topo.tp_size)])
            if e == topo.ep_rank:
                tp_comm = TorchDistBackend(g)
        for t in range(topo.tp_size):
            g = dist.new_group([e * topo.tp_size + t for e in range(topo.ep_size)])
            if t == topo.tp_rank:
                ep_comm = TorchDistBackend(g)
    pctx = ParallelCtx(topo.tp_rank, topo.tp_size, topo.ep_rank, topo.ep_size, tp_comm, ep_comm)
    return topo, pctx, device
