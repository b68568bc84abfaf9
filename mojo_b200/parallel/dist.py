"""One process per GPU. `torch.distributed` carries the plumbing (rendezvous, handle exchange, host-side control
messages, and the NCCL collectives used as baseline/oracle); the hot-path transfers are the library's own
kernels over peer memory (see `symm.py`, `tp.py`, `ep.py`)."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DistInfo:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    group: object = None        # device collectives (nccl on CUDA, gloo on CPU)
    host_group: object = None   # gloo group for small host-side control messages


_INFO: DistInfo | None = None


def init_distributed(device_type: str | None = None, timeout_s: float = 600.0) -> DistInfo:
    """Initialise from the torchrun environment (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT).
    A single process without those variables gets a world of one and no process group."""
    global _INFO
    if _INFO is not None:
        return _INFO
    import datetime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    device = torch.device("cuda", local) if device_type == "cuda" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    group = host_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        backend = "nccl" if device.type == "cuda" else "gloo"
        to = datetime.timedelta(seconds=timeout_s)
        if not dist.is_initialized():
            if backend == "nccl":
                dist.init_process_group(backend, rank=rank, world_size=world, timeout=to, device_id=device)
            else:
                dist.init_process_group(backend, rank=rank, world_size=world, timeout=to)
        group = dist.group.WORLD
        host_group = dist.new_group(backend="gloo", timeout=to) if backend == "nccl" else group
    _INFO = DistInfo(rank, world, local, device, group, host_group)
    return _INFO


def host_broadcast_object(obj, info: DistInfo, src: int = 0):
    """Broadcast a small Python object from `src` over the host (gloo) group."""
    if info.world_size == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=info.host_group)
    return box[0]


def shutdown() -> None:
    global _INFO
    if dist.is_initialized():
        dist.destroy_process_group()
    _INFO = None
