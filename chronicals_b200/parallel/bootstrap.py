"""Process-group bootstrap: one process per GPU, ``torch.distributed`` for plumbing.

The reference is single-process (its only use of the device count is a banner,
chronicals/training/chronicals_trainer.py:689), so everything here is new.
Rendezvous always uses 127.0.0.1 on a single node (container hostnames may not
resolve).  NCCL on GPUs, gloo on CPU.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def env_world() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment (defaults: single process)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> Tuple[int, int, int]:
    """Initialise the default process group when the launcher asked for more than one rank."""
    rank, local_rank, world = env_world()
    if world <= 1:
        return rank, local_rank, world
    if dist.is_initialized():
        return dist.get_rank(), local_rank, dist.get_world_size()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    kw = {}
    if use_cuda:
        torch.cuda.set_device(local_rank)
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
    dist.init_process_group(backend=backend, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, local_rank, world


def shutdown() -> None:
    if dist.is_available() and dist.is_initialized():
        from .watchdog import stop_all
        stop_all()                                 # heartbeat threads write to the store that goes away below
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()


def is_main() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def max_over_ranks(value: float, device=None) -> float:
    """Device-timed numbers are reported as the maximum over ranks."""
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                            if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
