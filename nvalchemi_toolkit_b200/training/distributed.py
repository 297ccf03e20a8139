# SPDX-License-Identifier: Apache-2.0
"""Rank helpers that accept either a manager object (duck-typed ``rank / world_size / local_rank``) or plain
``torch.distributed`` (reference ``nvalchemi/training/distributed.py:84-217``)."""
from __future__ import annotations

import os
from typing import Any

import torch
import torch.distributed as dist


def _ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_rank(manager: Any = None) -> int:
    if manager is not None and hasattr(manager, "rank"):
        return int(manager.rank)
    return dist.get_rank() if _ready() else int(os.environ.get("RANK", "0"))


def get_world_size(manager: Any = None) -> int:
    if manager is not None and hasattr(manager, "world_size"):
        return int(manager.world_size)
    return dist.get_world_size() if _ready() else int(os.environ.get("WORLD_SIZE", "1"))


def get_local_rank(manager: Any = None) -> int:
    if manager is not None and hasattr(manager, "local_rank"):
        return int(manager.local_rank)
    return int(os.environ.get("LOCAL_RANK", "0"))


def init_distributed(backend: str | None = None, **kwargs: Any) -> None:
    if _ready():
        return
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend == "nccl":
        torch.cuda.set_device(get_local_rank())
    dist.init_process_group(backend, **kwargs)


def destroy_distributed() -> None:
    if _ready():
        dist.destroy_process_group()


def barrier(manager: Any = None) -> None:
    if _ready():
        dist.barrier()


def all_reduce(t: torch.Tensor, op: str = "sum", manager: Any = None) -> torch.Tensor:
    if _ready() and get_world_size(manager) > 1:
        dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op])
    return t
