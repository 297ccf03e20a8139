# SPDX-License-Identifier: Apache-2.0
"""Small runtime helpers (reference ``nvalchemi/distributed/_runtime.py:37-77``): world size / rank that work with or
without an initialised process group, and the device collectives should use for the active backend."""
from __future__ import annotations

import os
from typing import Any

import torch
import torch.distributed as dist


def resolve_world_size(group: Any = None) -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group)
    return int(os.environ.get("WORLD_SIZE", "1"))


def resolve_global_rank(group: Any = None) -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group)
    return int(os.environ.get("RANK", "0"))


def resolve_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def collective_device(group: Any = None) -> torch.device:
    """Tensors handed to collectives must live here: the current CUDA device for NCCL, the CPU for gloo."""
    if dist.is_available() and dist.is_initialized() and dist.get_backend(group) == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def init_from_env(backend: str | None = None) -> tuple[int, int]:
    """Initialise the default process group from ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` (no-op for one process)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(resolve_local_rank())
        dist.init_process_group(backend)
    return resolve_global_rank(), resolve_world_size()


def mesh_group(mesh: Any, dim: str | int | None = None) -> Any:
    """Process group of one dimension of a ``DeviceMesh`` (``None``: the default group; a process group is returned as
    is).  Reference: ``nvalchemi/distributed/_core/collectives.py`` (``mesh_group``)."""
    if mesh is None:
        return None
    if isinstance(mesh, dist.ProcessGroup):
        return mesh
    if dim is None:
        return mesh.get_group()
    return mesh.get_group(dim)
