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


class DistributedManager:
    """Process-wide view of the launcher's environment and the default process group (the role physicsnemo's
    ``DistributedManager`` plays for the reference): ``initialize()`` once per process (idempotent), then ``rank``,
    ``world_size``, ``local_rank``, ``device``.  Every helper of this package that takes a ``manager`` accepts it."""

    _instance: "DistributedManager | None" = None

    def __new__(cls) -> "DistributedManager":
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance._ready = False
        return cls._instance

    @classmethod
    def is_initialized(cls) -> bool:
        return cls._instance is not None and cls._instance._ready

    @classmethod
    def initialize(cls, backend: str | None = None, **kwargs: Any) -> "DistributedManager":
        """Join the process group described by ``RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT`` (a single
        process without them), NCCL on CUDA machines, gloo otherwise."""
        import os

        me = cls()
        if me._ready:
            return me
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1 and not dist.is_initialized():
            backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if backend == "nccl":
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group(backend, **kwargs)
            me._owns_group = True
        else:
            me._owns_group = False
        me._ready = True
        return me

    @property
    def rank(self) -> int:
        return resolve_global_rank()

    @property
    def world_size(self) -> int:
        return resolve_world_size()

    @property
    def local_rank(self) -> int:
        import os

        return int(os.environ.get("LOCAL_RANK", "0"))

    @property
    def distributed(self) -> bool:
        return self.world_size > 1

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", self.local_rank) if torch.cuda.is_available() else torch.device("cpu")

    @classmethod
    def cleanup(cls) -> None:
        me = cls._instance
        if me is not None and me._ready:
            if getattr(me, "_owns_group", False) and dist.is_initialized():
                dist.destroy_process_group()
            me._ready = False
