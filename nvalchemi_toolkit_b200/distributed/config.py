# SPDX-License-Identifier: Apache-2.0
"""Domain-decomposition configuration (reference ``nvalchemi/distributed/config.py:31-173``)."""
from __future__ import annotations

from enum import Enum
from typing import Any

from pydantic import BaseModel, ConfigDict, model_validator


class StrategyKind(str, Enum):
    HALO = "halo"
    GRAPH_PARTITION = "graph_partition"


class HookScope(str, Enum):
    """Where a dynamics hook runs under domain decomposition: on each rank's local atoms, on the gathered global
    batch (every rank), or on the gathered batch of rank 0 only."""

    LOCAL = "local"
    GLOBAL = "global"
    RANK_ZERO = "rank_zero"


class DomainConfig(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True)
    cutoff: float
    skin: float = 0.0
    ghost_width: float | None = None          # None -> cutoff + skin (times the model's number of message passes)
    strategy: StrategyKind = StrategyKind.HALO
    compile: bool = False                      # API parity only: True warns (kernels are hand-written, nothing is traced)
    require_nondegenerate: bool = True
    #: raise (instead of warning on rank 0) when some rank's ghost layer covers the whole system: such a run is correct
    #: but exercises no halo boundary, so tests of the decomposition should switch this on
    strict_partition_health: bool = False
    mesh: Any = None
    mesh_dim: str = "domain"
    grid_dims: tuple[int, int, int] | None = None
    scripted_marshal: bool = False
    migration_hysteresis: float | None = None  # None -> skin / 2; must stay below skin
    #: Verlet skin of the neighbour list built over owned + ghost rows (None -> ``skin``).  ``skin`` sizes the ghost
    #: layer and decides when ownership and ghost lists are rebuilt; a dense system can afford a list rebuilt every step
    #: (0.0) while keeping a ghost layer that lasts many steps.
    neighbor_skin: float | None = None
    #: ghost rows through peer-mapped memory and this package's NVLink kernels (True), through ``torch.distributed``
    #: collectives only (False), or peer memory whenever the model, device and process group allow it (None)
    peer_memory: bool | None = None
    #: peer-memory engine with an integrator whose closing update is the plain half kick (NVE, NVT Langevin): the kernel that
    #: collects the ghost copies' position gradients also writes the forces and applies ``v += dt/2 F/m``, and the
    #: integrator's own closing update is skipped.  Hooks that run between AFTER_COMPUTE and BEFORE_POST_UPDATE then see the
    #: velocities AFTER the kick; switch off if a hook depends on the velocities of the half step.
    fuse_integrator_finalize: bool = True

    @model_validator(mode="after")
    def _defaults(self) -> "DomainConfig":
        if self.cutoff <= 0:
            raise ValueError("cutoff must be positive")
        if self.ghost_width is None:
            self.__dict__["ghost_width"] = self.cutoff + self.skin
        if self.migration_hysteresis is None:
            self.__dict__["migration_hysteresis"] = 0.5 * self.skin
        if self.compile or self.scripted_marshal:
            import warnings

            warnings.warn("DomainConfig.compile / scripted_marshal have no effect in this package: the distributed "
                          "forward runs precompiled kernels and is never traced", UserWarning, stacklevel=2)
        if self.neighbor_skin is None:
            self.__dict__["neighbor_skin"] = self.skin
        if self.neighbor_skin > self.skin:
            raise ValueError("neighbor_skin cannot exceed skin (the ghost layer must outlast the neighbour list)")
        if self.skin > 0 and not self.migration_hysteresis < self.skin:
            raise ValueError("migration_hysteresis must be smaller than skin")
        return self
