# SPDX-License-Identifier: Apache-2.0
"""``DistributedModel``: evaluates any ``BaseModelMixin`` wrapper on a :class:`ShardedBatch`.

Reference: ``nvalchemi/distributed/distributed_model.py:120-380`` and ``output_consolidation.py`` (reverse-halo force
correction, sums of per-system quantities).  The model runs unchanged on the padded (owned + ghost) cluster; the spec
selects how results are consolidated:

* ``DIRECT_MASKED``: ghost rows get an empty neighbour list; owned rows are complete as computed.
* ``WEIGHTED_ENERGY``: the model differentiates ``sum_i w_i e_i`` (``w = 1`` owned, ``0`` ghost); gradients that land on
  ghost rows are returned to the owners with a reverse halo exchange.
* ``REPLICATED``: no neighbours involved; the model runs on the owned rows only.

Per-system sums (energy, virial, stress) are all-reduced; every rank ends up with the full values.
"""
from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from nvalchemi_toolkit_b200.distributed.config import DomainConfig
from nvalchemi_toolkit_b200.distributed.sharded_batch import ShardedBatch
from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec
from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook


def consolidate_outputs(out: dict, sharded: ShardedBatch, spec: MLIPSpec, halo: Any = None) -> dict:
    """Owned-row views of node outputs (with the reverse-halo correction) and globally summed system outputs."""
    n = sharded.n_owned
    halo = halo if halo is not None else sharded.halo
    debug = os.environ.get("NVA_CONSOLIDATE_DEBUG", "0") not in ("", "0") and sharded.rank == 0
    n_ghost = halo.n_ghost if spec.consolidation != Consolidation.REPLICATED else 0
    res: dict[str, Any] = {}
    for key, value in out.items():
        if not isinstance(value, torch.Tensor):
            res[key] = value
            continue
        if debug:
            rule = "all-reduce" if key in spec.extensive_outputs else ("owned rows" + (
                " + reverse halo" if key == "forces" and spec.consolidation == Consolidation.WEIGHTED_ENERGY else "")
                if value.dim() >= 1 and value.shape[0] == n + n_ghost else "pass-through")
            print(f"[consolidate] {key}: shape {tuple(value.shape)} -> {rule}", flush=True)
        if key in spec.extensive_outputs:
            v = value.detach().clone()
            if sharded.world > 1:
                dist.all_reduce(v, group=sharded.group)
            res[key] = v
        elif value.dim() >= 1 and value.shape[0] == n + n_ghost:
            own = value.detach()[:n].clone()
            if key == "forces" and spec.consolidation == Consolidation.WEIGHTED_ENERGY:
                halo.reverse_add(value.detach()[n:], own)  # collective: every rank takes part
            res[key] = own
        else:
            res[key] = value.detach()
    return res


def partition_health_verdict(n_owned: int, n_padded: int, group: Any, device: Any) -> tuple[bool, bool, int]:
    """``(any_empty, any_trivial, n_global)``, identical on every rank (reference ``distributed_model.py:200-227``):
    some rank owns nothing; some rank's owned + ghost rows already cover every atom (correct, but that rank does the
    whole system's work).  One SUM for the atom count and one MAX over the two flags, so that no rank acts alone."""
    import torch.distributed as dist

    total = torch.tensor([float(n_owned)], dtype=torch.float64, device=device)
    flags_in = None
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(total, group=group)
    n_global = int(round(float(total)))
    flags_in = torch.tensor([int(n_owned == 0), int(n_padded >= n_global)], dtype=torch.int32, device=device)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(flags_in, op=dist.ReduceOp.MAX, group=group)
    return bool(flags_in[0]), bool(flags_in[1]), n_global


def resolve_partition_health(any_empty: bool, any_trivial: bool, n_global: int, *, world_size: int, strict: bool,
                             rank: int) -> str | None:
    """Act on a verdict (no collectives: every rank holds the same flags and therefore does the same thing).  An empty
    rank is always an error.  A trivial decomposition (a rank whose halo covers the whole system) raises when ``strict``
    (a force-equivalence check would prove nothing about the halo path), else rank 0 warns.  Returns the message."""
    if any_empty:
        raise RuntimeError(f"degenerate domain decomposition: a rank owns no atoms (world size {world_size}, {n_global} "
                           "atoms); use fewer ranks or a larger system")
    if not any_trivial or world_size == 1:
        return None
    msg = (f"trivial domain decomposition: a rank's ghost layer already covers all {n_global} atoms, so it evaluates the "
           "whole system and nothing is gained from the decomposition (box / ranks <= about 2 x ghost width); use fewer "
           "ranks or a larger system")
    if strict:
        raise RuntimeError(msg + " (strict_partition_health=True)")
    if rank == 0:
        import warnings

        warnings.warn(msg + "; results are still correct", RuntimeWarning, stacklevel=3)
    return msg


def _keep_owned_senders(padded: Any, n_owned: int) -> None:
    """Edge partition for folding policies: a rank keeps the edges whose SENDER it owns (the receiver may be a ghost, its
    partial sum is folded into the owner afterwards), so every edge is evaluated exactly once over all ranks.  Rows of
    the neighbour matrix are re-compacted in place (idempotent)."""
    nm, num = padded.neighbor_matrix, padded.num_neighbors
    k = nm.shape[1]
    slot = torch.arange(k, device=nm.device)[None, :]
    valid = (slot < num.long()[:, None]) & (nm.long() < n_owned)
    order = torch.argsort((~valid).to(torch.int8), dim=1, stable=True)
    nm.copy_(torch.gather(nm, 1, order))
    sh = padded.neighbor_matrix_shifts
    if sh is not None:
        sh.copy_(torch.gather(sh, 1, order[..., None].expand(-1, -1, sh.shape[-1])))
    num.copy_(valid.sum(1).to(num.dtype))


def _keep_edges(padded: Any, keep: torch.Tensor) -> None:
    """Edge-list form of the two rules above: every edge ``(receiver, sender)`` exists on each rank that holds both
    atoms, so a per-receiver sum must see it on exactly one of them.  The edge group is rebuilt from the kept rows (one
    system per padded batch, so the per-system edge count is the number kept).  Reference: the edge-list branch of
    ``nvalchemi/distributed/distributed_model.py`` marks such rows as padding for the wrappers to drop."""
    from nvalchemi_toolkit_b200.data.level_storage import SegmentedLevelStorage

    edges = padded._storage.groups["edges"]
    data = {k: v[keep] for k, v in edges.data.items()}
    n = int(next(iter(data.values())).shape[0]) if data else 0
    counts = torch.zeros(padded.num_graphs, dtype=torch.int32, device=keep.device)
    if n:
        owner = padded.batch_idx.long()[data["neighbor_list"][:, 0]]
        counts = torch.bincount(owner, minlength=padded.num_graphs).to(torch.int32)
    padded._storage.groups["edges"] = SegmentedLevelStorage(data, counts, num_elements=n, device=padded.device)


class DistributedModel(nn.Module):
    def __init__(self, model: Any, config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None,
                 max_neighbors: int | None = None, own_halo: bool = False) -> None:
        super().__init__()
        self.model, self.config, self.group, self.own_halo = model, config, group, own_halo
        self.spec = spec if spec is not None else model.distribution_spec(config.strategy)
        if self.spec is None:
            raise ValueError(f"{type(model).__name__} declares no distribution spec; pass spec=MLIPSpec(...)")
        from nvalchemi_toolkit_b200.distributed.config import StrategyKind

        graph = StrategyKind(config.strategy) == StrategyKind.GRAPH_PARTITION
        if graph and self.spec.message_passes > 1 and not self.spec.refresh_per_layer:
            # index blocks keep one hop of senders; deeper models refresh those rows before every layer
            self.spec = self.spec.with_(refresh_per_layer=True)
        self.engine: Any = None
        if spec is None and not own_halo and config.peer_memory is not False and not graph:
            from nvalchemi_toolkit_b200.distributed.peer_halo import PeerHaloEngine, peer_memory_available

            params = list(model.parameters()) if isinstance(model, nn.Module) else []
            device = params[0].device if params else torch.device("cpu")
            if peer_memory_available(model, device, group):
                # ghost layer one cutoff (+ skin) deep, feature rows refreshed from the owners before every interaction
                self.spec = self.spec.with_(name=self.spec.name + "_peer", refresh_per_layer=True)
                self.engine = PeerHaloEngine(model, config, group, max_neighbors=max_neighbors)
            elif config.peer_memory:
                raise RuntimeError("peer_memory=True needs a float32 native MACE on CUDA under an NCCL group of >= 2 ranks")
        self.model_config = model.model_config
        nc = self.model_config.neighbor_config
        self.neighbor_hook = NeighborListHook(nc, skin=config.neighbor_skin, max_neighbors=max_neighbors) if nc is not None else None
        if nc is not None and self.spec.requires_full_list and nc.half_list:
            raise ValueError("domain decomposition needs a full neighbour list (each owned row must be complete)")
        self._halo_builds = -1
        self.last_dispatch_stats: dict = {}
        self.partition_health: str | None = None  # message of the one-time check (None: healthy or not yet run)
        self._health_checked = False

    @property
    def wants_local_periodic(self) -> bool:
        """The peer-memory engine keeps uncut periodic dimensions periodic in the local cluster."""
        return self.engine is not None

    def forward(self, sharded: ShardedBatch, **kwargs: Any) -> dict:
        spec = self.spec
        if self.engine is not None:
            return self.engine.forward(sharded, set(self.model_config.active_outputs))
        if spec.consolidation == Consolidation.REPLICATED:
            out = self.model(sharded.owned, **kwargs)
            return consolidate_outputs(dict(out), sharded, spec)
        halo = sharded.halo_for(spec.ghost_width(self.config.cutoff, self.config.skin)) if self.own_halo else sharded.halo
        padded = sharded.padded_batch(halo)
        if not self._health_checked:  # once, at the first halo forward (two small collectives)
            self._health_checked = True
            empty, trivial, n_global = partition_health_verdict(sharded.n_owned, sharded.n_owned + halo.n_ghost, self.group,
                                                                padded.positions.device)
            self.partition_health = resolve_partition_health(
                empty and self.config.require_nondegenerate, trivial, n_global, world_size=sharded.world,
                strict=self.config.strict_partition_health, rank=sharded.rank)
        if self.neighbor_hook is not None:
            if halo.num_builds != self._halo_builds:  # ghost rows changed identity: start from a fresh list
                self.neighbor_hook._bufs = None
                self._halo_builds = halo.num_builds
            self.neighbor_hook(SimpleNamespace(batch=padded), None)
            coo = getattr(padded, "neighbor_matrix", None) is None  # an edge-list model (``NeighborListFormat.COO``)
            if spec.consolidation == Consolidation.DIRECT_MASKED or (spec.refresh_per_layer and not self._policy_folds()):
                if coo:
                    _keep_edges(padded, padded.neighbor_list[:, 0] < sharded.n_owned)
                else:
                    padded.num_neighbors[sharded.n_owned:] = 0  # ghost atoms send, they do not receive
            elif spec.refresh_per_layer and halo.n_ghost > 0:
                if coo:
                    _keep_edges(padded, padded.neighbor_list[:, 1] < sharded.n_owned)
                else:
                    _keep_owned_senders(padded, sharded.n_owned)  # fold policy: every edge lives on its sender's owner
        if spec.refresh_per_layer and halo.n_ghost > 0:
            from nvalchemi_toolkit_b200.distributed.dispatch import HaloDispatchMode

            with HaloDispatchMode(halo, sharded.n_owned, self._policy(), group=sharded.group,
                                  global_ids=sharded.global_ids) as mode:
                out = self.model(padded, **kwargs)
            self.last_dispatch_stats = dict(mode.stats)
        else:
            out = self.model(padded, **kwargs)
        return consolidate_outputs(dict(out), sharded, spec, halo)

    def _policy(self) -> Any:
        from nvalchemi_toolkit_b200.distributed.storage_policy import RefreshOnlyHaloPolicy, policy_from_dict

        d = self.spec.storage_policy
        return policy_from_dict(d) if d is not None else RefreshOnlyHaloPolicy()

    def _policy_folds(self) -> bool:
        return getattr(self._policy(), "scatter_mode", "local") != "local"


class DistributedPipelineModel(nn.Module):
    """Domain-decomposed ``PipelineModelWrapper``: every member of a direct group is evaluated with a halo of its own
    depth over the one owned partition, and the consolidated member outputs are summed like the pipeline does.
    Reference: ``nvalchemi/distributed/distributed_pipeline.py:65-448``.

    A group that differentiates its summed energy (``use_autograd``) or passes outputs along wires (predicted charges
    into an electrostatics member) is decomposed AS ONE MODEL: the whole group runs on owned + ghost atoms with a ghost
    layer as deep as the members' receptive fields chained together (a wired quantity on a ghost atom must itself be
    exact before the next member reads it), every member sums its energy with the per-atom ``energy_weights`` of the
    padded batch (1 owned, 0 ghost: MACE, DFT-D3, Ewald / PME and the pair potentials do), the group's autograd pass
    yields gradients on all local rows and the ghost rows' share returns to the owners by the reverse halo."""

    def __init__(self, pipeline: Any, config: DomainConfig, group: Any = None, max_neighbors: int | None = None) -> None:
        super().__init__()
        from nvalchemi_toolkit_b200.models._utils import sum_outputs
        from nvalchemi_toolkit_b200.models.pipeline import PipelineModelWrapper

        self.pipeline, self.config, self._sum = pipeline, config, sum_outputs
        self.model_config = pipeline.model_config
        self.members = nn.ModuleList()
        active = set(pipeline.model_config.active_outputs)

        def member_config(cutoff: float) -> DomainConfig:
            d = {k: v for k, v in config.model_dump().items() if k != "ghost_width"}
            d["cutoff"] = cutoff
            return DomainConfig(**d)

        for g in pipeline.groups:
            if g.use_autograd or any(s.wire for s in g.steps):
                depth = 0.0
                for s in g.steps:
                    nc = s.model.model_config.neighbor_config
                    spec = s.model.distribution_spec(config.strategy)
                    passes = max(1, spec.message_passes) if spec is not None else 1
                    depth += passes * ((nc.cutoff if nc is not None else 0.0) + config.skin)
                sub = PipelineModelWrapper([g], additive_keys=set(pipeline.additive_keys))
                sub.model_config.active_outputs = set(active) & set(sub.model_config.outputs)
                group_spec = MLIPSpec("pipeline_group", message_passes=1, consolidation=Consolidation.WEIGHTED_ENERGY)
                self.members.append(DistributedModel(sub, member_config(depth - config.skin), spec=group_spec, group=group,
                                                     max_neighbors=max_neighbors, own_halo=True))
                continue
            for s in g.steps:
                nc = s.model.model_config.neighbor_config
                self.members.append(DistributedModel(s.model, member_config(nc.cutoff if nc is not None else config.cutoff),
                                                     group=group, max_neighbors=max_neighbors, own_halo=True))
        deepest = max(m.spec.ghost_width(m.config.cutoff, m.config.skin) for m in self.members)
        self.spec = MLIPSpec("pipeline", message_passes=1, consolidation=Consolidation.WEIGHTED_ENERGY)
        self.required_ghost_width = deepest

    def forward(self, sharded: ShardedBatch, **kwargs: Any) -> dict:
        outs = [m(sharded, **kwargs) for m in self.members]
        return self._sum(*outs, additive_keys=frozenset(self.pipeline.additive_keys))
