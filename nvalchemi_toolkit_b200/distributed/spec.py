# SPDX-License-Identifier: Apache-2.0
"""``MLIPSpec``: what the domain-decomposition layer needs to know about a model.

The reference (``nvalchemi/distributed/spec.py:50-410``) describes, per model, which tensors are node/edge/system
sharded and which dispatch interceptions (halo refresh after scatter, halo-receiver edge masks, MACE reshape and
autograd workarounds) keep a traced forward correct.  Nothing is traced or intercepted here; the distributed forward is
an explicit ghost-atom evaluation, so the spec reduces to three facts:

* ``message_passes``: how many neighbour hops influence an atom's energy; ghosts are kept within
  ``message_passes * (cutoff + skin)`` of the sub-domain, which makes every owned atom's energy exact;
* ``consolidation``: how per-rank results combine.  ``DIRECT_MASKED`` suits kernels that produce forces directly from a
  full neighbour list: ghost rows get an empty neighbour list, so every owned row is complete and nothing is counted
  twice.  ``WEIGHTED_ENERGY`` suits differentiated models: the model sums node energies with per-atom weights (1 owned,
  0 ghost), differentiates that sum with respect to all local positions, and the ghost rows' gradients are added to
  their owners (reverse halo);
* which outputs are per-node and which are extensive per-system sums.

``refresh_per_layer=True`` selects the other design (the reference's default): a ghost layer one cutoff deep whose
feature rows are refreshed from the owners before each message-passing layer, by intercepting the model's gathers and
scatters (``distributed/dispatch.py``); deeper models then exchange features instead of recomputing a wider halo.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from nvalchemi_toolkit_b200.distributed.config import StrategyKind


class Consolidation(str, Enum):
    DIRECT_MASKED = "direct_masked"
    WEIGHTED_ENERGY = "weighted_energy"
    REPLICATED = "replicated"       # the model needs no neighbours (per-atom terms only)


class ForceStrategy(str, Enum):
    """Who produces the forces of a distributed forward (reference ``distributed/spec.py:211-238``).

    ``MODEL_INTERNAL``: the model returns forces itself (kernels with analytic forces); owned rows are complete because
    ghost rows carry empty neighbour lists.  ``FRAMEWORK_FROM_NODE_ENERGY``: the model returns per-node energies, the
    framework sums the owned ones, differentiates and returns ghost gradients to their owners.
    ``FRAMEWORK_FROM_GLOBAL_ENERGY``: the model itself consolidates the per-system energy (it consumes the per-atom
    ``energy_weights`` of the padded batch: 1 owned, 0 ghost) and the framework differentiates that energy as it is."""

    MODEL_INTERNAL = "model_internal"
    FRAMEWORK_FROM_NODE_ENERGY = "framework_from_node_energy"
    FRAMEWORK_FROM_GLOBAL_ENERGY = "framework_from_global_energy"


@dataclass(frozen=True)
class CompilePolicy:
    """Fixed-shape contract of a model under domain decomposition (reference ``distributed/spec.py:241-292``).

    The reference uses it to keep a ``torch.compile``-d trajectory compiled; here nothing is traced, and the same
    contract serves CUDA-graph replay and the peer-memory engine, whose buffers are sized once: ``static_shapes`` asks
    for per-rank capacities agreed over the ranks (``graph_padder.resolve_cap``) instead of exact sizes, ``graph_padder``
    names the padder (``None``: the COO edge-list padder), ``force_strategy`` declares who produces the forces and
    ``stress_via_strain`` lets the framework obtain the virial by straining positions and cell (only sound for models
    whose whole cell dependence is differentiable)."""

    static_shapes: bool = True
    graph_padder: object | None = None
    force_strategy: ForceStrategy = ForceStrategy.MODEL_INTERNAL
    stress_via_strain: bool = False

    @property
    def forces_via_autograd(self) -> bool:
        return self.force_strategy is not ForceStrategy.MODEL_INTERNAL

    @property
    def consolidate_node_energy(self) -> bool:
        return self.force_strategy is ForceStrategy.FRAMEWORK_FROM_NODE_ENERGY

    @property
    def energy_output(self) -> str:
        return "atomic_energies" if self.force_strategy is ForceStrategy.FRAMEWORK_FROM_NODE_ENERGY else "energy"


@dataclass(frozen=True)
class MLIPSpec:
    name: str
    strategy: StrategyKind = StrategyKind.HALO
    message_passes: int = 1
    consolidation: Consolidation = Consolidation.WEIGHTED_ENERGY
    node_energy_key: str = "atomic_energies"
    requires_full_list: bool = True
    node_outputs: tuple[str, ...] = ("forces", "atomic_energies", "charges", "node_embeddings")
    extensive_outputs: tuple[str, ...] = ("energy", "virial", "stress")
    needs_total_charge: bool = False
    notes: str = ""
    extra: dict = field(default_factory=dict)
    #: ghost layer one cutoff deep; ghost rows of node features are refreshed from their owners before every gather
    #: (``distributed/dispatch.py``) instead of being recomputed from a ``message_passes``-deep ghost layer
    refresh_per_layer: bool = False
    #: serialised storage policy of node features under ``refresh_per_layer`` (``None``: refresh only)
    storage_policy: dict | None = None

    #: fixed-shape / force-production contract (``None``: derived from ``consolidation``)
    compile: CompilePolicy | None = field(default=None, compare=False, hash=False)

    @property
    def force_strategy(self) -> ForceStrategy:
        """The declared strategy, or the one the consolidation mode implies."""
        if self.compile is not None:
            return self.compile.force_strategy
        if self.consolidation == Consolidation.WEIGHTED_ENERGY:
            return ForceStrategy.FRAMEWORK_FROM_NODE_ENERGY
        return ForceStrategy.MODEL_INTERNAL

    def ghost_width(self, cutoff: float, skin: float = 0.0) -> float:
        if self.refresh_per_layer:
            return cutoff + skin
        return max(1, self.message_passes) * (cutoff + skin)

    def with_outputs(self, outputs: "dict[str, object]") -> "MLIPSpec":
        """The spec with its output lists taken from per-output declarations (``{"stress": OutputSpec(OutputKind.PER_GRAPH,
        Reduce.ALL_REDUCE), ...}``, see ``distributed/output_kinds.py``)."""
        from nvalchemi_toolkit_b200.distributed.output_kinds import lower_outputs

        node, extensive = lower_outputs(outputs)
        return self.with_(node_outputs=node, extensive_outputs=extensive)

    def with_(self, **changes: object) -> "MLIPSpec":
        from dataclasses import replace

        return replace(self, **changes)

    def to_dict(self) -> dict:
        from dataclasses import asdict

        d = asdict(self)
        d["compile"] = None if self.compile is None else {
            "static_shapes": self.compile.static_shapes, "force_strategy": self.compile.force_strategy.value,
            "stress_via_strain": self.compile.stress_via_strain}  # the padder object is not serialised
        d["strategy"], d["consolidation"] = self.strategy.value, self.consolidation.value
        d["node_outputs"], d["extensive_outputs"] = list(self.node_outputs), list(self.extensive_outputs)
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "MLIPSpec":
        d = dict(d)
        d["strategy"], d["consolidation"] = StrategyKind(d["strategy"]), Consolidation(d["consolidation"])
        d["node_outputs"], d["extensive_outputs"] = tuple(d["node_outputs"]), tuple(d["extensive_outputs"])
        c = d.pop("compile", None)
        if c is not None:
            d["compile"] = CompilePolicy(static_shapes=bool(c.get("static_shapes", True)),
                                         force_strategy=ForceStrategy(c.get("force_strategy", "model_internal")),
                                         stress_via_strain=bool(c.get("stress_via_strain", False)))
        return cls(**d)

    def save(self, path: str) -> None:
        import json

        with open(path, "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2)

    @classmethod
    def load(cls, path: str) -> "MLIPSpec":
        import json

        with open(path, encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))


SPEC_LJ_HALO = MLIPSpec("lennard_jones", message_passes=1, consolidation=Consolidation.DIRECT_MASKED)
SPEC_PAIR_HALO = MLIPSpec("pair_potential", message_passes=1, consolidation=Consolidation.DIRECT_MASKED)
SPEC_DFTD3_HALO = MLIPSpec("dftd3", message_passes=2, consolidation=Consolidation.WEIGHTED_ENERGY,
                           notes="coordination numbers need one hop, the dispersion sum a second")
SPEC_EWALD_REAL_HALO = MLIPSpec("ewald_real_space", message_passes=1, consolidation=Consolidation.DIRECT_MASKED,
                                needs_total_charge=True,
                                notes="reciprocal-space part is evaluated on replicated structure factors")
SPEC_MACE_HALO = MLIPSpec("mace", message_passes=2, consolidation=Consolidation.WEIGHTED_ENERGY)
SPEC_MACE_CUEQ_HALO = SPEC_MACE_HALO.with_(name="mace_cueq")
SPEC_AIMNET2_HALO = MLIPSpec("aimnet2", message_passes=3, consolidation=Consolidation.WEIGHTED_ENERGY,
                             needs_total_charge=True)
SPEC_DEMO = MLIPSpec("demo", message_passes=0, consolidation=Consolidation.REPLICATED)
SPEC_MACE_GRAPH_PARTITION = MLIPSpec("mace_graph_partition", strategy=StrategyKind.GRAPH_PARTITION, message_passes=2,
                                     consolidation=Consolidation.WEIGHTED_ENERGY)
SPEC_AIMNET2_GRAPH_PARTITION = MLIPSpec("aimnet2_graph_partition", strategy=StrategyKind.GRAPH_PARTITION,
                                        message_passes=3, consolidation=Consolidation.WEIGHTED_ENERGY,
                                        needs_total_charge=True)

_REGISTRY = {s.name: s for s in (SPEC_LJ_HALO, SPEC_PAIR_HALO, SPEC_DFTD3_HALO, SPEC_EWALD_REAL_HALO, SPEC_MACE_HALO,
                                 SPEC_MACE_CUEQ_HALO, SPEC_AIMNET2_HALO, SPEC_DEMO, SPEC_MACE_GRAPH_PARTITION,
                                 SPEC_AIMNET2_GRAPH_PARTITION)}


def get_spec(name: str) -> MLIPSpec:
    return _REGISTRY[name]


def register_spec(spec: MLIPSpec) -> None:
    _REGISTRY[spec.name] = spec
