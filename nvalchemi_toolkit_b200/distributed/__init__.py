# SPDX-License-Identifier: Apache-2.0
"""Domain decomposition: one large system over many GPUs.

One API (``DomainParallel`` / ``ShardedBatch`` / ``DistributedModel`` / ``MLIPSpec``) with two transports behind it:
``torch.distributed`` collectives for any model wrapper on NCCL or gloo, and, for the native MACE on the GPUs of one
node, the peer-memory engine (``peer_halo.PeerHaloEngine``: ghost rows pulled from and returned to their owners by
NVLink kernels over symmetric buffers; selected automatically, ``DomainConfig(peer_memory=False)`` switches it off).

The generic layer evaluates a model either on a ghost layer as deep as its receptive field (nothing inside the model is
touched) or, with ``MLIPSpec(refresh_per_layer=True)``, on a ghost layer one cutoff deep whose feature rows are
refreshed from their owners before every message-passing layer (``dispatch.HaloDispatchMode`` intercepts the model's
dim-0 gathers and scatters; ``storage_policy`` says what a gather / scatter has to do; ``dispatch.OpAdapter`` gives
opaque fused operators the same treatment).  ``graph_padder`` keeps per-rank shapes fixed for CUDA-graph replay.
"""
from nvalchemi_toolkit_b200.distributed.config import DomainConfig, HookScope, StrategyKind
from nvalchemi_toolkit_b200.distributed.partitioner import IndexPartitioner, SpatialPartitioner, factor_grid
from nvalchemi_toolkit_b200.distributed.spec import (CompilePolicy, Consolidation, ForceStrategy, MLIPSpec, SPEC_AIMNET2_GRAPH_PARTITION,
                                                     SPEC_AIMNET2_HALO, SPEC_DEMO, SPEC_DFTD3_HALO,
                                                     SPEC_EWALD_REAL_HALO, SPEC_LJ_HALO, SPEC_MACE_CUEQ_HALO,
                                                     SPEC_MACE_GRAPH_PARTITION, SPEC_MACE_HALO, SPEC_PAIR_HALO, get_spec,
                                                     register_spec)
from nvalchemi_toolkit_b200.distributed.halo import HaloExchange, all_gather_rows, all_to_all_rows
from nvalchemi_toolkit_b200.distributed.sharded_batch import ShardedBatch
from nvalchemi_toolkit_b200.distributed.distributed_model import DistributedModel, DistributedPipelineModel, consolidate_outputs
from nvalchemi_toolkit_b200.distributed.domain_parallel import DomainParallel, DynamicsCoordinator
from nvalchemi_toolkit_b200.distributed.ops import (ShardTensor, distributed_all_reduce, gather_replicate, halo_forward,
                                                    halo_scatter_correct, per_system_reduce)
from nvalchemi_toolkit_b200.distributed.storage_policy import (GraphParallelPolicy, HaloStoragePolicy, PlainShard,
                                                               RefreshOnlyHaloPolicy, StoragePolicy, policy_from_dict,
                                                               policy_to_dict)
from nvalchemi_toolkit_b200.distributed.dispatch import (AdapterRegistry, AdapterStatus, FunctionAdapter, HaloDispatchMode,
                                                         JitAdapter, MethodAdapter, ModuleForwardAdapter, OpAdapter,
                                                         PythonAdapter, current_dispatch)
from nvalchemi_toolkit_b200.distributed.output_kinds import OutputKind, OutputSpec, Reduce
from nvalchemi_toolkit_b200.distributed.context import current_dd_context, reshard_by_destination
from nvalchemi_toolkit_b200.distributed._runtime import (DistributedManager, collective_device, resolve_global_rank,
                                                         resolve_world_size)
from nvalchemi_toolkit_b200.distributed.helpers import (autograd_target, distributed_method, localize,
                                                        neighbor_refresh_adapters, refresh_neighbors, scatter_to_owners,
                                                        system_sum, to_local)
from nvalchemi_toolkit_b200.distributed.graph_padder import (COOPadder, DenseBatchPadder, DensePadder, GraphPadder,
                                                             cap_agreement_group, resolve_cap)
from nvalchemi_toolkit_b200.distributed import helpers
from nvalchemi_toolkit_b200.distributed.pipeline2d import DomainPipeline
from nvalchemi_toolkit_b200.distributed.static_halo import (StaticHalo, StaticHaloRouting, halo_exchange_fixed, halo_forward_static,
                                                            halo_scatter_correct_static)
from nvalchemi_toolkit_b200.distributed.peer_halo import PeerFailure, PeerHaloEngine, build_pull_tables, peer_memory_available

__all__ = ["StaticHalo", "StaticHaloRouting", "halo_exchange_fixed", "halo_forward_static", "halo_scatter_correct_static", "CompilePolicy", "ForceStrategy", "DomainConfig", "HookScope", "StrategyKind", "SpatialPartitioner", "IndexPartitioner", "factor_grid", "MLIPSpec",
           "Consolidation", "get_spec", "register_spec", "HaloExchange", "ShardedBatch", "DistributedModel", "DistributedPipelineModel",
           "consolidate_outputs", "DomainParallel", "DomainPipeline", "DynamicsCoordinator", "ShardTensor", "halo_forward",
           "halo_scatter_correct", "helpers", "all_gather_rows", "all_to_all_rows", "SPEC_LJ_HALO", "SPEC_PAIR_HALO",
           "SPEC_DFTD3_HALO", "SPEC_EWALD_REAL_HALO", "SPEC_MACE_HALO", "SPEC_MACE_CUEQ_HALO", "SPEC_AIMNET2_HALO",
           "SPEC_DEMO", "SPEC_MACE_GRAPH_PARTITION", "SPEC_AIMNET2_GRAPH_PARTITION", "distributed_all_reduce",
           "gather_replicate", "per_system_reduce", "StoragePolicy", "PlainShard", "HaloStoragePolicy",
           "RefreshOnlyHaloPolicy", "GraphParallelPolicy", "policy_to_dict", "policy_from_dict", "HaloDispatchMode",
           "current_dispatch", "OpAdapter", "FunctionAdapter", "MethodAdapter", "ModuleForwardAdapter", "AdapterRegistry",
           "GraphPadder", "COOPadder", "DensePadder", "DenseBatchPadder", "resolve_cap", "cap_agreement_group",
           "PeerHaloEngine", "PeerFailure", "build_pull_tables", "peer_memory_available", "AdapterStatus", "JitAdapter",
           "PythonAdapter", "OutputKind", "OutputSpec", "Reduce", "current_dd_context", "reshard_by_destination",
           "collective_device", "resolve_global_rank", "resolve_world_size", "autograd_target", "distributed_method",
           "localize", "neighbor_refresh_adapters", "refresh_neighbors", "scatter_to_owners", "system_sum", "to_local",
           "trace_and_validate", "infer_spec", "ParticleHaloConfig", "DistributionSpec", "Scope", "DistributedManager"]

#: reference names for objects that exist here under another name
ParticleHaloConfig = DomainConfig   # ghost width, skin and rank grid of the particle halo live on the domain config
DistributionSpec = MLIPSpec         # storage policy and adapters are fields of the one spec class
Scope = HookScope


def __getattr__(name: str):  # these spawn processes / trace models: loaded on first use
    if name == "trace_and_validate":
        from nvalchemi_toolkit_b200.distributed.validate import trace_and_validate

        return trace_and_validate
    if name == "infer_spec":
        from nvalchemi_toolkit_b200.distributed.infer_spec import infer_spec

        return infer_spec
    raise AttributeError(name)
