# SPDX-License-Identifier: Apache-2.0
"""Domain decomposition: one large system over many GPUs.

Two layers: a generic, backend-agnostic API (``DomainParallel`` / ``ShardedBatch`` / ``DistributedModel`` / ``MLIPSpec``;
any model wrapper, NCCL or gloo) and the single-node peer-memory engine for the native MACE path
(``slab_md.SlabDomainMD``: ghost features read from the owner GPU inside the convolution kernels).
"""
from nvalchemi_toolkit_b200.distributed.config import DomainConfig, HookScope, StrategyKind
from nvalchemi_toolkit_b200.distributed.partitioner import IndexPartitioner, SpatialPartitioner, factor_grid
from nvalchemi_toolkit_b200.distributed.spec import (Consolidation, MLIPSpec, SPEC_AIMNET2_GRAPH_PARTITION,
                                                     SPEC_AIMNET2_HALO, SPEC_DEMO, SPEC_DFTD3_HALO,
                                                     SPEC_EWALD_REAL_HALO, SPEC_LJ_HALO, SPEC_MACE_CUEQ_HALO,
                                                     SPEC_MACE_GRAPH_PARTITION, SPEC_MACE_HALO, SPEC_PAIR_HALO, get_spec,
                                                     register_spec)
from nvalchemi_toolkit_b200.distributed.halo import HaloExchange, all_gather_rows, all_to_all_rows
from nvalchemi_toolkit_b200.distributed.sharded_batch import ShardedBatch
from nvalchemi_toolkit_b200.distributed.distributed_model import DistributedModel, DistributedPipelineModel, consolidate_outputs
from nvalchemi_toolkit_b200.distributed.domain_parallel import DomainParallel, DynamicsCoordinator
from nvalchemi_toolkit_b200.distributed.ops import ShardTensor, halo_forward, halo_scatter_correct
from nvalchemi_toolkit_b200.distributed import helpers
from nvalchemi_toolkit_b200.distributed.pipeline2d import DomainPipeline

__all__ = ["DomainConfig", "HookScope", "StrategyKind", "SpatialPartitioner", "IndexPartitioner", "factor_grid", "MLIPSpec",
           "Consolidation", "get_spec", "register_spec", "HaloExchange", "ShardedBatch", "DistributedModel", "DistributedPipelineModel",
           "consolidate_outputs", "DomainParallel", "DomainPipeline", "DynamicsCoordinator", "ShardTensor", "halo_forward",
           "halo_scatter_correct", "helpers", "all_gather_rows", "all_to_all_rows", "SPEC_LJ_HALO", "SPEC_PAIR_HALO",
           "SPEC_DFTD3_HALO", "SPEC_EWALD_REAL_HALO", "SPEC_MACE_HALO", "SPEC_MACE_CUEQ_HALO", "SPEC_AIMNET2_HALO",
           "SPEC_DEMO", "SPEC_MACE_GRAPH_PARTITION", "SPEC_AIMNET2_GRAPH_PARTITION"]
