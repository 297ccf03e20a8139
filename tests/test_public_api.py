# SPDX-License-Identifier: Apache-2.0
"""The public surface: every name a user of the reference package imports from its sub-packages resolves here at the
same place, plus the small pieces that exist for that purpose (specs, adapters of module-level helpers, output kinds)."""
import importlib
import json

import pytest
import torch

REFERENCE_NAMES = {
    "dynamics": """BaseDynamics ConvergenceHook DataSink DemoDynamics DistributedPipeline DynamicsStage FIRE FIRE2
        FIRE2VariableCell FIREVariableCell FusedStage GPUBuffer Hook HostMemory NPH NPT NVE NVTLangevin NVTNoseHoover
        SizeAwareSampler ZarrData hooks initialize_velocities integrators optimizers""",
    "models": """AIMNet2Wrapper DFTD3ModelWrapper DemoModelWrapper EwaldModelWrapper LennardJonesModelWrapper MACEWrapper
        PMEModelWrapper PipelineGroup PipelineModelWrapper PipelineStep UMAWrapper""",
    "hooks": """BaseRichLayout BiasedPotentialHook CheckpointableHook DynamicsContext DynamicsRichLayout Hook HookContext
        HookRegistryMixin NeighborListHook Reporter ReporterMessage ReportingErrorPolicy ReportingOrchestrator ReportingState
        RichLayout RichReporter ScalarCallback ScalarSnapshot StageTimingHook TensorBoardReporter TensorBoardWriter
        TorchProfilerHook TrainContext TrainingRichLayout WrapPeriodicHook collect_scalars extract_dynamics_scalars
        extract_loss_scalars extract_optimizer_lr_scalars extract_scalars""",
    "data": """AtomicData AtomicDataZarrReader AtomicDataZarrWriter Batch BatchDatasetProtocol Compose DataLoader Dataset
        InMemoryDataset Reader transforms""",
    "training": """BaseLossFunction BaseSpec BatchValidationCallback CheckpointHook CheckpointManifest CheckpointValidator
        ComposedLossFunction ComposedLossOutput ConstantWeight CosineWeight DDPHook DTypePolicy EMAHook EnergyHuberLoss
        EnergyMAELoss EnergyMSELoss FineTuningStrategy ForceHuberLoss ForceL2NormLoss ForceMSELoss LinearWeight
        LossTargetAssemblyProtocol LossWeightSchedule OptimizerConfig PiecewiseWeight ReductionContext StressHuberLoss
        StressMSELoss TrainingStage TrainingStrategy ValidationConfig ValidationLoop assemble_loss_targets
        configure_dataloader configure_parallelism create_model_spec create_model_spec_from_json default_training_fn
        freeze_unconfigured_models load_checkpoint loss_component_to_spec move_to_devices register_type_serializer
        save_checkpoint setup_optimizers step_lr_schedulers step_optimizers zero_gradients""",
    "distributed": """AdapterRegistry AdapterStatus COOPadder CompilePolicy DenseBatchPadder DensePadder DistributedManager
        DistributedModel DistributedPipelineModel DistributionSpec DomainConfig DomainParallel ForceStrategy FunctionAdapter
        GraphPadder HookScope JitAdapter MLIPSpec MethodAdapter OpAdapter OutputKind OutputSpec ParticleHaloConfig
        PythonAdapter Reduce Scope ShardedBatch SpatialPartitioner autograd_target collective_device current_dd_context
        distributed_method localize neighbor_refresh_adapters refresh_neighbors reshard_by_destination resolve_cap
        resolve_global_rank resolve_world_size scatter_to_owners system_sum to_local trace_and_validate""",
}


@pytest.mark.parametrize("package", sorted(REFERENCE_NAMES))
def test_reference_names_resolve_from_the_same_subpackage(package):
    mod = importlib.import_module(f"nvalchemi_toolkit_b200.{package}")
    missing = [n for n in REFERENCE_NAMES[package].split() if not hasattr(mod, n)]
    assert missing == []
    for n in getattr(mod, "__all__", []):
        assert getattr(mod, n) is not None, n


def test_specs_round_trip_through_json_and_build_nested_objects():
    from nvalchemi_toolkit_b200.training import (BaseSpec, create_model_spec, create_model_spec_from_json,
                                                 register_type_serializer)

    spec = create_model_spec(torch.nn.Linear, in_features=3, out_features=2, bias=False, dtype=torch.float64)
    again = create_model_spec_from_json(spec.model_dump_json())
    layer = again.build()
    assert isinstance(layer, torch.nn.Linear) and layer.weight.dtype == torch.float64 and layer.bias is None
    assert again.in_features == 3 and again.cls_path.endswith("Linear") and again.timestamp == spec.timestamp
    assert again.build(out_features=5).weight.shape == (5, 3)          # overrides at build time
    with pytest.raises(TypeError, match="does not accept"):
        create_model_spec(torch.nn.Linear, in_features=3, out_feature=2)
    with pytest.raises(TypeError, match="needs"):
        create_model_spec(torch.nn.Linear, in_features=3)
    with pytest.raises(ValueError):
        BaseSpec(cls_path="no_such_module.Thing")
    # nested specs (here inside a tuple), tensors and classes survive the JSON form and are built inside out
    inner = create_model_spec(torch.nn.Linear, in_features=2, out_features=2)
    outer = create_model_spec(_Holder, parts=(inner, inner), scale=torch.tensor([1.5, 2.5]), act=torch.nn.SiLU)
    wire = json.loads(json.dumps(outer.model_dump(mode="json")))
    built = create_model_spec_from_json(wire).build()
    assert isinstance(built.parts, tuple) and all(isinstance(p, torch.nn.Linear) for p in built.parts)
    assert torch.equal(built.scale, torch.tensor([1.5, 2.5])) and built.act is torch.nn.SiLU
    assert isinstance(create_model_spec_from_json(wire).parts[0], BaseSpec)    # attribute access decodes without building
    # a type the spec layer does not know is taught once
    register_type_serializer(_Units, lambda u: {"name": u.name}, lambda d: _Units(d["name"]))
    spec_u = create_model_spec(_Holder, parts=(), scale=None, act=_Units("eV"))
    assert create_model_spec_from_json(spec_u.model_dump_json()).build().act.name == "eV"


class _Holder:
    def __init__(self, parts, scale, act):
        self.parts, self.scale, self.act = parts, scale, act


class _Units:
    def __init__(self, name):
        self.name = name


def test_python_and_jit_adapters_swap_helpers_and_report_status():
    import math

    from nvalchemi_toolkit_b200.distributed import AdapterRegistry, AdapterStatus, JitAdapter, PythonAdapter
    from nvalchemi_toolkit_b200.distributed import distributed_method

    @distributed_method
    def guarded(original, mode, x):
        return -1.0                                       # only inside a distributed forward

    reg = AdapterRegistry([PythonAdapter("math", "sqrt", lambda x: 42.0), PythonAdapter("math", "floor", guarded(math.floor))])
    assert [s.state for s in reg.list_active()] == ["pending", "pending"]
    with reg:
        assert math.sqrt(4.0) == 42.0 and math.floor(2.5) == 2     # no dispatch mode active: the original runs
        st = reg.list_active()
        assert all(isinstance(s, AdapterStatus) and s.state == "installed" and s.kind == "python" for s in st)
        assert st[0].target == "math.sqrt" and st[0].install_site.startswith("test_public_api.py:")
    assert math.sqrt(4.0) == 2.0 and [s.state for s in reg.list_active()] == ["restored", "restored"]
    # a failing install rolls back what was already swapped and is listed as failed
    bad = AdapterRegistry([PythonAdapter("math", "sqrt", lambda x: 0.0), PythonAdapter("math", "no_such_function", abs)])
    with pytest.raises(AttributeError):
        bad.install()
    assert math.sqrt(9.0) == 3.0
    assert [s.state for s in bad.list_active()] == ["restored", "failed"] and "AttributeError" in bad.list_active()[1].error
    with pytest.raises(RuntimeError, match="no replacement"):
        AdapterRegistry([PythonAdapter("math", "sqrt")]).install()
    with pytest.raises(ValueError, match="needs a replacement"):
        JitAdapter("math", "sqrt", mode="eager")
    marshal = JitAdapter("math", "sqrt", mode="marshal", node_inputs=(0,))
    with AdapterRegistry([marshal]):
        assert math.sqrt(16.0) == 4.0 and hasattr(math.sqrt, "__wrapped_by_adapter__")   # opaque-operator treatment
    assert not hasattr(math.sqrt, "__wrapped_by_adapter__")


def test_output_declarations_lower_onto_the_spec_lists():
    from nvalchemi_toolkit_b200.distributed import MLIPSpec, OutputKind, OutputSpec, Reduce

    spec = MLIPSpec("m").with_outputs({
        "forces": OutputSpec(OutputKind.PER_NODE), "charges": OutputSpec(OutputKind.PER_NODE, Reduce.OWNED_ONLY),
        "energy": OutputSpec(OutputKind.PER_GRAPH, Reduce.ALL_REDUCE), "stress": OutputSpec(OutputKind.PER_GRAPH, Reduce.ALL_REDUCE),
        "cell": OutputSpec(OutputKind.PER_GRAPH, Reduce.OWNED_ONLY), "version": OutputSpec(OutputKind.GLOBAL)})
    assert spec.node_outputs == ("forces", "charges") and spec.extensive_outputs == ("energy", "stress")
    assert MLIPSpec.from_dict(json.loads(json.dumps(spec.to_dict()))).extensive_outputs == ("energy", "stress")
    with pytest.raises(ValueError, match="per-node output cannot be all-reduced"):
        MLIPSpec("m").with_outputs({"forces": OutputSpec(OutputKind.PER_NODE, Reduce.ALL_REDUCE)})
    with pytest.raises(ValueError, match="GLOBAL"):
        MLIPSpec("m").with_outputs({"v": OutputSpec(OutputKind.GLOBAL, Reduce.ALL_REDUCE)})
    with pytest.raises(TypeError):
        MLIPSpec("m").with_outputs({"forces": "per_node"})


def test_small_distributed_helpers_and_manager_without_a_process_group(monkeypatch):
    from nvalchemi_toolkit_b200.distributed import (DistributedManager, ShardTensor, autograd_target, localize,
                                                    neighbor_refresh_adapters)

    x = torch.ones(3, requires_grad=True)
    assert autograd_target(x) is x and localize({"a": x, "n": 3}) == {"a": x, "n": 3}

    class Block(torch.nn.Module):
        def forward(self, h):
            return h

    class Sub(Block):
        pass

    adapters = neighbor_refresh_adapters(torch.nn.ModuleList([Block(), Sub(), Block()]), output=0)
    assert len(adapters) == 1 and adapters[0].owner is Block and adapters[0].node_outputs == (0,)   # one per class defining forward
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    DistributedManager.cleanup()
    assert not DistributedManager.is_initialized()
    m = DistributedManager.initialize()
    assert m is DistributedManager() and DistributedManager.is_initialized()
    assert (m.rank, m.world_size, m.local_rank, m.distributed) == (0, 1, 0, False) and m.device.type in ("cpu", "cuda")
    DistributedManager.cleanup()
    assert not DistributedManager.is_initialized()
    del ShardTensor


SECOND_LEVEL = {
    "dynamics.hooks": """AlignCellHook ConvergedSnapshotHook EnergyDriftMonitorHook FreezeAtomsHook LoggingHook MaxForceClampHook
        NaNDetectorHook SnapshotHook StageTimingHook TorchProfilerHook""",
    "training.hooks": """CheckpointHook DDPHook EMAHook MixedPrecisionHook ModulePatchHook TorchProfilerHook
        TrainableParameterHook TrainingUpdateHook TrainingUpdateOrchestrator""",
    "training.losses": """BaseLossFunction ComposedLossFunction ComposedLossOutput DTypePolicy LossTargetAssemblyProtocol
        LossWeightSchedule ReductionContext assemble_loss_targets assert_same_shape frobenius_mse loss_component_to_spec
        per_graph_mean per_graph_sum""",
    "dynamics.integrators": "NPH NPT NVE NVTLangevin NVTNoseHoover",
    "dynamics.optimizers": "FIRE FIRE2 FIRE2VariableCell FIREVariableCell",
    "hooks.reporting": """BaseRichLayout DEFAULT_REPORT_STAGES DynamicsRichLayout Reporter ReportingOrchestrator RichReporter
        TensorBoardWriter TrainingRichLayout extract_scalars""",
    "data.datapipes": """AtomicDataZarrReader AtomicDataZarrWriter BatchDatasetProtocol DataLoader Dataset
        DistributedSamplerProtocol InMemoryDataset MultiDataset MultiDatasetBatchSampler MultiDatasetSampler Reader
        ZarrArrayConfig ZarrWriteConfig""",
}


@pytest.mark.parametrize("package", sorted(SECOND_LEVEL))
def test_second_level_reference_names_resolve(package):
    mod = importlib.import_module(f"nvalchemi_toolkit_b200.{package}")
    assert [n for n in SECOND_LEVEL[package].split() if not hasattr(mod, n)] == []


def test_update_hooks_compose_in_priority_order_and_shape_checks():
    from nvalchemi_toolkit_b200.training.hooks import (GradientAccumulationHook, GradientClipHook, LossSpikeSkipHook,
                                                       MixedPrecisionHook, TrainingUpdateHook, TrainingUpdateOrchestrator)
    from nvalchemi_toolkit_b200.training.losses import assert_same_shape

    chain = LossSpikeSkipHook() + GradientClipHook(1.0) + MixedPrecisionHook() + GradientAccumulationHook(4)
    assert isinstance(chain, TrainingUpdateOrchestrator)
    assert [type(h).__name__ for h in chain.hooks] == ["GradientAccumulationHook", "MixedPrecisionHook", "GradientClipHook",
                                                      "LossSpikeSkipHook"]
    assert all(isinstance(h, TrainingUpdateHook) for h in chain.hooks)
    a, b = torch.zeros(4, 1), torch.zeros(4, 3)
    assert_same_shape(a, b, name="x")                                   # broadcast-compatible passes by default ...
    with pytest.raises(ValueError, match="differ"):
        assert_same_shape(a, b, name="x", strict=True)                  # ... and is what strict is for
    with pytest.raises(ValueError, match="do not broadcast"):
        assert_same_shape(torch.zeros(4, 2), b, name="x")
    with pytest.raises(ValueError, match="float64"):
        assert_same_shape(a, b.double(), name="x", prediction_key="p", target_key="t")
