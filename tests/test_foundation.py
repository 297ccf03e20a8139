# SPDX-License-Identifier: Apache-2.0
"""Foundation modules: optional dependencies, serialisation, typing enums, element tables, unit conversion, autograd
helpers shared by the model wrappers."""
import json
import math

import pytest
import torch

from nvalchemi_toolkit_b200 import _serialization as ser
from nvalchemi_toolkit_b200._optional import MissingDependencyError, OptionalDependency
from nvalchemi_toolkit_b200._typing import AtomCategory
from nvalchemi_toolkit_b200.dynamics import _units
from nvalchemi_toolkit_b200.models import _utils
from nvalchemi_toolkit_b200.utils import elements


def test_optional_dependency_gates_functions_and_classes():
    assert OptionalDependency.YAML.is_available() and OptionalDependency.YAML.import_module().__name__ == "yaml"
    missing = OptionalDependency.PYMATGEN
    if missing.is_available():
        pytest.skip("pymatgen is installed here")
    with pytest.raises(MissingDependencyError, match="pip install pymatgen"):
        missing.import_module()

    @missing.require
    def needs_it(x):
        return x + 1

    with pytest.raises(MissingDependencyError, match="needs_it"):
        needs_it(1)

    @missing.require
    class NeedsIt:
        def __init__(self, a):
            self.a = a

    with pytest.raises(MissingDependencyError, match="NeedsIt"):
        NeedsIt(3)

    @OptionalDependency.YAML.require
    def fine(x):
        return 2 * x

    assert fine(4) == 8 and fine.__name__ == "fine"  # present dependency: plain call, metadata kept
    assert isinstance(MissingDependencyError("x"), ImportError)


def test_dtype_device_and_tensor_json_round_trips():
    for dt in (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int32, torch.int64, torch.bool, torch.uint8):
        assert ser.str_to_dtype(ser.dtype_to_str(dt)) is dt
    assert ser.str_to_dtype(torch.float32) is torch.float32
    with pytest.raises((KeyError, ValueError)):
        ser.str_to_dtype("float7")
    assert ser.str_to_device(ser.device_to_str("cuda:1")) == torch.device("cuda", 1)
    t = torch.arange(6, dtype=torch.int64).reshape(2, 3)
    back = ser.tensor_from_json(json.loads(json.dumps(ser.tensor_to_json(t))))
    assert back.dtype == torch.int64 and torch.equal(back, t)
    empty = ser.tensor_from_json(ser.tensor_to_json(torch.zeros(0, 3)))
    assert empty.shape == (0, 3)
    assert ser.tensor_to_json(None) is None and ser.tensor_from_json(None) is None
    assert torch.equal(ser.tensor_from_json([1.0, 2.0]), torch.tensor([1.0, 2.0]))


def test_import_paths_and_nested_config_round_trip():
    from nvalchemi_toolkit_b200.training.optimizers import OptimizerConfig

    assert ser.import_from_path("torch.optim.Adam") is torch.optim.Adam
    assert ser.import_from_path("torch.optim:Adam") is torch.optim.Adam
    assert ser.import_from_path(ser.type_to_path(OptimizerConfig)) is OptimizerConfig
    with pytest.raises(ImportError):
        ser.import_from_path("no_such_package_anywhere.thing")
    with pytest.raises(AttributeError):
        ser.import_from_path("torch.optim.NoSuchOptimizer")
    with pytest.raises(ValueError, match="importable"):
        ser.type_to_path(lambda: None)
    config = {"dtype": torch.float64, "device": torch.device("cpu"), "act": torch.nn.SiLU, "shift": torch.tensor([1.5, -2.0]),
              "nested": [{"k": (1, 2)}, {"cls": torch.optim.SGD}], "plain": 3}
    wire = json.loads(json.dumps(ser.to_jsonable(config)))
    back = ser.from_jsonable(wire)
    assert back["dtype"] is torch.float64 and back["device"] == torch.device("cpu") and back["act"] is torch.nn.SiLU
    assert torch.equal(back["shift"], config["shift"]) and back["nested"][0]["k"] == [1, 2]
    assert back["nested"][1]["cls"] is torch.optim.SGD and back["plain"] == 3


class _Widget(ser.SerializableClass):
    def __init__(self, width: int, dtype: torch.dtype = torch.float32, scale: torch.Tensor | None = None):
        self._init_kwargs = {"width": width, "dtype": dtype, "scale": scale}
        self.width, self.dtype, self.scale = width, dtype, scale


def test_serializable_class_round_trips_through_json():
    w = _Widget(7, torch.float64, torch.tensor([0.5]))
    spec = json.loads(json.dumps(w.to_spec()))
    assert spec["cls"].endswith("test_foundation._Widget")
    again = ser.SerializableClass.from_spec(spec)
    assert isinstance(again, _Widget) and again.width == 7 and again.dtype is torch.float64
    assert torch.equal(again.scale, torch.tensor([0.5]))


def test_atom_categories_elements_and_units():
    assert AtomCategory.SPECIAL.value == -1 and AtomCategory(5) is AtomCategory.BULK and len(AtomCategory) == 12
    assert elements.SYMBOLS[1] == "H" and elements.SYMBOL_TO_Z["Cu"] == 29 and elements.SYMBOL_TO_Z["Og"] == 118
    assert float(elements.ATOMIC_MASSES[6]) == pytest.approx(12.011, abs=1e-3)
    assert float(elements.ATOMIC_MASSES[29]) == pytest.approx(63.546, abs=1e-3)
    assert bool((elements.ATOMIC_MASSES[1:100] > 0).all()) and len(elements.SYMBOLS) == elements.ATOMIC_MASSES.numel()
    # internal time unit sqrt(amu A^2 / eV) in femtoseconds, from CODATA constants
    amu, ev = 1.66053906660e-27, 1.602176634e-19
    assert _units.FS_PER_INTERNAL_TIME == pytest.approx(math.sqrt(amu * 1e-20 / ev) * 1e15, rel=1e-9)
    assert _units.fs_to_internal_time(_units.FS_PER_INTERNAL_TIME) == pytest.approx(1.0)
    assert _units.per_fs_to_internal_rate(1.0 / _units.FS_PER_INTERNAL_TIME) == pytest.approx(1.0)
    assert _units.KB_EV == pytest.approx(1.380649e-23 / ev, rel=1e-9)


def test_autograd_helpers_match_analytic_forces_and_stress():
    """Harmonic pair energy in a strained periodic box: forces and stress from the shared helpers against the closed
    forms (stress = sum over pairs of r (x) dE/dr / V)."""
    torch.manual_seed(0)
    pos0 = torch.rand(5, 3, dtype=torch.float64) * 3
    cell0 = (torch.eye(3, dtype=torch.float64) * 6).reshape(1, 3, 3)
    bidx = torch.zeros(5, dtype=torch.long)
    pos_in = pos0.clone().requires_grad_()
    pos, cell, strain = _utils.prepare_strain(pos_in, cell0, bidx)
    assert torch.equal(pos.detach(), pos0) and torch.equal(cell.detach(), cell0) and strain.shape == (1, 3, 3)
    i, j = torch.triu_indices(5, 5, 1)
    r = pos[j] - pos[i]
    energy = 0.5 * 1.7 * (r * r).sum()
    f, s = _utils.autograd_forces_and_stresses(energy.reshape(1), pos_in, strain, cell0)
    r0 = pos0[j] - pos0[i]
    want_f = torch.zeros_like(pos0).index_add_(0, i, 1.7 * r0).index_add_(0, j, -1.7 * r0)
    want_s = 1.7 * torch.einsum("pa,pb->ab", r0, r0) / 216.0
    assert torch.allclose(f, want_f, atol=1e-10) and torch.allclose(s[0], want_s, atol=1e-12)
    assert torch.allclose(s[0], s[0].T)
    pos_in2 = pos0.clone().requires_grad_()
    e2 = 0.5 * 1.7 * ((pos_in2[j] - pos_in2[i]) ** 2).sum()
    assert torch.allclose(_utils.autograd_forces(e2, pos_in2), want_f, atol=1e-10)
    # training=True keeps the graph: the force itself can be differentiated (force-matching losses)
    pos_in3 = pos0.clone().requires_grad_()
    k = torch.tensor(1.7, dtype=torch.float64, requires_grad=True)
    e3 = 0.5 * k * ((pos_in3[j] - pos_in3[i]) ** 2).sum()
    f3 = _utils.autograd_forces(e3, pos_in3, training=True)
    (gk,) = torch.autograd.grad((f3 ** 2).sum(), k)
    assert float(gk) == pytest.approx(float(2 * (want_f ** 2).sum() / 1.7), rel=1e-9)


def test_sum_outputs_and_cell_cache():
    a = {"energy": torch.tensor([1.0]), "forces": torch.ones(2, 3), "charges": torch.tensor([0.1, 0.2]), "stress": None}
    b = {"energy": torch.tensor([2.0]), "forces": 2 * torch.ones(2, 3), "charges": None, "stress": torch.eye(3)[None]}
    out = _utils.sum_outputs(a, b)
    assert float(out["energy"]) == 3.0 and float(out["forces"].sum()) == 18.0
    assert torch.equal(out["charges"], a["charges"])      # non-additive: the last value that is not None
    assert torch.equal(out["stress"], b["stress"])        # None + tensor -> tensor
    cell = torch.eye(3)[None] * 5
    assert _utils.cell_cache_needs_update(None, cell)
    assert not _utils.cell_cache_needs_update(cell.clone(), cell)
    assert _utils.cell_cache_needs_update(cell.clone(), cell * 1.001)
    assert _utils.cell_cache_needs_update(torch.eye(3)[None].repeat(2, 1, 1), cell)
