# SPDX-License-Identifier: Apache-2.0
"""Native MACE: symmetry properties of the torch path (CPU) and kernel-vs-oracle numerics (GPU)."""
import numpy as np
import pytest
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.models.base import NeighborListFormat
from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper, o3
from nvalchemi_toolkit_b200.neighbors import compute_neighbors
from nvalchemi_toolkit_b200.ops import gemm
from tests.helpers import fcc_supercell, random_batch


def _edges(pos, cutoff=5.0):
    d = (pos[:, None] - pos[None]).norm(dim=-1)
    i, j = torch.where((d < cutoff) & (d > 0))
    return torch.stack([i, j])


def test_tables_normalisation():
    v = torch.randn(7, 3, dtype=torch.float64)
    Y = o3.spherical_harmonics(v)
    for l in range(4):
        assert torch.allclose((Y[:, o3.lm_slice(l)] ** 2).sum(-1), torch.full((7,), 2.0 * l + 1, dtype=torch.float64))
    assert len(o3.conv_paths([0, 1])) == 10 and o3.mid_layout(o3.conv_paths([0, 1]))[2] == 40
    c = o3.cg(1, 1, 2)
    assert abs(float((c ** 2).sum()) - 5.0) < 1e-9


def test_torch_path_is_equivariant_and_conservative():
    torch.manual_seed(0)
    m = MACE(MACEConfig(atomic_numbers=[1, 8], channels=8, avg_num_neighbors=8.0), backend="torch").double()
    n = 10
    pos = torch.rand(n, 3, dtype=torch.float64) * 4
    z = torch.tensor([1, 8])[torch.randint(0, 2, (n,))]

    def run(p):
        return m({"positions": p.clone(), "atomic_numbers": z, "edge_index": _edges(p), "ptr": torch.tensor([0, n])})

    o1 = run(pos)
    R = torch.tensor(o3._random_rotation(np.random.default_rng(1)))
    o2 = run(pos @ R.T + 0.7)
    assert abs(float(o1["energy"] - o2["energy"])) < 1e-10
    assert float((o1["forces"] @ R.T - o2["forces"]).abs().max()) < 1e-10
    o3_ = run(-pos)
    assert abs(float(o1["energy"] - o3_["energy"])) < 1e-10
    eps = 1e-5
    p2, p3 = pos.clone(), pos.clone()
    p2[2, 0] += eps
    p3[2, 0] -= eps
    fd = -(run(p2)["energy"] - run(p3)["energy"]) / (2 * eps)
    assert abs(float(fd - o1["forces"][2, 0])) < 1e-6


def test_wrapper_matrix_and_coo_agree_with_pbc():
    torch.manual_seed(1)
    cfg = dict(atomic_numbers=[29], channels=8, avg_num_neighbors=40.0)
    w = MACEWrapper(MACE(MACEConfig(**cfg), backend="torch"))
    w.model_config.active_outputs = {"energy", "forces", "stress"}
    b = Batch.from_data_list([fcc_supercell(2, noise=0.1), fcc_supercell(2, a=3.8, noise=0.1, seed=4)])
    compute_neighbors(b, config=w.model_config.neighbor_config)
    o_m = w(b)
    w2 = MACEWrapper(w.model, neighbor_format=NeighborListFormat.COO)
    w2.model_config.active_outputs = {"energy", "forces", "stress"}
    b2 = Batch.from_data_list([fcc_supercell(2, noise=0.1), fcc_supercell(2, a=3.8, noise=0.1, seed=4)])
    compute_neighbors(b2, config=w2.model_config.neighbor_config)
    o_c = w2(b2)
    assert o_m["energy"].shape == (2, 1)
    assert torch.allclose(o_m["energy"], o_c["energy"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(o_m["forces"], o_c["forces"], rtol=1e-4, atol=1e-5)
    assert torch.allclose(o_m["stress"], o_c["stress"], rtol=1e-4, atol=1e-6)
    assert float(o_m["forces"].sum(0).abs().max()) < 1e-4  # momentum conservation


def test_stress_matches_finite_difference_of_cell():
    torch.manual_seed(2)
    m = MACE(MACEConfig(atomic_numbers=[29], channels=4, avg_num_neighbors=40.0), backend="torch").double()
    w = MACEWrapper(m)
    w.model_config.active_outputs = {"energy", "forces", "stress"}
    d = fcc_supercell(2, noise=0.1, dtype=torch.float64)

    def energy(scale):
        dd = d.clone()
        dd.__dict__["positions"] = d.positions * scale
        dd.__dict__["cell"] = d.cell * scale
        b = Batch.from_data_list([dd])
        compute_neighbors(b, config=w.model_config.neighbor_config)
        return w(b), b

    o, b = energy(1.0)
    eps = 1e-5
    de = (energy(1 + eps)[0]["energy"] - energy(1 - eps)[0]["energy"]) / (2 * eps)  # dE/d(iso strain) = tr(dE/deps)
    vol = torch.linalg.det(b.cell[0])
    assert abs(float(de.squeeze() / vol - torch.trace(o["stress"][0]))) < 1e-6 * max(1.0, abs(float(de)))


# ----------------------------------------------------------------------------------------- GPU numerics
@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(300, 128, 64), (1000, 1280, 64), (257, 100, 384), (128, 64, 32), (4096, 256, 128)])
def test_tcgen05_gemm_matches_fp32(m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda")
    w = torch.randn(k, n, device="cuda")
    ref = (a.double() @ w.double()).float()
    out = gemm.matmul(a, w)
    assert gemm.check_errors(a) == 0
    err = (out - ref).abs().max() / ref.abs().max()
    assert float(err) < 2e-3  # TF32 inputs, FP32 accumulation
    out2 = gemm.matmul(a, w, alpha=0.5, act=1)
    ref2 = torch.nn.functional.silu(0.5 * ref) * 1.6790176868438721
    assert float((out2 - ref2).abs().max() / ref2.abs().max()) < 3e-3
    if m % 2 == 0:  # interleaved (value, tangent) rows: activation and its derivative in the epilogue
        out3 = gemm.matmul(a, w, act=2)
        av, tv = ref[0::2], ref[1::2]
        sg = torch.sigmoid(av)
        ref3 = torch.stack([av * sg, sg * (1 + av * (1 - sg)) * tv], dim=1).reshape(ref.shape) * 1.6790176868438721
        assert float((out3 - ref3).abs().max() / ref3.abs().max()) < 6e-3


@pytest.mark.gpu
@pytest.mark.parametrize("precision", ["fp32", "tf32"])
def test_native_matches_oracle(precision):
    torch.manual_seed(3)
    cfg = MACEConfig(atomic_numbers=[29, 28], channels=32, avg_num_neighbors=40.0)
    model = MACE(cfg, backend="native").cuda()  # "native" raises instead of silently taking the PyTorch path
    oracle = MACE(cfg, backend="torch").double().cuda()
    oracle.load_state_dict({k: v.double() for k, v in model.state_dict().items()})
    d1, d2 = fcc_supercell(3, noise=0.1), fcc_supercell(2, a=3.9, noise=0.1, seed=7)
    d2.__dict__["atomic_numbers"] = torch.where(torch.arange(d2.num_nodes) % 2 == 0, 29, 28)
    b = Batch.from_data_list([d1, d2], device="cuda")
    w = MACEWrapper(model).eval()  # the kernels serve inference; a module in training mode uses the PyTorch path
    w.model_config.active_outputs = {"energy", "forces", "stress"}
    compute_neighbors(b, config=w.model_config.neighbor_config)
    gemm.set_precision(precision)
    try:
        out = w(b)
    finally:
        gemm.set_precision("tf32")
    assert gemm.check_errors(b.positions) == 0
    wo = MACEWrapper(oracle)
    wo.model_config.active_outputs = {"energy", "forces", "stress"}
    bo = b.clone().to(dtype=torch.float64)
    ref = wo(bo)
    tol = 2e-4 if precision == "fp32" else 2e-2
    fscale = float(ref["forces"].abs().max())
    assert float((out["energy"].double() - ref["energy"]).abs().max()) < tol * max(1.0, float(ref["energy"].abs().max()))
    assert float((out["forces"].double() - ref["forces"]).abs().max()) < tol * fscale
    assert float((out["stress"].double() - ref["stress"]).abs().max()) < tol * float(ref["stress"].abs().max())


@pytest.mark.gpu
def test_fused_tensor_core_convolution_matches_unfused():
    """128-channel model: radial weights produced by tcgen05 inside the convolution kernel vs the GEMM + SIMT path."""
    from nvalchemi_toolkit_b200.models.mace import native

    torch.manual_seed(5)
    cfg = MACEConfig(atomic_numbers=[29, 28], channels=128, avg_num_neighbors=40.0)
    model = MACE(cfg, backend="native").cuda()
    d1, d2 = fcc_supercell(3, noise=0.1), fcc_supercell(2, a=3.9, noise=0.1, seed=7)
    d2.__dict__["atomic_numbers"] = torch.where(torch.arange(d2.num_nodes) % 2 == 0, 29, 28)
    w = MACEWrapper(model).eval()
    w.model_config.active_outputs = {"energy", "forces", "stress"}
    outs = {}
    for fused in (True, False):
        b = Batch.from_data_list([d1, d2], device="cuda")
        compute_neighbors(b, config=w.model_config.neighbor_config)
        native.FUSED = fused
        try:
            outs[fused] = w(b)
        finally:
            native.FUSED = True
    assert native.fused_error_status(torch.device("cuda", 0)) == 0 and gemm.check_errors(b.positions) == 0
    ref, got = outs[False], outs[True]
    # the two paths round different operands to tf32 (the fused one keeps the first layer's input features in fp32):
    # measured 2e-4 / 2e-4 / 1e-3
    assert float((got["energy"] - ref["energy"]).abs().max()) < 1e-3 * max(1.0, float(ref["energy"].abs().max()))
    assert float((got["forces"] - ref["forces"]).abs().max()) < 3e-3 * float(ref["forces"].abs().max())
    assert float((got["stress"] - ref["stress"]).abs().max()) < 3e-3 * float(ref["stress"].abs().max())
    oracle = MACE(cfg, backend="torch").double().cuda()
    oracle.load_state_dict({k: v.double() for k, v in model.state_dict().items()})
    wo = MACEWrapper(oracle)
    bo = Batch.from_data_list([d1, d2], device="cuda").to(dtype=torch.float64)
    compute_neighbors(bo, config=wo.model_config.neighbor_config)
    exact = wo(bo)
    assert float((got["forces"].double() - exact["forces"]).abs().max()) < 2e-2 * float(exact["forces"].abs().max())
    # against the float64 oracle the fused path must not be worse than the unfused one (both are tf32-limited)
    e_fused = float((got["energy"].double() - exact["energy"]).abs().max())
    e_unfused = float((ref["energy"].double() - exact["energy"]).abs().max())
    assert e_fused < max(2.0 * e_unfused, 2e-4 * float(exact["energy"].abs().max()))
    err = {k: float((got[k] - ref[k]).abs().max() / ref[k].abs().max()) for k in ("energy", "forces", "stress")}
    print("fused vs unfused relative errors:", err, "| vs float64 oracle (forces):",
          float((got["forces"].double() - exact["forces"]).abs().max() / exact["forces"].abs().max()))


@pytest.mark.gpu
def test_fused_backward_feature_gradient_matches_unfused_elementwise():
    """Intermediate gradients of the two backward convolution paths agree element by element: a wrong layout of the
    feature gradient would be an O(1) error here even if the final forces hid it."""
    from nvalchemi_toolkit_b200.models.mace import native

    torch.manual_seed(11)
    cfg = MACEConfig(atomic_numbers=[29], channels=128, avg_num_neighbors=40.0)
    model = MACE(cfg, backend="native").cuda()
    w = MACEWrapper(model).eval()
    w.model_config.active_outputs = {"energy", "forces"}
    seen = {}
    orig = native._per_l_linear

    def spy(x, wt, ls, transpose=False, **kw):
        if transpose and x.dim() == 3 and x.shape[1] == 4:  # the feature gradient of layer 2 enters here
            seen.setdefault(native.FUSED, []).append(x.detach().clone())
        return orig(x, wt, ls, transpose=transpose, **kw)

    native._per_l_linear = spy
    try:
        for fused in (True, False):
            b = Batch.from_data_list([fcc_supercell(3, noise=0.1, seed=2)], device="cuda")
            compute_neighbors(b, config=w.model_config.neighbor_config)
            native.FUSED = fused
            w(b)
    finally:
        native.FUSED = True
        native._per_l_linear = orig
    assert set(seen) == {True, False}, {k: [tuple(t.shape) for t in v] for k, v in seen.items()}
    a, r = seen[True][0], seen[False][0]
    assert a.shape == r.shape and float(r.abs().max()) > 0
    assert float((a - r).abs().max()) < 5e-3 * float(r.abs().max())


@pytest.mark.gpu
def test_neighbor_matrix_gpu_matches_cpu():
    b = Batch.from_data_list([fcc_supercell(4), fcc_supercell(1, a=3.0, seed=5)])
    compute_neighbors(b, 5.0)
    g = b.clone().cuda()
    compute_neighbors(g, 5.0)
    assert torch.equal(g.num_neighbors.cpu(), b.num_neighbors)

    def canon(x):
        nm, num, sh = x.neighbor_matrix.cpu(), x.num_neighbors.cpu(), x.neighbor_matrix_shifts.cpu()
        return {(i, int(nm[i, q]), *sh[i, q].tolist()) for i in range(nm.shape[0]) for q in range(int(num[i]))}

    assert canon(g) == canon(b)
    m = random_batch([12, 30, 7])
    compute_neighbors(m, 4.0)
    mg = m.clone().cuda()
    compute_neighbors(mg, 4.0)
    assert torch.equal(mg.num_neighbors.cpu(), m.num_neighbors)


def test_radial_cache_pool_reuses_and_releases_storage():
    from nvalchemi_toolkit_b200.models.mace import native

    like = torch.zeros(1)
    a = native._pooled(("t", 0), 1000, like)
    assert a.numel() >= 1000 and native._pooled(("t", 0), 900, like) is a     # smaller request: same storage
    b = native._pooled(("t", 0), a.numel() + 1, like)
    assert b is not a and b.numel() > a.numel()                                # grown, old buffer dropped
    assert not native._radial_cache_fits(torch.device("cpu"), 10, 2)           # only used on CUDA devices
    native.release_radial_cache()
    assert not native._h3_pool


def test_hessian_output_matches_finite_differences_of_forces():
    """``hessian`` (d2E / dr dr, ``[3N, 3N]``) from the wrapper against central differences of the forces."""
    torch.manual_seed(3)
    cfg = MACEConfig(atomic_numbers=[29], channels=8, avg_num_neighbors=10.0, r_max=4.0)
    w = MACEWrapper(MACE(cfg, backend="torch").double()).eval()
    d = fcc_supercell(1, a=3.7, noise=0.15, dtype=torch.float64)
    w.model_config.active_outputs = {"energy", "forces", "hessian"}
    b = Batch.from_data_list([d])
    compute_neighbors(b, config=w.model_config.neighbor_config)
    out = w(b)
    n = b.num_nodes
    H = out["hessian"].detach()
    assert H.shape == (3 * n, 3 * n) and torch.allclose(H, H.t(), atol=1e-9)
    w.model_config.active_outputs = {"energy", "forces"}
    eps = 1e-5
    for col in (0, 4, 3 * n - 1):
        f = []
        for sgn in (1.0, -1.0):
            bb = Batch.from_data_list([d])
            pos = bb.positions.clone().reshape(-1)
            pos[col] += sgn * eps
            bb["positions"] = pos.reshape(-1, 3)
            compute_neighbors(bb, config=w.model_config.neighbor_config)
            f.append(w(bb)["forces"].detach().reshape(-1))
        fd = -(f[0] - f[1]) / (2 * eps)
        assert torch.allclose(H[:, col], fd, atol=1e-6), float((H[:, col] - fd).abs().max())


def test_agnesi_distance_transform():
    """The species-pair distance transform of the MACE foundation models: maps (0, inf) onto (1, 0) monotonically, equals
    1 / (1 + a / 2) at the covalent distance, changes the energy, keeps forces consistent with finite differences."""
    from nvalchemi_toolkit_b200.models.mace.model import COVALENT_RADII, agnesi_transform

    r = torch.linspace(0.3, 6.0, 200, dtype=torch.float64)
    t = agnesi_transform(r, torch.tensor(1.32, dtype=torch.float64))
    assert bool((t[1:] < t[:-1]).all()) and 0.0 < float(t[-1]) < float(t[0]) < 1.0
    at_r0 = agnesi_transform(torch.tensor(1.32, dtype=torch.float64), torch.tensor(1.32, dtype=torch.float64))
    assert abs(float(at_r0) - 1.0 / (1.0 + 1.0805 / 2.0)) < 1e-12
    assert COVALENT_RADII[1] == 0.31 and COVALENT_RADII[6] == 0.76 and COVALENT_RADII[29] == 1.32 and len(COVALENT_RADII) == 87
    torch.manual_seed(0)
    plain = MACE(MACEConfig(atomic_numbers=[29, 28], channels=8, avg_num_neighbors=20.0), backend="torch").double()
    agn = MACE(MACEConfig(atomic_numbers=[29, 28], channels=8, avg_num_neighbors=20.0, distance_transform="Agnesi"), backend="torch").double()
    agn.load_state_dict(plain.state_dict())
    d = fcc_supercell(2, noise=0.1, dtype=torch.float64)
    d.__dict__["atomic_numbers"] = torch.where(torch.arange(d.num_nodes) % 2 == 0, 29, 28)
    b = Batch.from_data_list([d])
    w0, w1 = MACEWrapper(plain), MACEWrapper(agn)
    for w in (w0, w1):
        w.model_config.active_outputs = {"energy", "forces"}
    compute_neighbors(b, config=w0.model_config.neighbor_config)
    e0, out = w0(b)["energy"], w1(b)
    assert abs(float(e0 - out["energy"])) > 1e-6
    i, eps = 3, 1e-5
    bp, bm = b.clone(), b.clone()
    bp.positions[i, 0] += eps
    bm.positions[i, 0] -= eps
    fd = -(float(w1(bp)["energy"]) - float(w1(bm)["energy"])) / (2 * eps)
    assert abs(fd - float(out["forces"][i, 0])) < 1e-6 * max(1.0, abs(fd))
    with pytest.raises(RuntimeError, match="distance_transform"):
        MACE(MACEConfig(atomic_numbers=[29], channels=8, distance_transform="Agnesi"), backend="native")._use_native(b.positions, False)
