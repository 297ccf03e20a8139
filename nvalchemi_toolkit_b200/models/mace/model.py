# SPDX-License-Identifier: Apache-2.0
"""Native MACE network (``ScaleShiftMACE`` architecture) with two execution paths.

The reference only *wraps* the external ``mace-torch`` network (``nvalchemi/models/mace.py:518-1158``);
this module provides the network itself.  Architecture (Batatia et al., as used by the reference's
training recipe ``examples/advanced/_mace_models.py:134-207``): linear node embedding, Bessel radial basis
with polynomial cutoff, spherical harmonics up to ``max_ell``, ``num_interactions`` residual interaction
blocks (``linear_up`` → radial-MLP-weighted channel-wise tensor product with neighbour aggregation →
``linear`` / ``avg_num_neighbors``; element-dependent skip connection), symmetric-contraction product basis of
the given ``correlation``, linear readouts (MLP readout on the last layer), scale/shift and per-element E0.

Paths:

* ``backend="torch"`` — plain differentiable PyTorch (any dtype, double backward): the numerical oracle and
  the path used for force-matching training.
* ``backend="native"`` — hand-written sm_100a kernels (``torch.ops.nvalchemi.mace_*``) for energy and analytic
  forces: fused edge geometry + tensor product + neighbour aggregation without atomics, symmetric contraction,
  TMEM/tcgen05 channel mixes.  Used for MD / relaxation.

Feature tensors are ``[N, n_lm, C]`` (channel fastest).  Edge vectors point from sender to receiver,
``r_receiver - r_sender + shift``, messages are summed at the receiver (MACE convention).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200.models.mace import o3

SILU_NORM = 1.6790176868438721  # 1 / sqrt(E[silu(z)^2]), z ~ N(0,1): unit second moment after the activation


@dataclass
class MACEConfig:
    atomic_numbers: list[int] = field(default_factory=lambda: [29])
    r_max: float = 5.0
    num_bessel: int = 8
    num_polynomial_cutoff: int = 5
    max_ell: int = 3
    num_interactions: int = 2
    channels: int = 128
    hidden_lmax: int = 1  # "128x0e+128x1o"
    mlp_readout_dim: int = 16
    correlation: int = 3
    radial_mlp: list[int] = field(default_factory=lambda: [64, 64, 64])
    avg_num_neighbors: float = 1.0
    atomic_energies: list[float] | None = None
    scale: float = 1.0
    shift: float = 0.0
    #: ``"None"`` or ``"Agnesi"``: the radial basis then sees a species-pair dependent transform of the distance
    #: (``mace.modules.radial.AgnesiTransform``, used by the MACE-MP foundation models); the PyTorch path implements it,
    #: the native kernels evaluate the plain Bessel basis only, so a model with a transform runs the PyTorch path
    distance_transform: str = "None"

    def __post_init__(self) -> None:
        if self.distance_transform not in ("None", "Agnesi"):
            raise ValueError(f"distance_transform must be 'None' or 'Agnesi', got {self.distance_transform!r}")

    @classmethod
    def from_hidden_irreps(cls, hidden_irreps: str, **kw: Any) -> "MACEConfig":
        """Accepts e3nn-style strings such as ``"128x0e+128x1o"``."""
        parts = [p.strip() for p in hidden_irreps.split("+")]
        mul = int(parts[0].split("x")[0])
        lmax = max(int(p.split("x")[1][0]) for p in parts)
        return cls(channels=mul, hidden_lmax=lmax, **kw)


def bessel_basis(r: torch.Tensor, r_max: float, n: int) -> torch.Tensor:
    k = torch.arange(1, n + 1, dtype=r.dtype, device=r.device) * (math.pi / r_max)
    return math.sqrt(2.0 / r_max) * torch.sin(k * r.unsqueeze(-1)) / r.unsqueeze(-1)


# Covalent radii in Angstrom (Cordero et al., Dalton Trans. 2008; the table ASE ships), indexed by atomic number.
COVALENT_RADII = (0.2, 0.31, 0.28, 1.28, 0.96, 0.84, 0.76, 0.71, 0.66, 0.57, 0.58, 1.66, 1.41, 1.21, 1.11, 1.07, 1.05, 1.02, 1.06,
                  2.03, 1.76, 1.70, 1.60, 1.53, 1.39, 1.39, 1.32, 1.26, 1.24, 1.32, 1.22, 1.22, 1.20, 1.19, 1.20, 1.20, 1.16,
                  2.20, 1.95, 1.90, 1.75, 1.64, 1.54, 1.47, 1.46, 1.42, 1.39, 1.45, 1.44, 1.42, 1.39, 1.39, 1.38, 1.39, 1.40,
                  2.44, 2.15, 2.07, 2.04, 2.03, 2.01, 1.99, 1.98, 1.98, 1.96, 1.94, 1.92, 1.92, 1.89, 1.90, 1.87, 1.87,
                  1.75, 1.70, 1.62, 1.51, 1.44, 1.41, 1.36, 1.36, 1.32, 1.45, 1.46, 1.48, 1.40, 1.50, 1.50)


def agnesi_transform(r: torch.Tensor, r0: torch.Tensor, q: float = 0.9183, p: float = 4.5791, a: float = 1.0805) -> torch.Tensor:
    """``1 / (1 + a x^q / (1 + x^(q - p)))`` with ``x = r / r0`` and ``r0`` the mean covalent radius of the pair: a smooth,
    monotonically decreasing map of the distance onto (0, 1) that resolves the bonding region
    (``mace/modules/radial.py`` ``AgnesiTransform``)."""
    x = r / r0
    return 1.0 / (1.0 + a * x.pow(q) / (1.0 + x.pow(q - p)))


def polynomial_cutoff(r: torch.Tensor, r_max: float, p: int) -> torch.Tensor:
    x = r / r_max
    env = (1.0 - 0.5 * (p + 1) * (p + 2) * x ** p + p * (p + 2) * x ** (p + 1) - 0.5 * p * (p + 1) * x ** (p + 2))
    return env * (x < 1.0)


class InteractionParams(nn.Module):
    """Weights of one interaction + product + readout layer."""

    def __init__(self, cfg: MACEConfig, layer: int) -> None:
        super().__init__()
        C, Z = cfg.channels, len(cfg.atomic_numbers)
        last = layer == cfg.num_interactions - 1
        self.l_in = [0] if layer == 0 else list(range(cfg.hidden_lmax + 1))
        self.l_out = [0] if last else list(range(cfg.hidden_lmax + 1))
        self.paths = o3.conv_paths(self.l_in, cfg.max_ell, cfg.max_ell)
        self.mid_off, self.paths_per_l, self.n_mid = o3.mid_layout(self.paths, cfg.max_ell)
        P = len(self.paths)
        self.linear_up = nn.Parameter(torch.randn(len(self.l_in), C, C))
        dims = [cfg.num_bessel] + list(cfg.radial_mlp) + [P * C]
        self.radial = nn.ParameterList([nn.Parameter(torch.randn(a, b)) for a, b in zip(dims[:-1], dims[1:])])
        self.linear = nn.ParameterList(
            [nn.Parameter(torch.randn(self.paths_per_l[l] * C, C)) for l in range(cfg.max_ell + 1)])
        self.skip = nn.Parameter(torch.randn(len(self.l_out), Z, C, C))
        self.sym = nn.ParameterDict()
        for L in self.l_out:
            for nu in range(1, cfg.correlation + 1):
                nb = o3.load_tables()[f"sym_U_{nu}_{L}"].shape[0]
                self.sym[f"w{nu}_{L}"] = nn.Parameter(torch.randn(Z, nb, C) / max(nb, 1))
        self.product_linear = nn.Parameter(torch.randn(len(self.l_out), C, C))
        if last:
            self.readout_w1 = nn.Parameter(torch.randn(C, cfg.mlp_readout_dim))
            self.readout_w2 = nn.Parameter(torch.randn(cfg.mlp_readout_dim))
        else:
            self.readout_w1 = nn.Parameter(torch.randn(C))
            self.readout_w2 = None
        self.last = last


class MACE(nn.Module):
    """Native ScaleShiftMACE.  ``forward`` takes and returns the dictionary contract of the reference wrapper
    (``nvalchemi/models/mace.py:756-870``)."""

    def __init__(self, config: MACEConfig | None = None, backend: str = "auto", **kw: Any) -> None:
        super().__init__()
        cfg = config or MACEConfig(**kw)
        if cfg.max_ell != 3 or cfg.hidden_lmax not in (0, 1) or cfg.correlation not in (1, 2, 3):
            raise NotImplementedError("native MACE supports max_ell=3, hidden_lmax in {0,1}, correlation <= 3")
        self.config = cfg
        self.backend = backend
        Z, C = len(cfg.atomic_numbers), cfg.channels
        self.register_buffer("atomic_numbers", torch.tensor(cfg.atomic_numbers, dtype=torch.long))
        self.r_max = cfg.r_max
        self.node_embedding = nn.Parameter(torch.randn(Z, C))
        e0 = cfg.atomic_energies if cfg.atomic_energies is not None else [0.0] * Z
        self.register_buffer("atomic_energies", torch.tensor(e0, dtype=torch.get_default_dtype()))
        self.register_buffer("scale", torch.tensor(float(cfg.scale)))
        self.register_buffer("shift", torch.tensor(float(cfg.shift)))
        self.interactions = nn.ModuleList([InteractionParams(cfg, t) for t in range(cfg.num_interactions)])
        z_lut = torch.full((int(max(cfg.atomic_numbers)) + 1,), -1, dtype=torch.long)
        z_lut[torch.tensor(cfg.atomic_numbers)] = torch.arange(Z)
        self.register_buffer("z_lut", z_lut, persistent=False)
        self._tables: dict[tuple, Any] = {}

    # ------------------------------------------------------------------ helpers
    def species_index(self, atomic_numbers: torch.Tensor) -> torch.Tensor:
        idx = self.z_lut[atomic_numbers.long().clamp(0, self.z_lut.numel() - 1)]
        return idx

    def hidden_dim(self) -> int:
        return self.config.channels * (self.config.hidden_lmax + 1) ** 2

    def _cg(self, l1: int, l2: int, l3: int, ref: torch.Tensor) -> torch.Tensor:
        key = ("cg", l1, l2, l3, ref.dtype, ref.device)
        if key not in self._tables:
            self._tables[key] = o3.cg(l1, l2, l3, ref.dtype, ref.device)
        return self._tables[key]

    def _sym(self, nu: int, L: int, ref: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        key = ("sym", nu, L, ref.dtype, ref.device)
        if key not in self._tables:
            t = o3.load_tables()
            self._tables[key] = (torch.as_tensor(t[f"sym_mono_{nu}"], device=ref.device),
                                 torch.as_tensor(t[f"sym_U_{nu}_{L}"], dtype=ref.dtype, device=ref.device))
        return self._tables[key]

    def _use_native(self, positions: torch.Tensor, training: bool) -> bool:
        if self.backend == "torch":
            return False
        if self.config.distance_transform != "None":
            if self.backend == "native":
                raise RuntimeError("backend='native' evaluates the plain Bessel basis; distance_transform needs the PyTorch path")
            return False
        ok = positions.is_cuda and positions.dtype == torch.float32 and not training
        if self.backend == "native" and not ok:
            raise RuntimeError("backend='native' needs float32 CUDA tensors and training=False")
        return ok

    # ------------------------------------------------------------------ torch path
    def radial_weights(self, ip: InteractionParams, edge_feats: torch.Tensor) -> torch.Tensor:
        x = edge_feats
        n = len(ip.radial)
        for k, w in enumerate(ip.radial):
            x = x @ (w / math.sqrt(w.shape[0]))
            if k < n - 1:
                x = torch.nn.functional.silu(x) * SILU_NORM
        return x.reshape(x.shape[0], len(ip.paths), self.config.channels)

    def _conv_torch(self, ip: InteractionParams, u: torch.Tensor, Y: torch.Tensor, R: torch.Tensor,
                    sender: torch.Tensor, receiver: torch.Tensor, n: int) -> torch.Tensor:
        C = self.config.channels
        us = u[sender]  # [E, nin, C]
        mid_e = us.new_zeros(us.shape[0], ip.n_mid, C)
        seen = [0] * (self.config.max_ell + 1)
        in_off = {l: sum(2 * k + 1 for k in ip.l_in[: ip.l_in.index(l)]) for l in ip.l_in}
        for p, (l1, l2, l3) in enumerate(ip.paths):
            cgt = self._cg(l1, l2, l3, u)
            a = us[:, in_off[l1]: in_off[l1] + 2 * l1 + 1]
            b = Y[:, o3.lm_slice(l2)]
            m = torch.einsum("eac,eb,abm->emc", a, b, cgt) * R[:, p].unsqueeze(1)
            k = seen[l3]
            seen[l3] += 1
            idx = [ip.mid_off[l3] + m3 * ip.paths_per_l[l3] + k for m3 in range(2 * l3 + 1)]
            mid_e[:, idx] = mid_e[:, idx] + m
        return u.new_zeros(n, ip.n_mid, C).index_add_(0, receiver, mid_e)

    def _linear_mid(self, ip: InteractionParams, mid: torch.Tensor) -> torch.Tensor:
        C = self.config.channels
        outs = []
        for l in range(self.config.max_ell + 1):
            npl = ip.paths_per_l[l]
            blk = mid[:, ip.mid_off[l]: ip.mid_off[l] + (2 * l + 1) * npl].reshape(mid.shape[0], 2 * l + 1, npl * C)
            outs.append(blk @ (ip.linear[l] / math.sqrt(npl * C)))
        return torch.cat(outs, dim=1) / self.config.avg_num_neighbors  # [N, 16, C]

    def _symcon_torch(self, ip: InteractionParams, msg: torch.Tensor, species: torch.Tensor) -> torch.Tensor:
        outs = []
        x = msg  # [N, 16, C]
        for L in ip.l_out:
            acc = msg.new_zeros(msg.shape[0], 2 * L + 1, msg.shape[2])
            for nu in range(1, self.config.correlation + 1):
                monos, U = self._sym(nu, L, msg)
                if U.shape[0] == 0:
                    continue
                mono_val = x[:, monos[:, 0]]
                for q in range(1, nu):
                    mono_val = mono_val * x[:, monos[:, q]]  # [N, T, C]
                w = ip.sym[f"w{nu}_{L}"][species]  # [N, nb, C]
                basis = torch.einsum("emt,ntc->nemc", U, mono_val)
                acc = acc + torch.einsum("nemc,nec->nmc", basis, w)
            outs.append(acc)
        return torch.cat(outs, dim=1)  # [N, n_lm_out, C]

    @staticmethod
    def _per_l_linear(x: torch.Tensor, w: torch.Tensor, ls: list[int]) -> torch.Tensor:
        """x [N, n_lm, C] @ w[l_index] per irrep (1/sqrt(C) path normalisation)."""
        C = x.shape[-1]
        outs, off = [], 0
        for i, l in enumerate(ls):
            outs.append(x[:, off: off + 2 * l + 1] @ (w[i] / math.sqrt(C)))
            off += 2 * l + 1
        return torch.cat(outs, dim=1)

    def _skip(self, ip: InteractionParams, h: torch.Tensor, species: torch.Tensor) -> torch.Tensor:
        C, Z = self.config.channels, len(self.config.atomic_numbers)
        outs, off = [], 0
        for i, l in enumerate(ip.l_out):
            if l in ip.l_in:
                o = sum(2 * k + 1 for k in ip.l_in[: ip.l_in.index(l)])
                w = ip.skip[i][species] / math.sqrt(C * Z)  # [N, C, C]
                outs.append(torch.einsum("nmc,ncd->nmd", h[:, o: o + 2 * l + 1], w))
            else:
                outs.append(h.new_zeros(h.shape[0], 2 * l + 1, C))
            off += 2 * l + 1
        return torch.cat(outs, dim=1)

    def _readout(self, ip: InteractionParams, h: torch.Tensor) -> torch.Tensor:
        C = self.config.channels
        s = h[:, 0]  # scalars [N, C]
        if ip.last:
            y = torch.nn.functional.silu(s @ (ip.readout_w1 / math.sqrt(C))) * SILU_NORM
            return y @ (ip.readout_w2 / math.sqrt(ip.readout_w2.shape[0]))
        return s @ (ip.readout_w1 / math.sqrt(C))

    def node_energies_torch(self, positions: torch.Tensor, species: torch.Tensor, sender: torch.Tensor,
                            receiver: torch.Tensor, shifts: torch.Tensor, return_features: bool = False
                            ) -> Any:
        cfg = self.config
        n = positions.shape[0]
        vec = positions[receiver] - positions[sender] + shifts
        r = vec.norm(dim=-1)
        Y = o3.spherical_harmonics(vec, cfg.max_ell, normalize=True)
        r_basis = r
        if cfg.distance_transform == "Agnesi":
            rc = torch.tensor(COVALENT_RADII, dtype=r.dtype, device=r.device)[
                torch.tensor(cfg.atomic_numbers, device=r.device)][species]
            r_basis = agnesi_transform(r, 0.5 * (rc[sender] + rc[receiver]))
        ef = bessel_basis(r_basis, cfg.r_max, cfg.num_bessel) * polynomial_cutoff(r, cfg.r_max, cfg.num_polynomial_cutoff).unsqueeze(-1)
        Z = len(cfg.atomic_numbers)
        h = (self.node_embedding / math.sqrt(Z))[species].unsqueeze(1)  # [N,1,C]
        total = positions.new_zeros(n)
        feats = []
        for ip in self.interactions:
            sc = self._skip(ip, h, species)
            u = self._per_l_linear(h, ip.linear_up, ip.l_in)
            R = self.radial_weights(ip, ef)
            mid = self._conv_torch(ip, u, Y, R, sender, receiver, n)
            msg = self._linear_mid(ip, mid)
            B = self._symcon_torch(ip, msg, species)
            h = self._per_l_linear(B, ip.product_linear, ip.l_out) + sc
            feats.append(h)
            total = total + self._readout(ip, h)
        e = self.atomic_energies.to(positions.dtype)[species] + total * self.scale.to(positions.dtype) + self.shift.to(positions.dtype)
        return (e, feats) if return_features else e

    # ------------------------------------------------------------------ public forward
    def forward(self, data: dict[str, torch.Tensor], compute_force: bool = True, compute_stress: bool = False,
                compute_displacement: bool = False, training: bool = False, compute_hessian: bool = False
                ) -> dict[str, torch.Tensor | None]:
        """``data``: ``positions [N,3]``, ``node_attrs [N,Z]`` (one-hot) or ``atomic_numbers [N]``, ``batch [N]``,
        ``ptr [B+1]``, ``edge_index [2,E]`` (sender, receiver), ``shifts [E,3]``, ``cell [B,3,3]``; optionally the
        dense neighbour format ``neighbor_matrix``, ``num_neighbors``, ``neighbor_matrix_shifts`` (preferred by the
        native path)."""
        positions = data["positions"]
        if "node_attrs" in data and data["node_attrs"] is not None:
            species = data["node_attrs"].argmax(dim=-1)
        else:
            species = self.species_index(data["atomic_numbers"])
        batch = data.get("batch")
        if batch is None:
            batch = torch.zeros(positions.shape[0], dtype=torch.long, device=positions.device)
        num_graphs = int(data["ptr"].numel() - 1) if data.get("ptr") is not None else int(data.get("num_graphs", 1))
        cell = data.get("cell")
        if self._use_native(positions, training) and not compute_hessian:
            from nvalchemi_toolkit_b200.models.mace import native

            return native.forward(self, data, species, batch.long(), num_graphs, compute_force, compute_stress,
                                  energy_weights=data.get("energy_weights"))
        sender, receiver, shifts = self._edges_from(data, positions, batch.long(), cell)
        need_grad = compute_force or compute_stress or compute_hessian
        keep_graph = need_grad or training or (positions.requires_grad and torch.is_grad_enabled())
        with torch.enable_grad() if keep_graph else torch.no_grad():
            pos = positions
            strain = None
            if compute_stress and cell is not None:
                from nvalchemi_toolkit_b200.models._utils import prepare_strain

                if not pos.requires_grad:
                    pos = pos.detach().requires_grad_(True)
                unit = data.get("unit_shifts")
                spos, scell, strain = prepare_strain(pos, cell, batch)
                if unit is not None:
                    shifts = torch.einsum("ei,eij->ej", unit.to(pos.dtype), scell[batch[sender]])
                else:
                    sym = 0.5 * (strain + strain.transpose(-1, -2))
                    shifts = shifts + torch.einsum("ei,eij->ej", shifts, sym[batch[sender]])
                pos_in = spos
            else:
                if need_grad and not pos.requires_grad:
                    pos = pos.detach().requires_grad_(True)
                pos_in = pos
            node_e = self.node_energies_torch(pos_in, species, sender, receiver, shifts)
            ew = data.get("energy_weights")  # per-atom weights of the energy sum (domain decomposition: 0 on ghosts)
            energy = pos.new_zeros(num_graphs).index_add_(0, batch.long(), node_e if ew is None else node_e * ew.to(node_e.dtype))
            out: dict[str, torch.Tensor | None] = {"energy": energy, "node_energy": node_e, "forces": None,
                                                    "stress": None, "hessian": None}
            if compute_force and strain is not None:
                gp, gs = torch.autograd.grad(energy.sum(), [pos, strain], create_graph=training, retain_graph=training or compute_hessian)
                out["forces"] = -gp
                vol = torch.linalg.det(cell).abs()
                out["stress"] = gs / vol[:, None, None]
                out["virial"] = -gs
            elif compute_force:
                (gp,) = torch.autograd.grad(energy.sum(), pos, create_graph=training or compute_hessian,
                                            retain_graph=training or compute_hessian)
                out["forces"] = -gp
            if compute_hessian:
                f = out["forces"].reshape(-1)
                rows = [torch.autograd.grad(f[i], pos, retain_graph=True)[0].reshape(-1) for i in range(f.numel())]
                out["hessian"] = -torch.stack(rows)
        return out

    @staticmethod
    def _edges_from(data: dict, positions: torch.Tensor, batch: torch.Tensor, cell: torch.Tensor | None
                    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if data.get("edge_index") is not None:
            ei = data["edge_index"].long()
            sh = data.get("shifts")
            if sh is None:
                sh = positions.new_zeros(ei.shape[1], 3)
            return ei[0], ei[1], sh.to(positions.dtype)
        nm, num = data["neighbor_matrix"], data["num_neighbors"]
        n, k = nm.shape
        valid = torch.arange(k, device=nm.device)[None, :] < num[:, None].clamp_max(k)
        recv = torch.arange(n, device=nm.device)[:, None].expand(n, k)[valid]
        send = nm[valid].long()
        S = data.get("neighbor_matrix_shifts")
        if S is not None and cell is not None:
            sh = -torch.einsum("ei,eij->ej", S[valid].to(positions.dtype), cell[batch[recv]].to(positions.dtype))
        else:
            sh = positions.new_zeros(send.shape[0], 3)
        return send, recv, sh

    def extra_repr(self) -> str:
        return ", ".join(f"{k}={v}" for k, v in asdict(self.config).items())
