# SPDX-License-Identifier: Apache-2.0
"""Energy + analytic forces of the native MACE through the sm_100a kernels.

The backward pass is written out by hand (no autograd graph): every layer keeps only the tensors its
adjoint needs (``u``, the aggregated message ``msg`` and the post-product features), the radial weights are
recomputed per receiver chunk, and forces come from the adjoint of the fused convolution kernel.  This is
the path used by MD and relaxation; the differentiable torch path in :mod:`model` is the oracle.

Replaces, for the reference's MACE wrapper (``nvalchemi/models/mace.py:872-910``), the e3nn/cuEquivariance
forward plus ``torch.autograd.grad`` for forces.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any

import torch

from nvalchemi_toolkit_b200.models.mace.model import SILU_NORM
from nvalchemi_toolkit_b200.ops import _native, gemm

from nvalchemi_toolkit_b200.ops._native_counter import ops  # noqa: E402

#: upper bound on the radial-weight scratch per chunk (bytes); [E_chunk, 2, P, C] floats in the backward
CHUNK_BYTES = 2 << 30
#: chunk bound while the radial activations are kept for the adjoint anyway (the buffers are pooled and resident, so
#: small chunks would only multiply kernel launches: eleven chunks per layer at 1 M atoms with the bound above)
CACHED_CHUNK_BYTES = 24 << 30


@dataclass
class EdgeCSR:
    """Receiver-major edge list derived from the dense neighbour matrix."""

    eptr: torch.Tensor   # [N+1] int32
    esend: torch.Tensor  # [E] int32
    erecv: torch.Tensor  # [E] int32
    eS: torch.Tensor     # [E,3] int32 (integer images of the sender)
    eptr_host: list[int] | None = None
    num_edges: int = 0
    max_count: int = 0   # largest neighbour count seen (a value above the matrix width signals overflow)


def build_csr(nm: torch.Tensor, num: torch.Tensor, shifts: torch.Tensor | None) -> EdgeCSR:
    n, k = nm.shape
    cnt = num.clamp_max(k).to(torch.int32)
    if (nm.is_cuda and nm.dtype == torch.int32 and nm.is_contiguous() and _native.available()
            and (shifts is None or (shifts.dtype == torch.int32 and shifts.is_contiguous()))):
        # one pass over the matrix instead of boolean-mask gathers (each of which is a select + gather over N x K)
        eptr = torch.zeros(n + 1, dtype=torch.int32, device=nm.device)
        torch.cumsum(cnt, 0, out=eptr[1:])
        stats = torch.stack([eptr[-1], num.max().to(torch.int32) if n else eptr[-1]]).tolist()  # one host read
        e, mx = int(stats[0]), (int(stats[1]) if n else 0)
        esend = torch.empty(e, dtype=torch.int32, device=nm.device)
        erecv = torch.empty(e, dtype=torch.int32, device=nm.device)
        eS = torch.empty(e, 3, dtype=torch.int32, device=nm.device)
        ops.csr_fill(nm, shifts, eptr, esend, erecv, eS)
        return EdgeCSR(eptr, esend, erecv, eS, None, e, mx)
    valid = torch.arange(k, device=nm.device, dtype=torch.int32)[None, :] < cnt[:, None]
    esend = nm[valid].to(torch.int32).contiguous()
    e = esend.numel()
    eptr = torch.zeros(n + 1, dtype=torch.int32, device=nm.device)
    torch.cumsum(cnt, 0, out=eptr[1:])
    erecv = torch.repeat_interleave(torch.arange(n, device=nm.device, dtype=torch.int32), cnt.long(), output_size=e)
    eS = shifts[valid].to(torch.int32).contiguous() if shifts is not None else \
        torch.zeros(e, 3, dtype=torch.int32, device=nm.device)
    mx = int(num.max()) if n else 0  # one host read per neighbour-list build (also sizes the edge arrays)
    return EdgeCSR(eptr, esend, erecv, eS, None, e, mx)


def csr_from_edge_index(edge_index: torch.Tensor, unit_shifts: torch.Tensor | None, n: int) -> EdgeCSR:
    """COO (sender, receiver) → receiver-major CSR.  ``unit_shifts`` follow the MACE convention
    (``vec = r_recv - r_send + S @ cell``); the kernels use ``vec = r_i - (r_j + S' @ cell)`` so ``S' = -S``."""
    send, recv = edge_index[0].long(), edge_index[1].long()
    order = torch.argsort(recv, stable=True)
    cnt = torch.bincount(recv, minlength=n).to(torch.int32)
    eptr = torch.zeros(n + 1, dtype=torch.int32, device=send.device)
    torch.cumsum(cnt, 0, out=eptr[1:])
    eS = (-unit_shifts[order]).round().to(torch.int32).contiguous() if unit_shifts is not None else \
        torch.zeros(order.numel(), 3, dtype=torch.int32, device=send.device)
    return EdgeCSR(eptr, send[order].to(torch.int32).contiguous(), recv[order].to(torch.int32).contiguous(), eS,
                   None, int(order.numel()))


def _chunks(csr: EdgeCSR, n: int, bytes_per_edge: int, limit: int | None = None) -> list[tuple[int, int, int, int]]:
    """Receiver ranges ``(i0, i1, e0, e1)`` whose radial scratch stays below ``limit`` (default ``CHUNK_BYTES``)."""
    max_edges = max((limit or CHUNK_BYTES) // max(bytes_per_edge, 1), 1024)
    max_edges = min(max_edges, (1 << 30) - 1)  # two rows per edge must stay addressable by 32-bit TMA coordinates
    if csr.num_edges <= max_edges:
        return [(0, n, 0, csr.num_edges)]
    if csr.eptr_host is None:
        csr.eptr_host = csr.eptr.cpu().tolist()  # one host copy per neighbour-list build
    ptr = csr.eptr_host
    out, i0 = [], 0
    import bisect

    while i0 < n:
        i1 = bisect.bisect_right(ptr, ptr[i0] + max_edges, lo=i0 + 1, hi=n + 1) - 1
        i1 = max(i1, i0 + 1)
        out.append((i0, i1, ptr[i0], ptr[i1]))
        i0 = i1
    return out


def _silu_and_grad(a: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    s = torch.sigmoid(a)
    return a * s * SILU_NORM, s * (1.0 + a * (1.0 - s)) * SILU_NORM


def _radial_weights(ws: list[torch.Tensor], ef: torch.Tensor, with_grad: bool) -> torch.Tensor:
    """``ef [E, 1|2, nb]`` → ``[E, 1|2, P*C]``: MLP value and (forward-mode) derivative w.r.t. the distance.

    Value and tangent rows are interleaved ``[E, 2, H]`` so that each layer is one GEMM over ``2E`` rows followed by
    one fused activation kernel; without the tangent the activation runs in the GEMM epilogue."""
    e = ef.shape[0]
    if not with_grad:
        x = ef[:, 0]
        for k, w in enumerate(ws):
            x = gemm.matmul(x, w, act=1 if k < len(ws) - 1 else 0)
        return x.unsqueeze(1)
    xt = ef
    for w in ws[:-1]:
        if w.shape[0] >= 32 and gemm.get_precision() == "tf32":
            xt = gemm.matmul(xt.reshape(2 * e, -1), w, act=2).reshape(e, 2, -1)  # activation + tangent in the epilogue
        else:
            xt = gemm.matmul(xt.reshape(2 * e, -1), w).reshape(e, 2, -1)
            ops.mace_silu_tangent_(xt)
    return gemm.matmul(xt.reshape(2 * e, -1), ws[-1]).reshape(e, 2, -1)


#: run the last radial layer on the tensor cores inside the convolution kernel (radial weights stay in TMEM)
FUSED = True
_err_words: dict[torch.device, torch.Tensor] = {}


def fused_error_status(device: torch.device) -> int:
    """Status word of the fused convolution kernels (0 = no bounded wait expired)."""
    w = _err_words.get(device)
    return 0 if w is None else int(w.item())


def _fused_ok(model: Any, ip: Any) -> bool:
    return (FUSED and gemm.get_precision() == "tf32" and model.config.channels == 128 and ip.radial[-1].shape[0] == 64
            and len(ip.radial) >= 2)


#: run the hidden layers of the radial MLP as one tensor-core kernel (activations never leave the SM)
FUSED_RADIAL = True


def _split_tf32(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``w = hi + lo`` with ``hi`` exactly representable in tf32 (low 13 mantissa bits cleared)."""
    hi = (w.contiguous().view(torch.int32) & -8192).view(torch.float32)
    return hi, w - hi


#: storage of the radial activations kept between the forward pass and its adjoint, reused from step to step (the edge
#: count changes a little every step; asking the allocator for a new ~10 GB block each time would stall it)
_h3_pool: dict[tuple, torch.Tensor] = {}


def _pooled(key: tuple, numel: int, like: torch.Tensor) -> torch.Tensor:
    buf = _h3_pool.get(key)
    if buf is None or buf.numel() < numel or buf.device != like.device:
        buf = None
        _h3_pool.pop(key, None)
        cap = (int(numel * 1.03) + (1 << 22)) // (1 << 22) * (1 << 22)
        buf = _h3_pool[key] = torch.empty(cap, dtype=torch.float32, device=like.device)
    return buf


def release_radial_cache() -> None:
    """Frees the pooled storage of kept radial activations."""
    _h3_pool.clear()


def _hidden_fused(ws: list[torch.Tensor], ef: torch.Tensor, with_grad: bool, out_buf: torch.Tensor | None = None
                  ) -> torch.Tensor | None:
    if not (FUSED_RADIAL and ef.is_cuda and ef.dtype == torch.float32 and gemm.get_precision() == "tf32" and len(ws) == 4
            and tuple(ws[0].shape) == (8, 64) and tuple(ws[1].shape) == (64, 64) and tuple(ws[2].shape) == (64, 64)):
        return None
    hi, lo = _split_tf32(ws[0].t().contiguous())           # [64, 8]
    w1t = torch.zeros(64, 32, dtype=torch.float32, device=ef.device)
    w1t[:, 0:8], w1t[:, 8:16], w1t[:, 16:24] = hi, hi, lo
    err = _err_words.setdefault(ef.device, torch.zeros(1, dtype=torch.int32, device=ef.device))
    rows = ef if with_grad else ef[:, 0]
    out = ops.mace_radial_hidden(rows.reshape(-1, 8).contiguous(), w1t, ws[1].t().contiguous(), ws[2].t().contiguous(),
                                 bool(with_grad), err, out_buf)
    return out.reshape(ef.shape[0], 2, 64) if with_grad else out


def _hidden(ws: list[torch.Tensor], ef: torch.Tensor, with_grad: bool, out_buf: torch.Tensor | None = None) -> torch.Tensor:
    """Radial MLP up to its last hidden layer: ``[E, 64]`` or, with the tangent, ``[E, 2, 64]`` (rows interleaved)."""
    fused = _hidden_fused(ws, ef, with_grad, out_buf)
    if fused is not None:
        return fused
    e = ef.shape[0]
    if not with_grad:
        x = ef[:, 0]
        for w in ws[:-1]:
            x = gemm.matmul(x, w, act=1)
        return x.contiguous()
    xt = ef
    for w in ws[:-1]:
        if w.shape[0] >= 32:
            xt = gemm.matmul(xt.reshape(2 * e, -1), w, act=2).reshape(e, 2, -1)
        else:
            xt = gemm.matmul(xt.reshape(2 * e, -1), w).reshape(e, 2, -1)
            ops.mace_silu_tangent_(xt)
    return xt.contiguous()


def _group_weights(ip: Any, w_last: torch.Tensor, c: int) -> list[torch.Tensor]:
    """Rows of ``W4^T`` ([paths*C, 64]) gathered per path group of the fused kernel."""
    from nvalchemi_toolkit_b200.models.mace import o3

    wt = w_last.t().contiguous().reshape(len(ip.paths), c, -1)
    return [wt[g].reshape(len(g) * c, -1).contiguous() for g in o3.path_groups(ip.l_in)]


#: first interaction in factorised form (``csrc/mace_l0.cu``): per-receiver moments of (harmonic x hidden radial
#: activation) per sender species, then one K = 64 GEMM; used while the number of species keeps the moments small
L0_MOMENTS = os.environ.get("NVA_L0_MOMENTS", "1") != "0"
L0_MOMENTS_MAX_SPECIES = 4
#: when forces are requested, the forward pass evaluates the radial network with its tangent rows and keeps the result
#: ([E, 2, 64] per interaction) for the adjoint instead of running the network twice; used only while it fits easily
RADIAL_CACHE = os.environ.get("NVA_RADIAL_CACHE", "1") != "0"


_free_memory_seen: dict[torch.device, tuple[int, int]] = {}  # device -> (free bytes at the last query, evaluations it stays valid for)


def _radial_cache_fits(dev: torch.device, num_edges: int, layers: int) -> bool:
    if not RADIAL_CACHE or dev.type != "cuda":
        return False
    need = num_edges * 512 * layers
    hit = _free_memory_seen.get(dev)
    if hit is not None and hit[1] > 0 and need < 0.02 * hit[0]:
        # far below the last reading (small batches of an inflight-batching run): the driver query (about a millisecond)
        # is not repeated for every evaluation
        _free_memory_seen[dev] = (hit[0], hit[1] - 1)
        return True
    free, _total = torch.cuda.mem_get_info(dev)
    free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
    free += sum(b.numel() * 4 for b in _h3_pool.values() if b.device == dev)  # storage already set aside for this
    _free_memory_seen[dev] = (free, 256)
    return need < 0.3 * free


def _l0_weights(ip: Any, w_last: torch.Tensor, table: torch.Tensor, c: int, avg: float) -> list[torch.Tensor]:
    """Per ``l`` the ``[species, 64, C]`` matrices that take the moments ``A[i, s, lm, :]`` straight to the message
    ``msg[i, lm, :]``: (last radial layer of path ``l``) x diag(species feature) x (channel mix of ``l``)."""
    from nvalchemi_toolkit_b200.models.mace import o3

    terms = o3.conv_terms(ip.paths, ip.l_in)
    w4 = w_last.reshape(w_last.shape[0], len(ip.paths), c)
    out = []
    for p, (l1, l2, l3) in enumerate(ip.paths):
        assert l1 == 0 and l2 == l3 == p and ip.paths_per_l[l3] == 1
        assert all(a_ == 0 and b_ == l3 * l3 + c_ and abs(coef - terms[p][0][3]) < 1e-12 for (a_, b_, c_, coef) in terms[p])
        lin = ip.linear[l3] / (math.sqrt(c) * avg)
        out.append(torch.stack([(w4[:, p, :] * (terms[p][0][3] * table[s_])) @ lin for s_ in range(table.shape[0])]))
    return out


def _cached(owner: Any, tag: str, params: list[torch.Tensor], build: Any) -> Any:
    """Constants derived from parameters (packed / scaled weight copies, host floats), kept ON the module that owns the
    parameters and rebuilt only when one of them changes (in MD they never do).  The cache lives and dies with its
    module, so two models can never see each other's entries."""
    store = owner.__dict__.setdefault("_nva_derived", {})
    stamp = tuple((p.data_ptr(), p._version, p.device, tuple(p.shape)) for p in params)
    hit = store.get(tag)
    if hit is None or hit[0] != stamp:
        hit = store[tag] = (stamp, build())
    return hit[1]


def _packed(owner: Any, tag: str, params: list[torch.Tensor], build: Any) -> tuple[torch.Tensor, list[int]]:
    """Packed weight matrix (+ first rows of its blocks) of a grouped channel mix, cached on ``owner``."""
    return _cached(owner, "pack:" + tag, params, lambda: gemm.pack_weights([b.detach().contiguous() for b in build()]))


def _rows2d(x: torch.Tensor) -> torch.Tensor:
    """``[N, a, b]`` (rows possibly a slice of a larger buffer) as ``[N, a * b]`` without a copy."""
    return x.reshape(x.shape[0], -1) if x.is_contiguous() else x.contiguous().reshape(x.shape[0], -1)


def _per_l_linear(x: torch.Tensor, w: torch.Tensor, ls: list[int], transpose: bool = False,
                  out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Per-irrep channel mix on ``[N, n_lm, C]``: one grouped GEMM launch, one group per ``lm`` row (reading and writing
    the strided slices in place, no gather / scatter copies), one weight block per ``l``."""
    c = x.shape[-1]
    out = torch.empty_like(x) if out is None else out
    packed, rows = _packed(w, "per_l_t" if transpose else "per_l", [w],  # cached on the parameter object itself
                           lambda: [w[i].t() if transpose else w[i] for i in range(len(ls))])
    groups, off = [], 0
    for i, l in enumerate(ls):
        for m in range(2 * l + 1):
            groups.append(((off + m) * c, c, rows[i], (off + m) * c))
        off += 2 * l + 1
    gemm.grouped(_rows2d(x), packed, out.view(out.shape[0], -1), c, groups, alpha=1.0 / math.sqrt(c), accumulate=accumulate)
    return out


def _skip(ip: Any, h: torch.Tensor, species: torch.Tensor, nz: int, transpose: bool = False,
          accumulate_into: torch.Tensor | None = None) -> torch.Tensor:
    """Element-dependent channel mix ``sc[:, l] = h[:, l] @ W[l, z]`` (or its adjoint).  With ``accumulate_into`` the
    result is added to that tensor (same shape as the result) instead of being returned in a new one."""
    c = h.shape[-1]
    src_ls, dst_ls = (ip.l_out, ip.l_in) if transpose else (ip.l_in, ip.l_out)
    n_dst = sum(2 * l + 1 for l in dst_ls)
    shared = [(i, l) for i, l in enumerate(ip.l_out) if l in ip.l_in]
    if nz == 1:
        full = len(shared) == len(dst_ls)  # every destination irrep is written: no need to clear first
        out = accumulate_into if accumulate_into is not None else \
            (h.new_empty(h.shape[0], n_dst, c) if full else h.new_zeros(h.shape[0], n_dst, c))
        packed, rows = _packed(ip, "skip_t" if transpose else "skip", [ip.skip],
                               lambda: [ip.skip[i, 0].t() if transpose else ip.skip[i, 0] for i, _ in shared])
        groups = []
        for b, (i, l) in enumerate(shared):
            so = sum(2 * k + 1 for k in src_ls[: src_ls.index(l)])
            do = sum(2 * k + 1 for k in dst_ls[: dst_ls.index(l)])
            groups += [((so + m) * c, c, rows[b], (do + m) * c) for m in range(2 * l + 1)]
        if groups:
            gemm.grouped(_rows2d(h), packed, out.view(out.shape[0], -1), c, groups, alpha=1.0 / math.sqrt(c * nz),
                         accumulate=accumulate_into is not None)
        return out
    # several species: one grouped launch per species over ALL rows, selected per row by a mask (no index lists, no host
    # synchronisation; the extra arithmetic is nz small K = C products per row)
    out = accumulate_into if accumulate_into is not None else h.new_zeros(h.shape[0], n_dst, c)
    tmp = h.new_empty(h.shape[0], n_dst, c)
    full = len(shared) == len(dst_ls)
    for z in range(nz):
        packed, rows = _packed(ip, f"skip{z}_t" if transpose else f"skip{z}", [ip.skip],
                               lambda z=z: [ip.skip[i, z].t() if transpose else ip.skip[i, z] for i, _ in shared])
        groups = []
        for b, (i, l) in enumerate(shared):
            so = sum(2 * k + 1 for k in src_ls[: src_ls.index(l)])
            do = sum(2 * k + 1 for k in dst_ls[: dst_ls.index(l)])
            groups += [((so + m) * c, c, rows[b], (do + m) * c) for m in range(2 * l + 1)]
        if not groups:
            break
        if not full:
            tmp.zero_()
        gemm.grouped(_rows2d(h), packed, tmp.view(tmp.shape[0], -1), c, groups, alpha=1.0 / math.sqrt(c * nz))
        out.addcmul_(tmp, (species == z).to(h.dtype)[:, None, None])
    return out


def _linear_mid(ip: Any, mid: torch.Tensor, avg: float, lmax: int) -> torch.Tensor:
    """``mid [N, n_mid, C]`` (components ordered ``(l, m, path)``) → ``msg [N, 16, C]``: one grouped launch, for every
    ``lm`` a product with ``K = paths(l) * C`` straight from the strided slice of ``mid``."""
    n, _, c = mid.shape
    out = mid.new_empty(n, (lmax + 1) ** 2, c)
    packed, rows = _packed(ip, f"mid{avg}", list(ip.linear),
                           lambda: [ip.linear[l] / (math.sqrt(ip.paths_per_l[l] * c) * avg) for l in range(lmax + 1)])
    groups = []
    for l in range(lmax + 1):
        npl = ip.paths_per_l[l]
        groups += [((ip.mid_off[l] + m * npl) * c, npl * c, rows[l], (l * l + m) * c) for m in range(2 * l + 1)]
    gemm.grouped(_rows2d(mid), packed, out.view(n, -1), c, groups)
    return out


def _linear_mid_bwd(ip: Any, dmsg: torch.Tensor, avg: float, lmax: int) -> torch.Tensor:
    n, _, c = dmsg.shape
    dmid = dmsg.new_empty(n, ip.n_mid, c)
    # out[:, o + j*C : o + (j+1)*C] = dmsg[:, lm] @ W_l[j*C:(j+1)*C, :]^T: one weight block of C rows per (l, path slot)
    blocks = [(l, j) for l in range(lmax + 1) for j in range(ip.paths_per_l[l])]
    packed, rows = _packed(ip, f"mid_t{avg}", list(ip.linear),
                           lambda: [(ip.linear[l][j * c: (j + 1) * c] / (math.sqrt(ip.paths_per_l[l] * c) * avg)).t()
                                    for l, j in blocks])
    row_of = {b: r for b, r in zip(blocks, rows)}
    groups = []
    for l in range(lmax + 1):
        npl = ip.paths_per_l[l]
        for m in range(2 * l + 1):
            o = (ip.mid_off[l] + m * npl) * c
            groups += [((l * l + m) * c, c, row_of[(l, j)], o + j * c) for j in range(npl)]
    gemm.grouped(_rows2d(dmsg), packed, dmid.view(n, -1), c, groups)
    return dmid


def _sym_weights(ip: Any, corr: int) -> tuple[torch.Tensor, torch.Tensor | None]:
    packs = []
    for L in ip.l_out:
        packs.append(torch.cat([ip.sym[f"w{nu}_{L}"] for nu in range(1, corr + 1)], dim=1).contiguous())
    return packs[0], (packs[1] if len(packs) > 1 else None)


@torch.no_grad()
def forward(model: Any, data: dict[str, torch.Tensor], species: torch.Tensor, batch: torch.Tensor,
            num_graphs: int, compute_force: bool, compute_stress: bool, dd: Any = None,
            energy_weights: torch.Tensor | None = None
            ) -> dict[str, torch.Tensor | None]:
    """Energy (+ forces, stress) with the native kernels.

    ``dd`` (optional) is a domain-decomposition view: node-level tensors then cover the ``dd.n_owned`` owned atoms,
    ``positions`` additionally holds ghost rows, sender features of ghost atoms are gathered from the owning GPU inside
    the convolution kernels (``dd.home_rank`` / ``dd.home_row`` + peer pointer tables), and the adjoint scatters feature
    and position gradients of ghosts back to their owners with reductions over NVLink.  ``dd.barrier()`` separates the
    phases.  The returned energy is then the partial sum over owned atoms."""
    _native.require(data["positions"])
    cfg = model.config
    pos = data["positions"].detach().contiguous()
    n_local = pos.shape[0]
    n = dd.n_owned if dd is not None else n_local
    dev = pos.device
    cell = data.get("cell")
    if cell is None:
        cell = torch.eye(3, device=dev, dtype=pos.dtype).expand(num_graphs, 3, 3)
    cell = cell.detach().to(pos.dtype).contiguous()
    b32 = batch.to(torch.int32).contiguous()
    sp32 = species.to(torch.int32).contiguous()
    csr = data.get("_csr")
    if csr is None:
        if data.get("neighbor_matrix") is not None:
            csr = build_csr(data["neighbor_matrix"][:n], data["num_neighbors"][:n],
                            None if data.get("neighbor_matrix_shifts") is None else data["neighbor_matrix_shifts"][:n])
        else:
            csr = csr_from_edge_index(data["edge_index"], data.get("unit_shifts"), n)
    C, nz, lmax = cfg.channels, len(cfg.atomic_numbers), cfg.max_ell
    rmax, nb, pc = float(cfg.r_max), cfg.num_bessel, cfg.num_polynomial_cutoff
    geom = (pos, cell, b32, csr.erecv, csr.esend, csr.eS)
    pull = dd is not None and getattr(dd, "prefetch", False)  # ghost rows copied / returned in bulk, kernels stay local
    hr = dd.home_rank if dd is not None and not pull else None
    hw = dd.home_row if dd is not None and not pull else None
    n_rows = dd.n_local if pull else n  # rows of the feature / gradient buffers the kernels see
    used = getattr(dd, "ghost_used", None) if pull else None  # ghost rows that some local edge references
    mark = getattr(dd, "_mark", None) or (lambda name: None)  # optional CUDA-event phase marks of the halo engine
    if dd is not None:
        dd.gpos.zero_()

    h = (model.node_embedding / math.sqrt(nz))[species].unsqueeze(1).contiguous()
    node_e = pos.new_zeros(n)
    saved = []
    keep_h3 = (compute_force or compute_stress) and _radial_cache_fits(dev, csr.num_edges, len(model.interactions))

    def radial_chunks(ws_: list, store: list | None, layer: int) -> Any:
        """Chunks ``(i0, i1, e0, e1, h3 value rows)``; with ``store`` the tangent rows are computed too and kept."""
        for ci, (i0_, i1_, e0_, e1_) in enumerate(_chunks(csr, n, (8 if store is not None else 4) * 64,
                                                          CACHED_CHUNK_BYTES if store is not None else None)):
            ef_ = ops.mace_edge_radial(*geom, e0_, e1_ - e0_, rmax, nb, pc, store is not None)
            buf = _pooled((id(model), dev, layer, ci), (e1_ - e0_) * 128, pos) if store is not None else None
            h3_ = _hidden(ws_, ef_, store is not None, buf)
            del ef_
            if store is not None:
                store.append((i0_, i1_, e0_, e1_, h3_))
                yield i0_, i1_, e0_, e1_, h3_[:, 0]
            else:
                yield i0_, i1_, e0_, e1_, h3_
    for li, ip in enumerate(model.interactions):
        ws = [w / math.sqrt(w.shape[0]) for w in ip.radial]
        P = len(ip.paths)
        sc = _skip(ip, h, species, nz)
        u_ptrs = du = du_ptrs = row_map = None
        # The input of the first interaction is the species embedding: its rows are identical for all atoms of a
        # species.  The fused kernels then read a [species, 1, C] table through a per-atom row map instead of
        # gathering per-atom rows from a multi-hundred-MB array (and no ghost rows have to be exchanged).
        sp_local = species if dd is None else getattr(dd, "species_local", None)
        if li == 0 and ip.l_in == [0] and _fused_ok(model, ip) and sp_local is not None and (dd is None or pull):
            table = model.node_embedding.to(pos.dtype) / math.sqrt(nz)
            u = (table @ (ip.linear_up[0] / math.sqrt(C))).unsqueeze(1).contiguous()
            row_map = sp_local.to(torch.int32).contiguous()
        elif dd is not None:
            u, u_ptrs = dd.feature_buffer(f"u{li}", (n_rows, h.shape[1], C))
            _per_l_linear(h, ip.linear_up, ip.l_in, out=u[:n])
            if li > 0 and compute_force:
                du, du_ptrs = dd.feature_buffer(f"du{li}", (n_rows, h.shape[1], C))
                du.zero_()
            mark("model")
            dd.barrier()  # every rank's u (and zeroed du / gradient buffers) is in place before peers touch it
            if pull:
                ops.halo_pull_rows(u, n, dd.ghost_home_rank, dd.ghost_home_row, None, u_ptrs, used)
                mark("halo_forward")
                pull_ptrs = (u_ptrs, du_ptrs)
                u_ptrs = du_ptrs = None  # the convolution kernels read and write local rows only
        else:
            u = _per_l_linear(h, ip.linear_up, ip.l_in).contiguous()
        fused = _fused_ok(model, ip)
        l0w = None
        if row_map is not None and L0_MOMENTS and nz <= L0_MOMENTS_MAX_SPECIES and lmax == 3 and ws[-1].shape[0] == 64:
            l0_params = [ip.radial[-1], model.node_embedding, ip.linear_up] + list(ip.linear)  # what the folded weights depend on
            l0w = True
            A = pos.new_empty(n, nz, 16, 64)
            h3c = [] if keep_h3 else None
            for (i0, i1, e0, e1, h3) in radial_chunks(ws, h3c, li):
                ops.mace_l0_moments(h3, pos, cell, b32, csr.eptr, csr.esend, csr.eS, row_map, i0, i1 - i0, e0, rmax, A)
                del h3
            msg = pos.new_empty(n, 16, C)
            for s_ in range(nz):  # one grouped launch per sender species (16 products each)
                pk, rws = _packed(ip, f"l0w{s_}", l0_params, lambda s_=s_, ip=ip, ws=ws, u=u: [
                    w_[s_] for w_ in _l0_weights(ip, ws[-1], u[:, 0], C, cfg.avg_num_neighbors)])
                gemm.grouped(A.view(n, -1), pk, msg.view(n, -1), C,
                             [((s_ * 16 + lm) * 64, 64, rws[l], lm * C) for l in range(lmax + 1)
                              for lm in range(l * l, (l + 1) * (l + 1))], accumulate=s_ > 0)
            del A
            wgs, mid = None, None
        elif fused:
            err = _err_words.setdefault(dev, torch.zeros(1, dtype=torch.int32, device=dev))
            wgs = _group_weights(ip, ws[-1], C)
            mid = pos.new_zeros(n, ip.n_mid, C)
            h3c = [] if keep_h3 else None
            for (i0, i1, e0, e1, h3) in radial_chunks(ws, h3c, li):
                for g, wg in enumerate(wgs):
                    ops.mace_conv_fused(0 if ip.l_in == [0] else 1, g, False, wg, h3, u, pos, cell, b32, csr.eptr, csr.esend,
                                        csr.eS, i0, i1 - i0, e0, rmax, mid, None, None, None, hr, hw, u_ptrs, None, None,
                                        err, row_map)
                del h3
        else:
            wgs, h3c = None, None
            mid = pos.new_empty(n, ip.n_mid, C)
            for (i0, i1, e0, e1) in _chunks(csr, n, 4 * P * C):
                ef = ops.mace_edge_radial(*geom, e0, e1 - e0, rmax, nb, pc, False)
                R = _radial_weights(ws, ef, False).reshape(e1 - e0, P, C)
                ops.mace_conv_fwd(u, pos, cell, b32, csr.eptr, csr.esend, csr.eS, R, i0, i1 - i0, e0, rmax, mid, hr, hw,
                                  u_ptrs)
                del ef, R
        if l0w is None:
            msg = _linear_mid(ip, mid, cfg.avg_num_neighbors, lmax)
        del mid
        w0, w1 = _sym_weights(ip, cfg.correlation)
        B = ops.mace_symcon_fwd(msg, sp32, w0, w1, max(ip.l_out), cfg.correlation)
        h_new = _per_l_linear(B, ip.product_linear, ip.l_out, out=sc, accumulate=True)  # skip connection + product mix
        # readout: e_i += w2 . silu(s_i W1) (last layer) or s_i . w1, fused with what the adjoint needs (one kernel)
        rw1 = _cached(ip, "ro_w1", [ip.readout_w1], lambda ip=ip: (ip.readout_w1.detach() / math.sqrt(C)).contiguous())
        rw2 = _cached(ip, "ro_w2", [ip.readout_w2], lambda ip=ip: (ip.readout_w2.detach() / math.sqrt(ip.readout_w2.shape[0]))
                      .contiguous()) if ip.last else None
        gy = ops.mace_readout_fwd(h_new, rw1, rw2, node_e)
        ro = (gy if ip.last else None, rw1)
        saved.append((ip, u, msg, ws, w0, w1, ro, u_ptrs, du, du_ptrs if not (pull and row_map is None) else pull_ptrs[1], wgs,
                      row_map, l0w, h3c))
        h = h_new
        del B, sc
    scale, shift = model.scale.to(pos.dtype), model.shift.to(pos.dtype)
    scale_f = _cached(model, "scale", [model.scale], lambda: float(model.scale))  # host copy for kernel arguments (read once)
    node_e = model.atomic_energies.to(pos.dtype)[species] + node_e * scale + shift
    ew = None if energy_weights is None else energy_weights[:n].to(pos.dtype)
    e_sum = node_e if ew is None else node_e * ew
    if num_graphs == 1:  # one system: a plain float64 sum instead of an indexed accumulation
        energy = e_sum.sum(dtype=torch.float64).reshape(1).to(pos.dtype)
    else:
        energy = torch.zeros(num_graphs, dtype=torch.float64, device=dev).index_add_(0, batch[:n], e_sum.double()).to(pos.dtype)
    out: dict[str, torch.Tensor | None] = {"energy": energy, "node_energy": node_e, "forces": None, "stress": None,
                                            "hessian": None}
    if not (compute_force or compute_stress):
        return out

    grad_pos = dd.gpos if dd is not None else torch.zeros_like(pos)
    fused_forces: torch.Tensor | None = None

    def tangent_chunks(ws_: list, kept: list | None) -> Any:
        """``(i0, i1, e0, e1, h3 [E, 2, 64])``: what the forward pass kept, else recomputed chunk by chunk."""
        if kept is not None:
            while kept:
                yield kept.pop(0)
            return
        for (i0_, i1_, e0_, e1_) in _chunks(csr, n, 8 * 64):
            ef_ = ops.mace_edge_radial(*geom, e0_, e1_ - e0_, rmax, nb, pc, True)
            h3_ = _hidden(ws_, ef_, True)
            del ef_
            yield i0_, i1_, e0_, e1_, h3_
    gp_ptrs = dd.gpos_ptrs if dd is not None and not pull else None
    strain_grad = torch.zeros(num_graphs, 9, dtype=torch.float64, device=dev) if compute_stress else None
    dh: torch.Tensor | None = None
    for li in range(len(saved) - 1, -1, -1):
        ip, u, msg, ws, w0, w1, ro, u_ptrs, du, du_ptrs, wgs, row_map, l0w, h3c = saved[li]
        k_du_ptrs = None if pull else du_ptrs  # pointer table handed to the kernels (none: local rows only)
        n_out = sum(2 * l + 1 for l in ip.l_out)
        dh_tot = pos.new_zeros(n, n_out, C) if dh is None else dh
        ops.mace_readout_bwd(ro[0], ro[1], scale_f, None if ew is None else ew.contiguous(), dh_tot)
        dB = _per_l_linear(dh_tot, ip.product_linear, ip.l_out, transpose=True).contiguous()
        dmsg = ops.mace_symcon_bwd(msg, sp32, w0, w1, max(ip.l_out), cfg.correlation, dB)
        del dB
        dmid = _linear_mid_bwd(ip, dmsg, cfg.avg_num_neighbors, lmax) if l0w is None else None
        P = len(ip.paths)
        if dd is None:
            du = torch.zeros_like(u) if li > 0 else None
        if l0w is not None:
            Q = pos.new_empty(n, nz, 16, 64)
            l0_params = [ip.radial[-1], model.node_embedding, ip.linear_up] + list(ip.linear)
            pk, rws = _packed(ip, "l0w_t", l0_params, lambda ip=ip, ws=ws, u=u: [
                w_[s_].t() for s_ in range(nz) for w_ in _l0_weights(ip, ws[-1], u[:, 0], C, cfg.avg_num_neighbors)])
            gemm.grouped(_rows2d(dmsg), pk, Q.view(n, -1), 64,
                         [(lm * C, C, rws[s_ * (lmax + 1) + l], (s_ * 16 + lm) * 64) for s_ in range(nz)
                          for l in range(lmax + 1) for lm in range(l * l, (l + 1) * (l + 1))])
            for (i0, i1, e0, e1, h3) in tangent_chunks(ws, h3c):
                ops.mace_l0_force(h3, Q, pos, cell, b32, csr.eptr, csr.esend, csr.eS, row_map, i0, i1 - i0, e0, rmax,
                                  grad_pos, strain_grad)
                del h3
            del Q
        elif wgs is not None:
            err = _err_words[dev]
            for (i0, i1, e0, e1, h3) in tangent_chunks(ws, h3c):
                for g, wg in enumerate(wgs):
                    ops.mace_conv_fused(0 if ip.l_in == [0] else 1, g, True, wg, h3, u, pos, cell, b32, csr.eptr, csr.esend,
                                        csr.eS, i0, i1 - i0, e0, rmax, dmid, du, grad_pos, strain_grad, hr, hw, u_ptrs,
                                        k_du_ptrs, gp_ptrs, err, row_map)
                del h3
        else:
            for (i0, i1, e0, e1) in _chunks(csr, n, 8 * P * C):
                ef = ops.mace_edge_radial(*geom, e0, e1 - e0, rmax, nb, pc, True)
                RD = _radial_weights(ws, ef, True).reshape(e1 - e0, 2, P, C)
                ops.mace_conv_bwd(u, dmid, pos, cell, b32, csr.eptr, csr.esend, csr.eS, RD, i0, i1 - i0, e0, rmax, du,
                                  grad_pos, strain_grad, hr, hw, u_ptrs, k_du_ptrs, gp_ptrs)
                del ef, RD
        del dmid, dmsg
        if pull:
            # return what was accumulated on ghost rows to the owners, once per row
            mark("model")
            dd.barrier()  # owners finished their own accumulation, holders finished theirs on the ghost copies
            if getattr(dd, "reverse_pull", False):
                rev = (dd.send_row, dd.send_peer, dd.send_peer_row)
                if li > 0:
                    ops.halo_pull_add_rows(du, *rev, du_ptrs, dd.used_ptrs, dd.send_used_index)
                if li == 0 and getattr(dd, "fused_force_return", False) and hasattr(dd, "copy_ptr"):
                    # reverse halo of the position gradient fused with its consumers: forces and, when the integrator's
                    # closing update is the plain half kick, the velocities (one pass, one thread per owned atom)
                    fused_forces = torch.empty(n, 3, dtype=grad_pos.dtype, device=dev)
                    fin = getattr(dd, "fused_finalize", None)
                    ops.halo_force_finalize(grad_pos, dd.copy_ptr, dd.copy_peer, dd.copy_row, dd.copy_used_index, dd.gpos_ptrs,
                                            dd.used_ptrs, fused_forces, *(fin if fin is not None else (None, None, None, None)))
                elif li == 0:
                    ops.halo_pull_add_rows(grad_pos, *rev, dd.gpos_ptrs, dd.used_ptrs, dd.send_used_index)
            else:
                if li > 0:
                    ops.halo_push_add_rows(du, n, dd.ghost_home_rank, dd.ghost_home_row, du_ptrs, used)
                if li == 0:
                    ops.halo_push_add_rows(grad_pos[:dd.n_local], n, dd.ghost_home_rank, dd.ghost_home_row, dd.gpos_ptrs, used)
        if dd is not None:
            dd.barrier()  # feature / position gradients pushed by peers have landed
            mark("halo_reverse")
        if li > 0 and dd is not None:
            du = du[:n]
        if li > 0 and wgs is not None:
            # the fused kernel accumulates the feature gradient as [row, channel, component] (vector reductions)
            du = du.view(du.shape[0], C, du.shape[1]).transpose(1, 2).contiguous()
        if li > 0:
            dh = _per_l_linear(du, ip.linear_up, ip.l_in, transpose=True)
            _skip(ip, dh_tot, species, nz, transpose=True, accumulate_into=dh)
        saved[li] = None
    out["forces"] = fused_forces if fused_forces is not None else -grad_pos[:n]
    if compute_stress:
        vol = torch.linalg.det(cell).abs().double()
        sg = strain_grad.reshape(num_graphs, 3, 3)
        sg = 0.5 * (sg + sg.transpose(-1, -2))
        out["stress"] = (sg / vol[:, None, None]).to(pos.dtype)
        out["virial"] = (-sg).to(pos.dtype)
    return out
