# SPDX-License-Identifier: Apache-2.0
"""O(3) building blocks of the native MACE: real spherical harmonics, Clebsch-Gordan tensors and the
symmetric-contraction basis, all for ``l <= 3``.

Nothing here depends on e3nn or cuEquivariance (the reference gets these pieces from
``mace-torch``/``e3nn``; see ``nvalchemi/models/mace.py:518-560``).  Conventions:

* real spherical harmonics in the standard ``m = -l..l`` order with the z axis as polar axis,
  *component* normalisation (``sum_m Y_lm^2 = 2l+1`` on the unit sphere); parity of ``Y_l`` is ``(-1)^l``;
* a feature row is ``[lm, channel]`` with ``lm = l^2 + l + m`` (16 components for ``l <= 3``);
* the coupling tensor of a path ``(l1, l2 -> l3)`` is the rotation-invariant element of
  ``l1 x l2 x l3`` (unique up to scale), scaled to Frobenius norm ``sqrt(2 l3 + 1)``;
* the symmetric-contraction basis of degree ``nu`` and output ``L`` spans all equivariant homogeneous
  polynomial maps of degree ``nu`` from the 16-component feature to ``L`` with parity ``(-1)^L``.

Tables are derived numerically in float64 (invariance under sampled rotations + inversion) by
:func:`generate_tables`, stored in ``tables.npz`` beside this file and exported to
``csrc/mace_tables.h`` for the CUDA kernels, so every code path shares the same numbers.
"""
from __future__ import annotations

import functools
import itertools
import os

import numpy as np
import torch

LMAX = 3
NLM = (LMAX + 1) ** 2
_HERE = os.path.dirname(os.path.abspath(__file__))
TABLE_FILE = os.path.join(_HERE, "tables.npz")


def lm_slice(l: int) -> slice:
    return slice(l * l, (l + 1) * (l + 1))


# --------------------------------------------------------------------------- spherical harmonics
def spherical_harmonics(vec: torch.Tensor, lmax: int = LMAX, normalize: bool = True) -> torch.Tensor:
    """Real SH ``[..., (lmax+1)^2]`` of ``vec [..., 3]`` (component normalisation)."""
    if normalize:
        vec = vec / vec.norm(dim=-1, keepdim=True).clamp_min(1e-30)
    x, y, z = vec.unbind(-1)
    out = [torch.ones_like(x)]
    if lmax >= 1:
        s3 = 3.0 ** 0.5
        out += [s3 * y, s3 * z, s3 * x]
    if lmax >= 2:
        s15, s5 = 15.0 ** 0.5, 5.0 ** 0.5
        out += [s15 * x * y, s15 * y * z, 0.5 * s5 * (3 * z * z - (x * x + y * y + z * z)), s15 * x * z,
                0.5 * s15 * (x * x - y * y)]
    if lmax >= 3:
        r2 = x * x + y * y + z * z
        s70, s105, s42, s7 = 70.0 ** 0.5, 105.0 ** 0.5, 42.0 ** 0.5, 7.0 ** 0.5
        out += [0.25 * s70 * y * (3 * x * x - y * y), s105 * x * y * z, 0.25 * s42 * y * (5 * z * z - r2),
                0.5 * s7 * z * (5 * z * z - 3 * r2), 0.25 * s42 * x * (5 * z * z - r2),
                0.5 * s105 * z * (x * x - y * y), 0.25 * s70 * x * (x * x - 3 * y * y)]
    if lmax >= 4:
        raise NotImplementedError("spherical harmonics are implemented for l <= 3")
    return torch.stack(out, dim=-1)


def _sh_np(v: np.ndarray) -> np.ndarray:
    return spherical_harmonics(torch.from_numpy(v), LMAX, normalize=True).numpy()


def _random_rotation(rng: np.random.Generator) -> np.ndarray:
    q, r = np.linalg.qr(rng.normal(size=(3, 3)))
    q = q * np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


def wigner_D(R: np.ndarray) -> np.ndarray:
    """Block-diagonal ``[16,16]`` representation matrix ``D`` with ``Y(R v) = D Y(v)`` (proper or improper R)."""
    rng = np.random.default_rng(12345)
    v = rng.normal(size=(64, 3))
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    y0, y1 = _sh_np(v), _sh_np(v @ R.T)
    D = np.zeros((NLM, NLM))
    for l in range(LMAX + 1):
        s = lm_slice(l)
        sol, *_ = np.linalg.lstsq(y0[:, s], y1[:, s], rcond=None)  # y1 = y0 @ sol -> D = sol^T
        D[s, s] = sol.T
    return D


def _group_samples(n: int = 6, seed: int = 7) -> list[np.ndarray]:
    rng = np.random.default_rng(seed)
    mats = [_random_rotation(rng) for _ in range(n)]
    mats.append(-np.eye(3))  # inversion fixes the parity
    return [wigner_D(R) for R in mats]


def _null_space(A: np.ndarray, tol: float = 1e-9) -> np.ndarray:
    _, s, vt = np.linalg.svd(A, full_matrices=True)
    rank = int((s > tol * max(1.0, s[0] if s.size else 1.0)).sum())
    return vt[rank:].T  # columns span the null space


def _fix_sign(t: np.ndarray) -> np.ndarray:
    flat = t.reshape(-1)
    k = int(np.argmax(np.abs(flat) > 1e-9))
    return t if flat[k] > 0 else -t


def clebsch_gordan(l1: int, l2: int, l3: int, Ds: list[np.ndarray] | None = None) -> np.ndarray | None:
    """Invariant tensor ``C[m1,m2,m3]`` with Frobenius norm ``sqrt(2 l3+1)``; ``None`` when the path is
    forbidden (triangle rule or parity ``(-1)^(l1+l2+l3) != 1``)."""
    if not (abs(l1 - l2) <= l3 <= l1 + l2) or (l1 + l2 + l3) % 2:
        return None
    Ds = Ds or _group_samples()
    d1, d2, d3 = 2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1
    rows = []
    eye = np.eye(d1 * d2 * d3)
    for D in Ds:
        a, b, c = D[lm_slice(l1), lm_slice(l1)], D[lm_slice(l2), lm_slice(l2)], D[lm_slice(l3), lm_slice(l3)]
        rows.append(np.kron(np.kron(a, b), c) - eye)
    ns = _null_space(np.concatenate(rows, 0))
    if ns.shape[1] != 1:
        raise RuntimeError(f"CG({l1},{l2},{l3}): expected a 1-dimensional invariant space, got {ns.shape[1]}")
    C = _fix_sign(ns[:, 0].reshape(d1, d2, d3))
    C = C / np.linalg.norm(C) * np.sqrt(d3)
    C[np.abs(C) < 1e-12] = 0.0
    return C


def conv_paths(l_in: list[int], l_sh_max: int = LMAX, l_out_max: int = LMAX) -> list[tuple[int, int, int]]:
    """Natural-parity tensor-product paths ``(l1, l2 -> l3)``, ordered by ``(l3, l1, l2)``."""
    paths = [(l1, l2, l3) for l3 in range(l_out_max + 1) for l1 in l_in for l2 in range(l_sh_max + 1)
             if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0]
    return paths


# --------------------------------------------------------------------------- symmetric contraction basis
def _monomials(nu: int) -> list[tuple[int, ...]]:
    return list(itertools.combinations_with_replacement(range(NLM), nu))


def _l_of(i: int) -> int:
    return int(np.floor(np.sqrt(i)))


def symmetric_basis(nu: int, L: int, Ds: list[np.ndarray] | None = None) -> tuple[list[tuple[int, ...]], np.ndarray]:
    """Basis of equivariant degree-``nu`` polynomial maps 16 -> (2L+1).

    Returns ``(monomials, U)`` with ``U [n_basis, 2L+1, n_monomials]``: ``P_eta,M(x) = sum_t U[eta,M,t] prod_{i in
    monomials[t]} x_i``.  The space is split by the multiset of ``l`` values of the factors, so every basis
    element only touches monomials of one ``l``-type (sparse tables)."""
    Ds = Ds or _group_samples()
    monos = _monomials(nu)
    index = {m: t for t, m in enumerate(monos)}
    types: dict[tuple[int, ...], list[int]] = {}
    for t, m in enumerate(monos):
        types.setdefault(tuple(sorted(_l_of(i) for i in m)), []).append(t)
    rng = np.random.default_rng(99)
    dL = 2 * L + 1
    basis: list[np.ndarray] = []
    for ltype, tidx in sorted(types.items()):
        if (sum(ltype) + L) % 2:  # parity of the monomial must match (-1)^L
            continue
        if not _can_couple(ltype, L):
            continue
        nt = len(tidx)
        pts = rng.normal(size=(max(3 * nt, 24), NLM))
        sub = [monos[t] for t in tidx]

        def mono_vals(x: np.ndarray) -> np.ndarray:
            return np.stack([np.prod(x[:, list(m)], axis=1) for m in sub], axis=1)  # [S, nt]

        m0 = mono_vals(pts)
        rows = []
        for D in Ds:
            m1 = mono_vals(pts @ D.T)  # monomials at the rotated point
            DL = D[lm_slice(L), lm_slice(L)]
            # unknown T[M, t]; constraint: sum_t T[M,t] m1[s,t] - sum_M' DL[M,M'] sum_t T[M',t] m0[s,t] = 0
            A = np.zeros((pts.shape[0], dL, dL, nt))
            for M in range(dL):
                A[:, M, M, :] += m1
                A[:, M, :, :] -= DL[M, :, None][None] * m0[:, None, :]
            rows.append(A.reshape(pts.shape[0] * dL, dL * nt))
        ns = _null_space(np.concatenate(rows, 0), tol=1e-8)
        for k in range(ns.shape[1]):
            T = np.zeros((dL, len(monos)))
            T[:, tidx] = ns[:, k].reshape(dL, nt)
            basis.append(T)
    del index
    if not basis:
        return monos, np.zeros((0, dL, len(monos)))
    U = np.stack(basis, 0)
    # canonical scale: unit mean-square output for unit-normal inputs, estimated by sampling
    x = rng.normal(size=(4096, NLM))
    mv = np.stack([np.prod(x[:, list(m)], axis=1) for m in monos], axis=1)
    val = np.einsum("emt,st->sem", U, mv)
    scale = np.sqrt((val ** 2).mean(axis=(0, 2)))
    U = U / scale[:, None, None]
    for e in range(U.shape[0]):
        U[e] = _fix_sign(U[e])
    U[np.abs(U) < 1e-10] = 0.0
    return monos, U


def _can_couple(ls: tuple[int, ...], L: int) -> bool:
    reach = {ls[0]}
    for l in ls[1:]:
        reach = {k for a in reach for k in range(abs(a - l), a + l + 1)}
    return L in reach


# --------------------------------------------------------------------------- table generation / loading
def generate_tables(path: str = TABLE_FILE, header: str | None = None) -> dict[str, np.ndarray]:
    """Derive all tables, save them to ``path`` and (optionally) write the C header for the kernels."""
    Ds = _group_samples()
    out: dict[str, np.ndarray] = {}
    for l1 in range(LMAX + 1):
        for l2 in range(LMAX + 1):
            for l3 in range(LMAX + 1):
                C = clebsch_gordan(l1, l2, l3, Ds)
                if C is not None:
                    out[f"cg_{l1}{l2}{l3}"] = C
    for L in (0, 1):
        for nu in (1, 2, 3):
            monos, U = symmetric_basis(nu, L, Ds)
            out[f"sym_mono_{nu}"] = np.asarray(monos, dtype=np.int64)
            out[f"sym_U_{nu}_{L}"] = U
    np.savez_compressed(path, **out)
    load_tables.cache_clear()
    if header:
        write_header(header)
    return out


@functools.lru_cache(maxsize=1)
def load_tables() -> dict[str, np.ndarray]:
    if not os.path.exists(TABLE_FILE):
        generate_tables()
    with np.load(TABLE_FILE) as f:
        return {k: f[k] for k in f.files}


def cg(l1: int, l2: int, l3: int, dtype: torch.dtype = torch.float64, device: torch.device | str = "cpu") -> torch.Tensor:
    return torch.as_tensor(load_tables()[f"cg_{l1}{l2}{l3}"], dtype=dtype, device=device)


def conv_terms(paths: list[tuple[int, int, int]], l_in: list[int]) -> list[list[tuple[int, int, int, float]]]:
    """Per path: sparse list of ``(in_comp, sh_comp, m3, coef)``; ``in_comp`` indexes the concatenated input
    irreps ``l_in`` (0e -> 0; 0e+1o -> 0..3), ``sh_comp`` is the ``lm`` index of the harmonic."""
    in_off = {l: sum(2 * k + 1 for k in l_in[: l_in.index(l)]) for l in l_in}
    t = load_tables()
    out = []
    for (l1, l2, l3) in paths:
        C = t[f"cg_{l1}{l2}{l3}"]
        terms = [(in_off[l1] + a, l2 * l2 + b, c, float(C[a, b, c])) for a in range(2 * l1 + 1)
                 for b in range(2 * l2 + 1) for c in range(2 * l3 + 1) if C[a, b, c] != 0.0]
        out.append(terms)
    return out


def mid_layout(paths: list[tuple[int, int, int]], l_out_max: int = LMAX) -> tuple[list[int], list[int], int]:
    """Layout of the aggregated message ``mid [N, n_mid, C]``: components are ordered ``(l3, m3, path-within-l3)``
    so that for a fixed ``(l3, m3)`` all paths are contiguous (the K axis of the following channel mix).

    Returns ``(l3_offset[l3], paths_per_l3[l3], n_mid)``."""
    npl = [sum(1 for p in paths if p[2] == l) for l in range(l_out_max + 1)]
    offs, acc = [], 0
    for l in range(l_out_max + 1):
        offs.append(acc)
        acc += (2 * l + 1) * npl[l]
    return offs, npl, acc


def sym_terms(nu: int, L: int) -> tuple[int, list[tuple[int, int, tuple[int, ...], float]]]:
    """``(n_basis, [(eta, M, monomial, coef), ...])`` sorted by ``(eta, M)``."""
    t = load_tables()
    monos, U = t[f"sym_mono_{nu}"], t[f"sym_U_{nu}_{L}"]
    terms = []
    for e in range(U.shape[0]):
        for M in range(U.shape[1]):
            nz = np.nonzero(U[e, M])[0]
            terms.extend((e, M, tuple(int(i) for i in monos[k]), float(U[e, M, k])) for k in nz)
    return int(U.shape[0]), terms


def path_groups(l_in: list[int]) -> list[list[int]]:
    """Split of the tensor-product paths into groups whose last-layer radial weights ([paths*C, 64] fp32) fit in the
    shared memory of one CTA of the fused convolution kernel (at most 5 paths = 160 KB).  Groups are balanced by the
    number of coupling terms."""
    paths = conv_paths(l_in)
    if len(paths) <= 5:
        return [list(range(len(paths)))]
    terms = conv_terms(paths, l_in)
    order = sorted(range(len(paths)), key=lambda p: -len(terms[p]))
    groups: list[list[int]] = [[], []]
    load = [0, 0]
    for p in order:
        g = 0 if (load[0] <= load[1] and len(groups[0]) < 5) or len(groups[1]) >= 5 else 1
        groups[g].append(p)
        load[g] += len(terms[p])
    return [sorted(g) for g in groups]


def write_header(path: str) -> None:
    """Emit ``mace_tables.h``: unrolled tensor-product bodies and symmetric-contraction term tables."""
    lines = ["// SPDX-License-Identifier: Apache-2.0",
             "// GENERATED by nvalchemi_toolkit_b200.models.mace.o3.write_header -- do not edit.",
             "// Coupling tables of the native MACE kernels (real SH, z polar axis, m=-l..l, component norm).",
             "#pragma once", ""]
    for tag, l_in in (("L0", [0]), ("L1", [0, 1])):
        paths = conv_paths(l_in)
        terms = conv_terms(paths, l_in)
        offs, npl, nmid = mid_layout(paths)
        nin = sum(2 * l + 1 for l in l_in)
        seen = [0] * (LMAX + 1)
        out_index = []
        for (l1, l2, l3) in paths:
            k = seen[l3]
            seen[l3] += 1
            out_index.append([offs[l3] + m3 * npl[l3] + k for m3 in range(2 * l3 + 1)])
        lines += [f"// ---- input irreps {l_in}: {len(paths)} paths {paths}",
                  f"#define MACE_{tag}_NIN {nin}", f"#define MACE_{tag}_NPATH {len(paths)}",
                  f"#define MACE_{tag}_NMID {nmid}",
                  f"#define MACE_{tag}_NTERMS {sum(len(t) for t in terms)}"]
        # forward: acc[o] += R[p] * sum coef*h[a]*Y[b]
        body = []
        for p, tl in enumerate(terms):
            by_out: dict[int, list[str]] = {}
            for (a, b, c, coef) in tl:
                by_out.setdefault(out_index[p][c], []).append(f"{coef:.9e}f*h[{a}]*Y[{b}]")
            for o, exprs in by_out.items():
                body.append(f"  acc[{o}] = fmaf(R[{p}], {' + '.join(exprs)}, acc[{o}]);")
        lines += [f"#define MACE_{tag}_FWD(h, Y, R, acc) do {{ \\"] + [b + " \\" for b in body] + ["} while (0)", ""]
        # backward, two stages.  Per receiver: T[(p,a,b)] = sum_c coef[a,b,c] * G[out(p,c)] (G is shared by all edges
        # of the receiver).  Per edge and path: A_a = sum_b T_ab Y_b;  S_p = sum_a h_a A_a;  dh_a += R_p A_a;
        # dY_b += R_p sum_a T_ab h_a.
        prep, edge, k = [], [], 0
        for p, tl in enumerate(terms):
            pairs: dict[tuple[int, int], list[str]] = {}
            for (a, b, c, coef) in tl:
                pairs.setdefault((a, b), []).append(f"{coef:.9e}f*G[{out_index[p][c]}]")
            tindex = {}
            for (a, b), exprs in pairs.items():
                prep.append(f"  T[{k}] = {' + '.join(exprs)};")
                tindex[(a, b)] = k
                k += 1
            edge.append(f"  {{ float s_ = 0.f, v_; const float r_ = R[{p}];")
            for a in sorted({ab[0] for ab in tindex}):
                expr = " + ".join(f"T[{tindex[(a, b)]}]*Y[{b}]" for (aa, b) in tindex if aa == a)
                edge.append(f"    v_ = {expr}; s_ = fmaf(h[{a}], v_, s_); dh[{a}] = fmaf(r_, v_, dh[{a}]);")
            for b in sorted({ab[1] for ab in tindex}):
                expr = " + ".join(f"T[{tindex[(a, bb)]}]*h[{a}]" for (a, bb) in tindex if bb == b)
                edge.append(f"    v_ = {expr}; dY[{b}] = fmaf(r_, v_, dY[{b}]);")
            edge.append(f"    S[{p}] = s_; }}")
        lines += [f"#define MACE_{tag}_NT {k}",
                  f"#define MACE_{tag}_BWD_PREP(G, T) do {{ \\"] + [t + " \\" for t in prep] + ["} while (0)"]
        lines += [f"#define MACE_{tag}_BWD_EDGE(h, Y, R, T, dh, dY, S) do {{ \\"] + [t + " \\" for t in edge] + \
                 ["} while (0)", ""]
    # ---- per-group variants for the fused (tensor-core radial weights in TMEM) convolution kernel.  Local path index q
    # runs over the group's paths; accumulators / gradients are compacted to the group's mid components.
    for tag, l_in in (("L0", [0]), ("L1", [0, 1])):
        paths = conv_paths(l_in)
        terms = conv_terms(paths, l_in)
        offs, npl, nmid = mid_layout(paths)
        seen = [0] * (LMAX + 1)
        out_index = []
        for (l1, l2, l3) in paths:
            k = seen[l3]
            seen[l3] += 1
            out_index.append([offs[l3] + m3 * npl[l3] + k for m3 in range(2 * l3 + 1)])
        for gi, grp in enumerate(path_groups(l_in)):
            gt = f"{tag}G{gi}"
            mids = sorted({o for p in grp for o in out_index[p]})
            loc = {o: k for k, o in enumerate(mids)}
            lines += [f"// ---- {gt}: paths {grp} -> {len(mids)} mid components",
                      f"#define MACE_{gt}_NP {len(grp)}", f"#define MACE_{gt}_NACC {len(mids)}",
                      f"#define MACE_{gt}_PATHS {{{', '.join(str(p) for p in grp)}}}",
                      f"#define MACE_{gt}_MIDS {{{', '.join(str(o) for o in mids)}}}"]
            body = []
            for q, p in enumerate(grp):
                by_out: dict[int, list[str]] = {}
                for (a_, b_, c_, coef) in terms[p]:
                    by_out.setdefault(loc[out_index[p][c_]], []).append(f"{coef:.9e}f*h[{a_}]*Y[{b_}]")
                for o, exprs in by_out.items():
                    body.append(f"  acc[{o}] = fmaf(R[{q}], {' + '.join(exprs)}, acc[{o}]);")
            lines += [f"#define MACE_{gt}_FWD(h, Y, R, acc) do {{ \\"] + [t + " \\" for t in body] + ["} while (0)"]
            # forward with the channel-independent factors hoisted: Z[k] = coef * Y[b] is prepared once per edge, the
            # per-channel work is one multiply-add per coupling term
            # per channel: a = R[q] * h[a_] once per (path, input component), then one multiply-add per coupling term
            zprep, zbody, kz = [], [], 0
            for q, p in enumerate(grp):
                zbody.append("  { " + " ".join(f"const float a{a_}_ = R[{q}]*h[{a_}];"
                                               for a_ in sorted({t[0] for t in terms[p]})))
                for (a_, b_, c_, coef) in terms[p]:
                    zprep.append(f"  Z[{kz}] = {coef:.9e}f*Y[{b_}];")
                    o = loc[out_index[p][c_]]
                    zbody.append(f"    acc[{o}] = fmaf(a{a_}_, Z[{kz}], acc[{o}]);")
                    kz += 1
                zbody.append("  }")
            lines += [f"#define MACE_{gt}_NZ {kz}",
                      f"#define MACE_{gt}_ZPREP(Y, Z) do {{ \\"] + [t + " \\" for t in zprep] + ["} while (0)"]
            lines += [f"#define MACE_{gt}_FWDZ(h, Z, R, acc) do {{ \\"] + [t + " \\" for t in zbody] + ["} while (0)"]
            prep, edge, k = [], [], 0
            for q, p in enumerate(grp):
                pairs: dict[tuple[int, int], list[str]] = {}
                for (a_, b_, c_, coef) in terms[p]:
                    pairs.setdefault((a_, b_), []).append(f"{coef:.9e}f*G[{loc[out_index[p][c_]]}]")
                tindex = {}
                for (a_, b_), exprs in pairs.items():
                    prep.append(f"  T[{k}] = {' + '.join(exprs)};")
                    tindex[(a_, b_)] = k
                    k += 1
                edge.append(f"  {{ float s_ = 0.f, v_; const float r_ = R[{q}];")
                for a_ in sorted({ab[0] for ab in tindex}):
                    expr = " + ".join(f"T[{tindex[(a_, b_)]}]*Y[{b_}]" for (aa, b_) in tindex if aa == a_)
                    edge.append(f"    v_ = {expr}; s_ = fmaf(h[{a_}], v_, s_); dh[{a_}] = fmaf(r_, v_, dh[{a_}]);")
                # dY_b += sum_a T_ab * (r h_a): the product r h_a is formed once per input component
                edge.append("    " + " ".join(f"const float a{a_}_ = r_*h[{a_}];" for a_ in sorted({ab[0] for ab in tindex})))
                for (a_, b_), ti in tindex.items():
                    edge.append(f"    dY[{b_}] = fmaf(T[{ti}], a{a_}_, dY[{b_}]);")
                edge.append(f"    S[{q}] = s_; }}")
            lines += [f"#define MACE_{gt}_NT {k}",
                      f"#define MACE_{gt}_BWD_PREP(G, T) do {{ \\"] + [t + " \\" for t in prep] + ["} while (0)"]
            lines += [f"#define MACE_{gt}_BWD_EDGE(h, Y, R, T, dh, dY, S) do {{ \\"] + [t + " \\" for t in edge] + \
                     ["} while (0)", ""]
    # symmetric contraction: straight-line polynomial evaluation (x[16], gradients dx[16] live in registers).
    # W(k) must expand to the weight of basis element k of the (nu, L) block for the thread's (element, channel).
    for L in (0, 1):
        for nu in (1, 2, 3):
            nb, terms = sym_terms(nu, L)
            lines.append(f"#define MACE_SYM_{nu}_{L}_NBASIS {nb}")
            groups: dict[tuple[int, int], list[tuple[tuple[int, ...], float]]] = {}
            for (e, M, mono, coef) in terms:
                groups.setdefault((e, M), []).append((mono, coef))
            fwd, bwd = [], []
            for (e, M), tl in groups.items():
                expr = " + ".join(f"{coef:.9e}f*" + "*".join(f"x[{i}]" for i in mono) for mono, coef in tl)
                fwd.append(f"  out[{M}] = fmaf(W({e}), {expr}, out[{M}]);")
                # adjoint of one (basis element, output component) block: d/dx_a of every monomial, merged per target a
                # and per remaining factor product, so that a term costs one fma on a product x_b*x_c that the compiler
                # can share between blocks (the parenthesised product is the same expression everywhere)
                bwd.append(f"  {{ const float s_ = W({e})*g[{M}]; float t_;")
                per_target: dict[int, dict[tuple[int, ...], float]] = {}
                for mono, coef in tl:
                    for q in range(len(mono)):
                        rest = tuple(sorted(i for k, i in enumerate(mono) if k != q))
                        acc = per_target.setdefault(mono[q], {})
                        acc[rest] = acc.get(rest, 0.0) + coef
                for a_, rests in sorted(per_target.items()):
                    items = [(r_, c_) for r_, c_ in sorted(rests.items()) if c_ != 0.0]
                    if not items:
                        continue
                    if len(items[0][0]) == 0:      # nu = 1: the derivative is the coefficient itself
                        bwd.append(f"    dx[{a_}] = fmaf(s_, {items[0][1]:.9e}f, dx[{a_}]);")
                        continue
                    prod = lambda r_: "(" + "*".join(f"x[{i}]" for i in r_) + ")"  # noqa: E731
                    bwd.append(f"    t_ = {items[0][1]:.9e}f*{prod(items[0][0])};")
                    for r_, c_ in items[1:]:
                        bwd.append(f"    t_ = fmaf({c_:.9e}f, {prod(r_)}, t_);")
                    bwd.append(f"    dx[{a_}] = fmaf(s_, t_, dx[{a_}]);")
                bwd.append("  }")
            lines += [f"#define MACE_SYM_FWD_{nu}_{L}(x, out) do {{ \\"] + [t + " \\" for t in fwd] + ["} while (0)"]
            lines += [f"#define MACE_SYM_BWD_{nu}_{L}(x, g, dx) do {{ \\"] + [t + " \\" for t in bwd] + ["} while (0)", ""]
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    csrc = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "csrc", "mace_tables.h")
    generate_tables(header=csrc)
    tb = load_tables()
    print({k: v.shape for k, v in tb.items() if k.startswith("sym_U")})
