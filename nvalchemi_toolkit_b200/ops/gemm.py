# SPDX-License-Identifier: Apache-2.0
"""Dense channel mixes: ``x @ w`` routed to the hand-written tcgen05/TMEM TF32 GEMM.

``matmul(x [..., K], w [K, N])`` flattens the leading axes.  On CUDA float32 inputs with TMA-compatible
shapes (``K % 4 == 0``, ``K >= 32``) the product runs on ``_nops.gemm_tf32`` (TF32 inputs, FP32
accumulation in tensor memory); other cases use ``torch.matmul``.  ``set_precision("fp32")`` forces the exact
FP32 library path everywhere (used by numerics tests that need tight tolerances against an FP64 oracle).
"""
from __future__ import annotations

import torch

from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops

_precision = "tf32"
_counters = {"tcgen05": 0, "library": 0}


def set_precision(mode: str) -> None:
    global _precision
    if mode not in ("tf32", "fp32"):
        raise ValueError("precision must be 'tf32' or 'fp32'")
    _precision = mode


def get_precision() -> str:
    return _precision


def launch_counts() -> dict[str, int]:
    return dict(_counters)


def _eligible(x2: torch.Tensor, k: int) -> bool:
    return (_precision == "tf32" and x2.is_cuda and x2.dtype == torch.float32 and k >= 32 and k % 4 == 0
            and x2.shape[0] > 0 and _native.available())


def _tma_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 4 == 0 and t.data_ptr() % 16 == 0


def matmul(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0, act: int = 0, out: torch.Tensor | None = None
           ) -> torch.Tensor:
    """``act(alpha * x @ w)``; ``act``: 0 none, 1 SiLU scaled to unit second moment, 2 the same for rows that
    alternate (value, tangent): even rows get ``silu(a)``, odd rows ``silu'(a_even) * t``.

    ``x`` may be a strided 2-D view (rows ``stride(0)`` apart, unit inner stride) and ``out`` a strided 2-D view: both
    are addressed in place by the TMA descriptors / the epilogue, so slices of wider feature tensors need no copies."""
    k, n = w.shape
    lead = x.shape[:-1]
    x2 = x if x.dim() == 2 else x.reshape(-1, k)
    if _eligible(x2, k):
        if not _tma_ok(x2):
            x2 = x2.contiguous()
        wt = w.t().contiguous()  # [N, K], K-major B operand; weights are small
        _counters["tcgen05"] += 1
        if out is not None and out.dim() == 2 and out.stride(1) == 1:
            _nops.gemm_tf32_out(x2, wt, float(alpha), int(act), out)
            return out
        res = _nops.gemm_tf32(x2, wt, float(alpha), int(act)).reshape(*lead, n)
        if out is not None:
            out.copy_(res)
            return out
        return res
    _counters["library"] += 1
    res = torch.matmul(x2, w)
    if alpha != 1.0:
        res = res * alpha
    if act == 1:
        res = torch.nn.functional.silu(res) * 1.6790176868438721
    elif act == 2:  # rows alternate (value, tangent)
        a, t = res[0::2], res[1::2]
        s = torch.sigmoid(a)
        res = torch.stack([a * s, s * (1.0 + a * (1.0 - s)) * t], dim=1).reshape(res.shape) * 1.6790176868438721
    res = res.reshape(*lead, n)
    if out is not None:
        out.copy_(res)
        return out
    return res


def pack_weights(blocks: list[torch.Tensor]) -> tuple[torch.Tensor, list[int]]:
    """Stack weight blocks ``w_i [K_i, N]`` as K-major rows ``[sum N, K_max]`` (zero padded); returns the packed matrix
    and the first row of every block.  The result is what :func:`grouped` takes as ``packed``."""
    n = blocks[0].shape[1]
    kmax = max(int(b.shape[0]) for b in blocks)
    out = blocks[0].new_zeros(len(blocks) * n, kmax)
    rows = []
    for i, b in enumerate(blocks):
        out[i * n: (i + 1) * n, : b.shape[0]] = b.t()
        rows.append(i * n)
    return out, rows


def grouped(a: torch.Tensor, packed: torch.Tensor, out: torch.Tensor, n_cols: int, groups: list[tuple[int, int, int, int]],
            alpha: float = 1.0, act: int = 0, accumulate: bool = False) -> torch.Tensor:
    """Many slice products in one launch: for every ``(a_col, k, b_row, c_col)`` of ``groups``

        ``out[:, c_col : c_col + n_cols] (+)= act(alpha * a[:, a_col : a_col + k] @ packed[b_row : b_row + n_cols, :k].T)``

    ``a`` and ``out`` are 2-D (unit inner stride); ``packed`` comes from :func:`pack_weights`.  CUDA float32 inputs in
    TF32 mode run as ONE tcgen05 kernel whose tile scheduler walks (row tile, group, column tile); anything else runs the
    same products one by one through ``torch.matmul``."""
    if (_precision == "tf32" and a.is_cuda and a.dtype == torch.float32 and a.shape[0] > 0 and _native.available()
            and _tma_ok(a) and out.stride(1) == 1 and all(g[1] % 32 == 0 and g[0] % 4 == 0 for g in groups)):
        for i in range(0, len(groups), 64):
            part = groups[i: i + 64]
            _counters["tcgen05"] += 1
            _nops.gemm_tf32_grouped(a, packed, out, int(n_cols), [g[0] for g in part], [g[1] for g in part],
                                    [g[2] for g in part], [g[3] for g in part], float(alpha), int(act), bool(accumulate))
        return out
    for a_col, k, b_row, c_col in groups:
        _counters["library"] += 1
        res = a[:, a_col: a_col + k] @ packed[b_row: b_row + n_cols, :k].t()
        if alpha != 1.0:
            res = res * alpha
        if act == 1:
            res = torch.nn.functional.silu(res) * 1.6790176868438721
        elif act != 0:
            raise ValueError("grouped: only act 0 and 1 are supported")
        dst = out[:, c_col: c_col + n_cols]
        if accumulate:
            dst += res
        else:
            dst.copy_(res)
    return out


def check_errors(like: torch.Tensor) -> int:
    """Status word of the GEMM kernels on ``like``'s device (0 = fine; non-zero = a bounded wait expired)."""
    if like.is_cuda and _native.available():
        return int(_nops.gemm_error_status(like))
    return 0
