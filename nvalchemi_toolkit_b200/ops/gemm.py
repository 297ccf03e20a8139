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


def check_errors(like: torch.Tensor) -> int:
    """Status word of the GEMM kernels on ``like``'s device (0 = fine; non-zero = a bounded wait expired)."""
    if like.is_cuda and _native.available():
        return int(_nops.gemm_error_status(like))
    return 0
