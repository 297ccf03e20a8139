# SPDX-License-Identifier: Apache-2.0
"""Row-copy primitives behind ``Batch.put`` / ``defrag`` / ``index_select``.

These replace the reference's 26 Warp buffer kernels
(``nvalchemi/data/buffer_kernels.py:58-1741``) with three primitives:
``expand_segments`` (segment list → element indices), ``copy_rows`` (gather rows
of one tensor into given rows of another) and ``compact_rows`` (in-place
forward compaction, safe because kept indices are sorted and destinations never
exceed sources).  CUDA tensors use the extension's kernels (any dtype, copied
as raw bytes, 16-byte vectorised when the row size allows); CPU tensors use
vectorised torch indexing.
"""
from __future__ import annotations

import torch

from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


def expand_segments(starts: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    """``concat_i arange(starts[i], starts[i]+lens[i])`` as int64."""
    lens = lens.long()
    starts = starts.long()
    total = int(lens.sum())
    if total == 0:
        return starts.new_zeros(0)
    if starts.is_cuda and _native.require(starts):
        return _nops.expand_segments(starts, lens, total)
    excl = torch.cumsum(lens, 0) - lens
    base = torch.repeat_interleave(starts - excl, lens, output_size=total)
    return base + torch.arange(total, device=starts.device)


def copy_rows(src: torch.Tensor, src_rows: torch.Tensor, dst: torch.Tensor, dst_rows: torch.Tensor) -> None:
    """``dst[dst_rows] = src[src_rows]`` (row-wise, dtype-preserving, no host sync)."""
    if src_rows.numel() == 0:
        return
    if dst.dtype != src.dtype:
        src = src.to(dst.dtype)
    if dst.is_cuda and _native.require(dst) and src.is_contiguous() and dst.is_contiguous():
        _nops.copy_rows(src, src_rows.long(), dst, dst_rows.long())
        return
    dst[dst_rows] = src[src_rows]


def compact_rows(buf: torch.Tensor, keep: torch.Tensor, dst_rows: torch.Tensor, num_live: int) -> None:
    """Move rows ``keep`` (sorted ascending) to ``dst_rows`` (= 0..n-1) and zero the vacated tail."""
    n = int(keep.numel())
    if n:
        if buf.is_cuda and _native.require(buf) and buf.is_contiguous():
            tmp = torch.empty((n,) + tuple(buf.shape[1:]), dtype=buf.dtype, device=buf.device)
            _nops.copy_rows(buf, keep.long(), tmp, dst_rows.long())
            buf[:n].copy_(tmp)
        else:
            buf[:n] = buf[keep]
    if num_live > n:
        buf[n:num_live].zero_()
