# SPDX-License-Identifier: Apache-2.0
"""Symmetric memory arenas and the peer-to-peer context used by the fused communication kernels.

One arena = one allocation of ``torch.distributed._symmetric_memory`` per rank, made with identical sizes on every
rank and exchanged once (``rendezvous``); sub-buffers are carved out with identical offsets everywhere, so the address
of a peer's sub-buffer is ``peer_base + offset`` and no further handshakes are needed.  Kernels receive the table of
peer addresses as an ``int64[world]`` device tensor and touch peer memory with plain loads, stores and reductions
over NVLink (never with TMA).

The reference has no counterpart: all its communication goes through ``torch.distributed`` collectives
(``nvalchemi/distributed/_core/gather_primitives.py``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


class SymmetricArena:
    """Bump allocator over a peer-mapped buffer.  All ranks must perform the same sequence of ``alloc`` calls."""

    def __init__(self, nbytes: int, device: torch.device, group: dist.ProcessGroup | None = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)  # 0: no NVLS multicast for this buffer
        self.offset = 0
        self.buf.zero_()

    def alloc(self, shape: tuple[int, ...], dtype: torch.dtype = torch.float32) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(local view, int64[world] device tensor with every rank's address of the same sub-buffer)``."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = (self.offset + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {off + nbytes} bytes, have {self.nbytes}")
        self.offset = off + nbytes
        view = self.buf[off: off + nbytes].view(dtype).reshape(shape)
        ptrs = torch.tensor([b + off for b in self.base_ptrs], dtype=torch.int64, device=self.device)
        return view, ptrs

    def offset_of(self, view: torch.Tensor) -> int:
        """Byte offset of a sub-buffer returned by :meth:`alloc` inside the arena."""
        return int(view.data_ptr() - self.buf.data_ptr())

    def reset(self) -> None:
        self.offset = 0


class _LocalArena:
    """Stand-in for :class:`SymmetricArena` inside ONE process: ``world`` plain device buffers play the ranks' arenas.
    Nothing ever writes the other "ranks'" flags, so every rendezvous runs into its bounded wait: this is how the
    time-out path is exercised on a single GPU without any peer."""

    def __init__(self, nbytes: int, device: torch.device, world: int) -> None:
        self.world, self.rank, self.device, self.group = world, 0, device, None
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self._bufs = [torch.zeros(self.nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.buf = self._bufs[0]
        self.base_ptrs = [int(b.data_ptr()) for b in self._bufs]
        self.multicast_ptr = 0
        self.offset = 0

    alloc = SymmetricArena.alloc
    offset_of = SymmetricArena.offset_of
    reset = SymmetricArena.reset


class P2PContext:
    """Arena + flag-based barrier with a bounded wait and a status word.

    The status word lives on the device; :meth:`post_status` mirrors it into pinned host memory without blocking and
    :meth:`check` raises :class:`~nvalchemi_toolkit_b200.distributed.failure.PeerFailure` once a mirrored value is
    non-zero, so that a peer that missed a rendezvous stops the run instead of letting later kernels work on incomplete
    buffers."""

    def __init__(self, arena_bytes: int, device: torch.device, group: dist.ProcessGroup | None = None,
                 _arena: object | None = None) -> None:
        self.arena = _arena if _arena is not None else SymmetricArena(arena_bytes + 4096, device, group)
        self.world, self.rank, self.device = self.arena.world, self.arena.rank, device
        self.flags, self.flag_ptrs = self.arena.alloc((64,), torch.int32)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self._err_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._err_event: torch.cuda.Event | None = None
        self.epoch = 0
        self.persistent_offset = self.arena.offset
        torch.cuda.synchronize(device)
        if _arena is None:
            dist.barrier(self.arena.group)

    @classmethod
    def single_process(cls, arena_bytes: int, device: torch.device, world: int = 2) -> "P2PContext":
        """A context whose peers are plain buffers of this process and never arrive at a barrier (time-out tests)."""
        return cls(arena_bytes, device, _arena=_LocalArena(arena_bytes + 4096, device, world))

    def post_status(self) -> None:
        """Start a non-blocking copy of the status word to the host (read later by :meth:`check`)."""
        self._err_host.copy_(self.err, non_blocking=True)
        self._err_event = torch.cuda.Event()
        self._err_event.record()

    def check(self, wait: bool = False) -> None:
        """Raise ``PeerFailure`` if the last posted status word reports an expired wait.  ``wait=False`` looks only at a
        copy that has already arrived (no host synchronisation); ``wait=True`` posts a fresh copy and waits for it."""
        from nvalchemi_toolkit_b200.distributed.failure import PeerFailure

        if wait:
            self.post_status()
        if self._err_event is None or (not wait and not self._err_event.query()):
            return
        self._err_event.synchronize()
        code = int(self._err_host[0])
        if code:
            raise PeerFailure([code - 100], f"did not reach a device-side rendezvous of rank {self.rank} within its bounded wait")

    def barrier(self) -> None:
        """Device-side rendezvous on the current stream: orders this rank's earlier peer writes before the peers'
        later reads.  A peer that does not arrive within about a second sets ``status()`` instead of hanging."""
        self.epoch += 1
        _nops.p2p_barrier(self.flag_ptrs, self.rank, self.world, self.epoch, self.err)

    def status(self) -> int:
        return int(self.err.item())

    def allreduce_(self, view: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None,
                   use_multimem: bool | None = None, check: str | None = "lazy", ptrs: torch.Tensor | None = None
                   ) -> torch.Tensor:
        """Sum a symmetric sub-buffer over all ranks (times ``scale``).

        With an NVLS multicast mapping the reduction runs in the switch (``multimem.ld_reduce`` / ``multimem.st``, each
        rank reducing one slice) and the result is left IN PLACE in every rank's buffer; otherwise every rank reads all
        peers' buffers and writes ``out``.  Both are bracketed by flag barriers with bounded waits.

        ``check``: ``"sync"`` reads the status word after the closing barrier (one host synchronisation) and raises
        ``PeerFailure`` before the result can be used; ``"lazy"`` (default) raises at the NEXT call for a wait that
        expired in this one (no synchronisation: the status travels through pinned memory), i.e. one reduction may be
        consumed before the failure surfaces; ``None`` leaves the status to the caller."""
        import os

        if check == "lazy":
            self.check(wait=False)
        n = view.numel()
        if view.dtype not in (torch.float32, torch.float64):
            raise TypeError(f"allreduce_ sums float32 or float64 buffers, got {view.dtype}")
        if view.dtype == torch.float64:
            use_multimem = False  # the in-switch path is written for float4 groups; doubles use ordered peer loads
        if use_multimem is None:
            use_multimem = self.arena.multicast_ptr != 0 and n % 4 == 0 and os.environ.get("NVA_MULTIMEM", "1") != "0"
        self.barrier()
        if use_multimem:
            _nops.multimem_allreduce(self.arena.multicast_ptr, self.arena.offset_of(view), n, self.rank, self.world,
                                     float(scale), view)
            result = view
        else:
            if ptrs is None:  # callers on a hot path pass the table of peer addresses they built once
                ptrs = torch.tensor([b + self.arena.offset_of(view) for b in self.arena.base_ptrs], dtype=torch.int64,
                                    device=self.device)
            result = out if out is not None else torch.empty_like(view)
            _nops.p2p_allreduce(ptrs, self.world, float(scale), result)
        self.barrier()
        if check == "sync":
            self.check(wait=True)
        elif check == "lazy":
            self.post_status()
        return result

    def release_transient(self) -> None:
        self.arena.offset = self.persistent_offset


class PeerReducer:
    """In-place sum of a tensor over the ranks of a group through peer memory: callable ``reducer(t) -> t``.

    Used where a model needs a GLOBAL sum in the middle of its evaluation (structure factors and charge meshes of the
    Ewald / particle-mesh models under domain decomposition, float64): the tensor is copied into a symmetric scratch
    buffer, a flag barrier orders the copies, every rank adds up all ranks' buffers in rank order with 16-byte peer
    loads (:func:`p2p_allreduce`) straight into ``t``, and a closing barrier keeps a fast rank from overwriting its
    scratch buffer while a slow one still reads it.  Payloads up to ``SMALL_BYTES`` (structure factors, net charges,
    dipoles: latency-bound) take ONE launch instead of four: ``p2p_allreduce_push`` stores the values into every rank's
    slot, publishes a flag per block, waits for the peers' flags and adds its local slots; two slot sets alternate so no
    closing rendezvous is needed.  The fixed order makes the result bitwise identical on every rank,
    which keeps replicated follow-up work (the reciprocal-space virial) in step.  Tensors that are not float32 / float64
    CUDA tensors, or larger than the scratch buffer, go through ``torch.distributed.all_reduce``."""

    SMALL_BYTES = 256 << 10  # payloads up to this size take the single-launch push kernel

    def __init__(self, group: dist.ProcessGroup | None, device: torch.device, capacity_bytes: int = 64 << 20,
                 _context: "P2PContext | None" = None) -> None:
        self.group, self.device, self.capacity = group, device, int(capacity_bytes)
        world = _context.world if _context is not None else dist.get_world_size(group)
        small = 2 * world * self.SMALL_BYTES + 16 * 32 * 4 + 1024
        self.ctx = _context if _context is not None else P2PContext(self.capacity + small, device, group)
        self.scratch, self.ptrs = self.ctx.arena.alloc((self.capacity,), torch.uint8)
        # single-launch path: [parity][rank][SMALL_BYTES] slots and a [block][rank] flag row per rank
        self.push_scratch, self.push_ptrs = self.ctx.arena.alloc((2 * world * self.SMALL_BYTES,), torch.uint8)
        self.push_flags, self.push_flag_ptrs = self.ctx.arena.alloc((16 * 32,), torch.int32)
        self.push_epoch = 0
        self.ctx.persistent_offset = self.ctx.arena.offset
        self.calls = 0      # reductions done through peer memory
        self.small_calls = 0  # ... of which by the single-launch kernel
        self.fallbacks = 0  # ... through the library collective

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        nbytes = t.numel() * t.element_size()
        if not t.is_cuda or t.dtype not in (torch.float32, torch.float64) or nbytes > self.capacity or nbytes == 0:
            self.fallbacks += 1
            if self.ctx.world > 1 and dist.is_initialized():
                dist.all_reduce(t, group=self.group)
            return t
        flat = t if t.is_contiguous() else t.contiguous()
        if nbytes <= self.SMALL_BYTES:
            # one kernel: push my values into every rank's slot, flag, wait for the peers' flags, add the local slots
            self.push_epoch += 1
            _nops.p2p_allreduce_push(flat.reshape(-1), self.push_ptrs, self.SMALL_BYTES // t.element_size(), self.push_flag_ptrs,
                                     self.ctx.rank, self.ctx.world, self.push_epoch, 1.0, self.ctx.err, flat.reshape(-1))
            if flat is not t:
                t.copy_(flat)
            self.calls += 1
            self.small_calls += 1
            return t
        view = self.scratch[:nbytes].view(t.dtype)
        view.copy_(flat.reshape(-1))
        out = flat.reshape(-1)
        if out.data_ptr() % 16:  # a slice of a larger tensor: reduce into an aligned temporary
            out = torch.empty_like(view)
        self.ctx.allreduce_(view, out=out, use_multimem=False, ptrs=self.ptrs)
        if out.data_ptr() != t.data_ptr() or flat is not t:
            t.copy_(out.reshape(t.shape))
        self.calls += 1
        return t


_REDUCERS: dict[tuple[int, int], "PeerReducer | None"] = {}


def peer_reducer(group: dist.ProcessGroup | None, device: torch.device) -> "PeerReducer | None":
    """The group's shared :class:`PeerReducer` (created on first use: a collective, so every rank of the group must ask
    in the same place), or ``None`` where peer memory is not an option: CPU tensors, a backend other than NCCL, or
    ``NVA_PEER_REDUCE=0``."""
    import os

    if device.type != "cuda" or not dist.is_initialized() or os.environ.get("NVA_PEER_REDUCE", "1") == "0":
        return None
    g = group if group is not None else dist.group.WORLD
    if "nccl" not in str(dist.get_backend(g)):
        return None
    key = (id(g), device.index if device.index is not None else torch.cuda.current_device())
    if key not in _REDUCERS:
        _REDUCERS[key] = PeerReducer(g, device)
    return _REDUCERS[key]
