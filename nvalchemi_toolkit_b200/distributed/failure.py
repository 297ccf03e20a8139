# SPDX-License-Identifier: Apache-2.0
"""Host-side failure detection for multi-rank runs.

The reference has no elastic recovery; its safety net is join timeouts in test harnesses and hooks that stop a run
(``test/distributed/_gloo_harness.py:139-172``, ``dynamics/hooks/safety.py``).  Here every rank can publish a heartbeat
in the process group's key-value store between steps and check its peers' before launching the next collective, so
a rank that raised, exited or stalled is noticed on the host instead of inside a device-side wait; device-side waits
are bounded anyway and report through a status word (``P2PContext.status``).  Recovery is restart from a checkpoint.
"""
from __future__ import annotations

import time
from typing import Any, Callable

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks: list[int], reason: str) -> None:
        super().__init__(f"ranks {ranks} {reason}")
        self.ranks = ranks


class HeartbeatMonitor:
    """``beat(step)`` publishes this rank's progress; ``check(step)`` raises :class:`PeerFailure` when a peer has
    announced a failure or has not reached ``step - max_lag`` within ``timeout`` seconds."""

    def __init__(self, store: Any, rank: int, world_size: int, timeout: float = 5.0, max_lag: int = 0,
                 prefix: str = "nva_hb") -> None:
        self.store, self.rank, self.world, self.timeout, self.max_lag, self.prefix = store, rank, world_size, timeout, max_lag, prefix
        self.store.set(f"{prefix}/{rank}", "-1")

    @classmethod
    def from_env(cls, timeout: float = 5.0, **kw: Any) -> "HeartbeatMonitor":
        """Uses the default process group's store (``torch.distributed`` must be initialised)."""
        store = dist.distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout, **kw)

    def beat(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", str(int(step)))

    def fail(self, reason: str) -> None:
        """Announce that this rank is leaving (call from an exception handler, between steps)."""
        self.store.set(f"{self.prefix}/{self.rank}", f"failed:{reason[:200]}")

    def _read(self, r: int) -> str:
        return self.store.get(f"{self.prefix}/{r}").decode()

    def check(self, step: int) -> None:
        deadline = time.monotonic() + self.timeout
        need = int(step) - self.max_lag
        while True:
            late, failed = [], []
            for r in range(self.world):
                if r == self.rank:
                    continue
                v = self._read(r)
                if v.startswith("failed:"):
                    failed.append(r)
                elif int(v) < need:
                    late.append(r)
            if failed:
                raise PeerFailure(failed, "announced a failure")
            if not late:
                return
            if time.monotonic() > deadline:
                raise PeerFailure(late, f"did not reach step {need} within {self.timeout} s")
            time.sleep(0.01)


def guarded_run(step_fn: Callable[[int], None], n_steps: int, monitor: HeartbeatMonitor,
                pre_step: Callable[[int], None] | None = None,
                on_failure: Callable[[PeerFailure], None] | None = None, check_every: int = 1) -> int:
    """Run ``step_fn(step)`` ``n_steps`` times with a host-side readiness handshake in front of every ``check_every``-th
    step: a rank first runs its own ``pre_step`` checks (NaN guards, user callbacks), then publishes "ready for step i"
    and waits until every peer is ready too.  A rank whose ``pre_step`` raises announces the failure instead, so its
    peers stop on the host *before* they launch kernels or collectives that would wait for it.  A failure in the middle
    of ``step_fn`` is outside this protocol: bounded device waits and the process-group timeout end it.  Returns the
    number of completed steps."""
    done = 0
    for step in range(n_steps):
        try:
            if pre_step is not None:
                pre_step(step)
        except Exception as exc:
            monitor.fail(repr(exc))
            raise
        if step % max(1, check_every) == 0:
            monitor.beat(step)
            try:
                monitor.check(step)
            except PeerFailure as exc:
                if on_failure is not None:
                    on_failure(exc)
                    return done
                raise
        step_fn(step)
        done += 1
    return done
