"""Host-side failure detection for tensor-parallel ranks.

Every rank bumps a counter in a shared key-value store once per serving step; before launching the
next step a rank checks that every peer has reached a recent step. A peer that stopped (crashed,
was killed, hangs in host code) is reported as :class:`PeerFailure` *before* any kernel that would
wait for it is launched, so no GPU ever spins on a dead partner. On the device side every wait on a
peer flag is bounded anyway (collectives.cu) and ends in a status code that
:func:`nanoflow_b200.ops.check_status` turns into an exception.

The reference has no failure handling: its cross-GPU waits spin without bound and a dead peer hangs
every GPU (pipeline/src/comm.cu, pipeline/include/networkManager.cuh:19-28).
"""
from __future__ import annotations

import time
from typing import Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, last_step: int, wanted: int):
        super().__init__(f"rank {rank} stopped at step {last_step} (needed step {wanted})")
        self.rank, self.last_step, self.wanted = rank, last_step, wanted


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, poll_s: float = 0.01,
                 prefix: str = "nf_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix
        self.step = 0
        for r in range(world):
            self.store.add(f"{prefix}/{r}", 0)          # create the counters

    def _read(self, r: int) -> int:
        return int(self.store.add(f"{self.prefix}/{r}", 0))

    def beat(self) -> int:
        """Announce that this rank is about to run its next step."""
        self.step = int(self.store.add(f"{self.prefix}/{self.rank}", 1))
        return self.step

    def check(self, timeout_s: Optional[float] = None) -> None:
        """Raise PeerFailure unless every peer has announced the step this rank announced."""
        deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                v = self._read(r)
                if v >= self.step:
                    break
                if time.monotonic() > deadline:
                    raise PeerFailure(r, v, self.step)
                time.sleep(self.poll_s)

    def leave(self) -> None:
        """Mark this rank as gone on purpose (tests use it to simulate a rank that stops between steps)."""
        self.store.set(f"{self.prefix}/left/{self.rank}", "1")
