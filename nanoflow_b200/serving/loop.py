"""The serving loop: trace -> scheduler -> engine, with the CPU one step ahead of the GPU.

Per cycle (``bench_text_gen`` in the reference, pipeline/utils/serve_8B.py:348-569):

1. release requests whose arrival time has passed (wall clock, or simulated time);
2. ``schedule()`` the next dense batch and allocate its KV pages while the GPU runs the previous one;
3. ``update`` + ``run_async``: stage metadata and launch iteration *i* behind iteration *i-1*;
4. ``run_async_wait`` for iteration *i-1* and hand its tokens to ``process_outputs``.

``skip_cycles`` advances the scheduler without touching the engine (token values zero), the
reference's way of reaching the steady-state batch mix before timing (serve_8B.py:657-662).
Throughput is counted like the reference: retired requests x (avg prompt + avg output) per second of
host wall clock (serve_8B.py:686-697, :755-761); per-iteration processed tokens are also kept.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .frontend import RequestManager
from .request import FlyRequestInfo
from .scheduler import BatchPlan, Scheduler


@dataclass
class LoopStats:
    cycles: int = 0
    wall_seconds: float = 0.0
    tokens_processed: int = 0            # dense-batch tokens executed (prefill + decode)
    retired: List[FlyRequestInfo] = field(default_factory=list)
    cycle_tokens: List[int] = field(default_factory=list)

    @property
    def retired_tokens(self) -> int:
        return sum(r.input_len + len(r.output) for r in self.retired)


class ServingLoop:
    def __init__(self, engine, scheduler: Scheduler, request_manager: RequestManager, *,
                 simulated_time: bool = True, est_cycle_time: float = 0.175, offload=None, health=None,
                 trace_phases: bool = False):
        """``trace_phases``: put a named range (NVTX + profiler) around every phase of a cycle: schedule,
        update, launch, wait_previous, process_outputs."""
        import contextlib

        from ..utils.nvtx import nvtx_range
        self._phase = nvtx_range if trace_phases else (lambda name: contextlib.nullcontext())
        self.engine, self.scheduler, self.rm = engine, scheduler, request_manager
        self.simulated_time = simulated_time
        self.est_cycle_time = est_cycle_time
        self.offload = offload
        self.health = health      # parallel.health.Heartbeat: peers are checked before every launch
        self._prev: Optional[BatchPlan] = None
        self.failed: Optional[Exception] = None     # set by _abandon when a peer failure stopped the loop
        self.stats = LoopStats()

    def _release(self) -> None:
        if self.simulated_time:
            self.rm.simulate_issue(self.est_cycle_time)
        else:
            self.rm.issue()

    def skip_cycles(self, n: int) -> int:
        """Scheduler-only cycles (no GPU work). Returns the number of cycles actually advanced."""
        done = 0
        for _ in range(n):
            self.rm.simulate_issue(self.est_cycle_time)
            plan = self.scheduler.schedule()
            if plan is None:
                if not self.scheduler.has_work:
                    break
                continue
            self.scheduler.process_outputs(plan, None)
            self.scheduler.release_held_pages(plan.iteration)
            done += 1
        self.scheduler.drain_retired()
        return done

    def step(self) -> Optional[BatchPlan]:
        """One cycle. Returns the plan that was launched (None if there was nothing to run)."""
        phase = self._phase
        self._release()
        with phase("schedule"):
            plan = self.scheduler.schedule()
        if self.health is not None:
            self.health.beat()
            try:
                self.health.check()    # raises PeerFailure before anything that waits on a peer is launched
            except Exception as failure:
                self._abandon(plan, failure)
                raise
        if plan is not None:
            with phase("update"):
                self.engine.update(plan)
            with phase("launch"):
                self.engine.run_async()
            if self.offload is not None:
                self.offload.on_iteration(plan)
        if self._prev is not None:
            with phase("wait_previous"):
                tokens = self.engine.run_async_wait()
            with phase("process_outputs"):
                self.scheduler.process_outputs(self._prev, tokens)
            if self.offload is not None:
                self.offload.on_complete(self._prev, self.scheduler)
            self.stats.tokens_processed += self._prev.num_tokens
            self.stats.cycle_tokens.append(self._prev.num_tokens)
        self._prev = plan
        self.stats.cycles += 1
        self.stats.retired.extend(self.scheduler.drain_retired())
        return plan

    def _abandon(self, plan: Optional[BatchPlan], failure: Exception) -> None:
        """A peer is gone: nothing new is launched. The iteration still in flight is waited for (its device
        waits are bounded, so this returns) and its tokens are dropped, every running request gives its
        pages back and returns to the head of the request queue (``Scheduler.requeue_running``), and the
        failure carries what was saved (``failure.requeued``, ``failure.retired``) to the caller, who can
        serve the queue again with a re-formed group. The plan scheduled in this cycle was never launched."""
        if self._prev is not None:
            try:
                self.engine.run_async_wait()
            except RuntimeError:
                pass          # a bounded device wait ran out on the way: expected when the peer died mid-iteration
            self._prev = None
        failure.requeued = self.scheduler.requeue_running()
        self.stats.retired.extend(self.scheduler.drain_retired())
        failure.retired = len(self.stats.retired)
        self.failed = failure

    def drain(self) -> None:
        if self._prev is not None:
            tokens = self.engine.run_async_wait()
            self.scheduler.process_outputs(self._prev, tokens)
            if self.offload is not None:
                self.offload.on_complete(self._prev, self.scheduler)
            self.stats.tokens_processed += self._prev.num_tokens
            self.stats.cycle_tokens.append(self._prev.num_tokens)
            self._prev = None
        self.stats.retired.extend(self.scheduler.drain_retired())

    def run(self, max_cycles: Optional[int] = None, until_empty: bool = True) -> LoopStats:
        t0 = time.perf_counter()
        n = 0
        while (max_cycles is None or n < max_cycles):
            if until_empty and not self.scheduler.has_work and self.rm.full_request_queue.size == 0 \
                    and self.rm.avaliable_request_queue.size == 0:
                break
            plan = self.step()
            n += 1
            if plan is None and self._prev is None and self.rm.full_request_queue.size == 0 \
                    and self.rm.avaliable_request_queue.size == 0 and not self.scheduler.has_work:
                break
        self.drain()
        # one more schedule() so requests whose last token just arrived are retired
        self.scheduler.schedule() if not self.scheduler.has_work else None
        self.stats.retired.extend(self.scheduler.drain_retired())
        self.stats.wall_seconds += time.perf_counter() - t0
        return self.stats
