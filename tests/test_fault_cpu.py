"""Failure detection without any GPU: ranks are CPU processes that share a TCPStore.

* a rank that stops between steps is detected by the others before their next launch (PeerFailure);
* a rank that never joins is detected the same way;
* KV exhaustion, bad configs and bad traces surface as typed errors (covered in the other CPU tests).
"""
import multiprocessing as mp
import time
from datetime import timedelta

import pytest

from nanoflow_b200.parallel.health import Heartbeat, PeerFailure


def _rank(rank, world, port, die_at, never_join, q):
    from torch.distributed import TCPStore

    try:
        if never_join and rank == never_join:
            time.sleep(0.2)
            q.put((rank, "absent", 0))
            return
        store = TCPStore("127.0.0.1", port, world_size=None, is_master=(rank == 0), timeout=timedelta(seconds=60),
                         wait_for_workers=False)
        hb = Heartbeat(store, rank, world, timeout_s=1.5)
        # Process start-up (interpreter + torch import) can differ by seconds between ranks on a busy
        # machine; the ranks that do take part meet here first so that the 1.5 s heartbeat timeout
        # measures a missing peer, not a slow import.
        present = world - (1 if never_join else 0)
        store.add("present", 1)
        t0 = time.monotonic()
        while int(store.add("present", 0)) < present:
            if time.monotonic() - t0 > 60:
                raise RuntimeError("start-up rendezvous timed out")
            time.sleep(0.01)
        for step in range(1, 8):
            if die_at is not None and rank == 1 and step == die_at:
                q.put((rank, "left", step))            # leaves between steps: nothing of its own in flight
                return
            hb.beat()
            hb.check()
            time.sleep(0.01)                           # the step's work
        q.put((rank, "done", 7))
        if rank == 0:
            time.sleep(1.0)                            # keep the store alive until the others have finished
    except PeerFailure as e:
        q.put((rank, "peer_failure", e.rank, e.last_step))
        if rank == 0:
            time.sleep(1.0)


def _free_port() -> int:
    import socket

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _run(world, port=None, die_at=None, never_join=None):
    port = port or _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, port, die_at, never_join, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    return {o[0]: o[1:] for o in out}


def test_all_ranks_healthy():
    res = _run(3)
    assert all(v[0] == "done" for v in res.values())


def test_rank_leaving_between_steps_is_detected_before_next_launch():
    res = _run(3, die_at=4)
    assert res[1][0] == "left"
    for r in (0, 2):
        assert res[r][0] == "peer_failure" and res[r][1] == 1 and res[r][2] == 3   # rank 1 stopped after step 3


def test_rank_that_never_joins_is_detected():
    res = _run(3, never_join=2)
    assert res[2][0] == "absent"
    for r in (0, 1):
        assert res[r][0] == "peer_failure" and res[r][1] == 2 and res[r][2] == 0


def test_serving_loop_gives_pages_back_and_requeues_requests_when_a_peer_is_gone():
    """The loop's reaction to a peer failure, on the CPU backend: nothing more is launched, the iteration in
    flight is waited for, every running request returns its KV pages and goes back to the head of the queue
    with its generated tokens folded into its prompt, and a fresh loop over the same queue serves them to
    the end (what a group re-formed without the dead rank would do)."""
    import numpy as np
    import torch

    from nanoflow_b200.config import builtin_config
    from nanoflow_b200.models import random_full_weights, shard_weights
    from nanoflow_b200.runtime.cpu_backend import CpuEngine
    from nanoflow_b200.serving import DistKVPool, RequestManager, Scheduler
    from nanoflow_b200.serving.loop import ServingLoop

    class FailingHealth:
        def __init__(self, fail_at):
            self.step, self.fail_at = 0, fail_at

        def beat(self):
            self.step += 1

        def check(self):
            if self.step >= self.fail_at:
                raise PeerFailure(1, self.fail_at - 1, self.step)

    cfg = builtin_config("tiny", gpu_num=1, global_batch_size=48, pipeline_type="NON_OVERLAP_LOCAL")
    cfg.engine.max_batch_size = 48
    fw = random_full_weights(cfg.model, seed=0)
    shards = [shard_weights(fw, cfg.model, 0, 1, dtype=torch.float32)]
    rm = RequestManager(vocab_size=1024, random_ids=True, seed=1)
    for _ in range(6):
        rm.add_request(24, 10, 0.0)
    rm.finalize_stats()
    pool = DistKVPool(2, 2, 64, 64, 16, 1)
    free0 = pool.num_free_pages if hasattr(pool, "num_free_pages") else None

    def make(health):
        sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=48, average_prefill_length=24,
                        average_decode_length=10, group_size=2)
        return ServingLoop(CpuEngine(cfg, shards, num_pages=64), sch, rm, est_cycle_time=1.0, health=health), sch

    loop, sch = make(FailingHealth(fail_at=6))
    with pytest.raises(PeerFailure) as info:
        loop.run()
    failure = info.value
    assert loop.failed is failure and failure.requeued > 0
    assert sch.in_flight == 0 and not sch._draining and not sch._held_pages
    if free0 is not None:
        assert pool.num_free_pages == free0                      # every page came back
    queued = list(rm.avaliable_request_queue._queue)
    assert len(queued) + failure.retired == 6
    assert [q.req_idx for q in queued] == sorted(q.req_idx for q in queued)
    partial = [q for q in queued if q.prompt.size > 24]
    assert partial and all(q.prompt.size + q.output_len == 24 + 10 for q in queued)
    done_before = {r.req_idx: len(r.output) for r in loop.stats.retired}
    # a second loop (the re-formed group) serves what was re-queued
    loop2, sch2 = make(None)
    st2 = loop2.run()
    assert len(st2.retired) == len(queued)
    assert all(len(r.output) + (r.input_len - 24) == 10 for r in st2.retired)
    assert set(done_before) | {r.req_idx for r in st2.retired} == set(range(6))
