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
