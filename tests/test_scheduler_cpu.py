"""Scheduler behaviour: chunked prefill, nano-batch cuts, device feedback indices, admission by
projected peak pages, retirement timing (EOS at i+2), preemption under KV pressure, page conservation."""
import numpy as np
import pytest

from nanoflow_b200.serving import DistKVPool, NewRequestQueue, RequestManager, Scheduler


def _mk(pool_pages=400, gbs=64, nano=None, n=10, in_len=50, out_len=8, **kw):
    rm = RequestManager(vocab_size=1000, random_ids=True)
    for _ in range(n):
        rm.add_request(in_len, out_len, 0.0)
    rm.finalize_stats()
    rm.simulate_issue(1.0)
    pool = DistKVPool(2, 2, 64, pool_pages, 16)
    s = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs, nanobatch_sizes=nano,
                  average_prefill_length=in_len, average_decode_length=out_len, group_size=2, **kw)
    return s, pool, rm


def _drive(s, tokens_fn=None, max_iter=2000):
    plans, prev = [], None
    for _ in range(max_iter):
        p = s.schedule()
        if prev is not None:
            toks = np.zeros(len(prev.sample_reqs), dtype=np.int32) if tokens_fn is None else tokens_fn(prev)
            s.process_outputs(prev, toks)
        prev = p
        if p is None:
            if not s.has_work:
                break
            continue
        plans.append(p)
    s.schedule()
    return plans


def test_chunked_prefill_and_layout():
    s, pool, _ = _mk(gbs=64, n=3, in_len=50, out_len=4)
    p = s.schedule()
    # 64 dense tokens: request 0 whole (50), request 1 chunked (14); decode-first layout, none yet
    assert p.num_tokens == 64 and p.num_decode == 0
    assert [(r.req_idx, a, n) for r, a, n in p.prefill] == [(0, 0, 50), (1, 0, 14)]
    assert p.sample_rows.tolist() == [49]                        # only request 0 finished its prompt
    assert p.positions[:50].tolist() == list(range(50)) and p.positions[50:].tolist() == list(range(14))
    assert p.kv_indptr.tolist() == [0, 4, 5] and p.kv_last_page_len.tolist() == [2, 14]
    s.process_outputs(p, np.array([7], dtype=np.int32))
    p2 = s.schedule()
    # request 0 decodes (token on device: feedback index = its sample slot), request 1 continues at 14
    assert p2.num_decode == 1 and p2.feedback_src[0] == -1 and p2.host_ids[0] == 7   # host already saw it
    assert (p2.prefill[0][0].req_idx, p2.prefill[0][1], p2.prefill[0][2]) == (1, 14, 36)
    assert p2.prefill[1][0].req_idx == 2 and p2.num_tokens == 64
    p3 = s.schedule()                                             # formed before p2's tokens are known
    assert p3.feedback_src[0] == p2.sample_reqs.index(p3.decode[0])
    assert p3.feedback_src[1] == p2.sample_reqs.index(p3.decode[1])


def test_nanobatch_cut_straddles_requests():
    s, pool, _ = _mk(gbs=64, nano=[24, 40], n=3, in_len=50, out_len=4)
    p = s.schedule()
    a, b = p.nano
    assert (a.token_start, a.token_count, b.token_start, b.token_count) == (0, 24, 24, 40)
    # request 0 (tokens 0..49) is split across the cut; tiles never cross it; tile = 128/group = 64 tokens
    assert a.items.tolist() == [[0, 0, 24]]
    assert b.items.tolist() == [[0, 24, 26], [1, 50, 14]]
    assert sum(it[2] for nb in p.nano for it in nb.items.tolist()) == p.num_tokens - p.num_decode


def test_all_requests_finish_with_exact_lengths_and_pages_return():
    s, pool, _ = _mk(pool_pages=400, gbs=96, nano=[32, 64], n=25, in_len=37, out_len=9)
    plans = _drive(s)
    assert len(s.retired) == 25 and all(len(r.output) == 9 for r in s.retired)
    assert pool.num_free_pages == 400
    assert all(p.num_tokens <= 96 for p in plans)
    # every iteration's sampled slots are unique and in range
    for p in plans:
        assert len(set(p.sample_rows.tolist())) == len(p.sample_rows) and (p.sample_rows < p.num_tokens).all()


def test_eos_retires_two_iterations_later():
    s, pool, _ = _mk(gbs=64, n=1, in_len=10, out_len=50, eos_token_id=2, stop_on_eos=True)
    emitted = {"n": 0}

    def toks(plan):
        emitted["n"] += 1
        return np.array([2 if emitted["n"] == 3 else 5] * len(plan.sample_reqs), dtype=np.int32)

    plans = _drive(s, toks)
    r = s.retired[0]
    assert r.output == [5, 5, 2]                                  # tokens after EOS are dropped
    # the EOS was sampled in iteration 2 (0-based). Iteration 3 had already been formed when those
    # tokens reached the host, so it still ran the request; the request is dropped when iteration 4
    # (= i + 2) is formed, which therefore has nothing left to run.
    assert len(plans) == 4


def test_admission_respects_projected_peak_pages():
    # each request will need ceil((50+30)/16) = 5 pages at its peak; 23 pages hold 4 of them, not 5
    s, pool, _ = _mk(pool_pages=23, gbs=512, n=10, in_len=50, out_len=30)
    plans = _drive(s)
    assert len(plans[0].prefill) == 4
    assert max(len(p.decode) + len(p.prefill) for p in plans) <= 4
    assert len(s.retired) == 10 and s.preemptions == 0 and pool.num_free_pages == 23


def test_usage_curve_matches_brute_force():
    s, pool, _ = _mk(in_len=100, out_len=50)
    rng = np.random.default_rng(0)
    c = rng.integers(1, 200, size=300)
    L = 152
    brute = np.zeros(L, dtype=np.int64)
    for cj in c:
        for t in range(max(1, min(L, L - 1 - cj))):
            brute[t] += (cj + t + 15) // 16
    assert np.array_equal(s._usage_curve(c), brute)


def test_preemption_when_outputs_outgrow_the_projection():
    """Outputs far longer than the trace average: the projection under-estimates, allocation fails,
    the newest decode request is evicted and recomputed; everything still finishes, no page leaks."""
    rm = RequestManager(vocab_size=1000, random_ids=True)
    for _ in range(6):
        rm.add_request(30, 120, 0.0)
    rm.finalize_stats()
    rm.average_decode_length = 10                                  # a lie, to provoke over-admission
    rm.simulate_issue(1.0)
    pool = DistKVPool(2, 2, 64, 30, 16)
    s = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=128, average_prefill_length=30,
                  average_decode_length=10, group_size=2)
    _drive(s, max_iter=5000)
    assert s.preemptions > 0
    done = {}
    for r in s.retired:
        done.setdefault(r.req_idx, 0)
        done[r.req_idx] += len(r.output)
    assert sorted(done) == list(range(6))
    assert pool.num_free_pages == 30


def test_prefill_items_balanced_over_persistent_ctas():
    """Work items are dealt so that CTA c (items c, c+G, ...) gets close to the average context length."""
    pool = DistKVPool(1, 8, 128, 4096, 16)
    rm = RequestManager(vocab_size=100, random_ids=True)
    for n in (900, 700, 500, 300, 100, 60):
        rm.add_request(n, 4, 0.0)
    rm.finalize_stats()
    rm.simulate_issue(1.0)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=4096, average_prefill_length=400,
                    average_decode_length=4, group_size=8, prefill_ctas=8)
    plan = sch.schedule()
    items = plan.nano[0].items
    assert items.shape[0] == sum(-(-n // 16) for n in (900, 700, 500, 300, 100, 60))
    # every token of every prompt is covered exactly once
    covered = np.zeros(plan.num_tokens, dtype=np.int32)
    for req, start, cnt in items:
        covered[start:start + cnt] += 1
    assert (covered[plan.num_decode:] == 1).all()
    # cost of an item = position of its last token within its prompt (all prompts start at 0 here)
    qo = plan.qo_indptr
    cost = np.array([start - qo[req] + cnt for req, start, cnt in items])
    G = 8
    per_cta = np.array([cost[c::G].sum() for c in range(G)])
    assert per_cta.max() <= 1.1 * per_cta.mean()
    naive = np.sort(cost)            # the order a plain token walk would give: short contexts first
    naive_per_cta = np.array([naive[c::G].sum() for c in range(G)])
    assert per_cta.max() - per_cta.min() < naive_per_cta.max() - naive_per_cta.min()


@pytest.mark.parametrize("nano,frac", [([48, 48], 0.5), ([32, 64], 0.5), ([64, 32], 0.3), ([32, 32, 32], 0.5), ([48, 48], 1.0)])
def test_decode_tail_puts_a_share_of_the_decode_context_into_the_last_nanobatch(nano, frac):
    """With ``decode_tail_fraction`` the batch is [head decode | prompt chunks | tail decode]: every
    token and request is covered exactly once, each nano-batch sees one contiguous range of decode
    requests whose tokens lie inside it, and the tail carries about the requested share of context."""
    gbs = sum(nano)
    s, pool, _ = _mk(pool_pages=2000, gbs=gbs, nano=nano, n=60, in_len=41, out_len=24, decode_tail_fraction=frac)
    s.max_batch_size = gbs
    plans = _drive(s)
    assert len(s.retired) == 60 and all(len(r.output) == 24 for r in s.retired)
    mixed = 0
    for p in plans:
        D, Dt, T, B = p.num_decode, p.num_tail_decode, p.num_tokens, p.num_requests
        Dh, P = D - Dt, len(p.prefill)
        assert 0 <= Dt <= D and p.qo_indptr[0] == 0 and p.qo_indptr[B] == T
        assert (np.diff(p.qo_indptr[:B + 1]) > 0).all()
        # token -> request map agrees with qo_indptr, decode requests have one token each
        assert (np.repeat(np.arange(B), np.diff(p.qo_indptr[:B + 1])) == p.token_req).all()
        lens = np.diff(p.qo_indptr[:B + 1])
        assert (lens[:Dh] == 1).all() and (lens[Dh + P:] == 1).all()
        assert [r for r in p.decode] == p.sample_reqs[:Dh] + p.sample_reqs[len(p.sample_reqs) - Dt:]
        # per nano-batch: the decode range is inside the nano-batch, ranges tile all decode requests
        seen = []
        covered = np.zeros(T, dtype=np.int32)
        for nb in p.nano:
            t0, t1 = nb.token_start, nb.token_start + nb.token_count
            for req in range(nb.dec_begin, nb.dec_begin + nb.dec_count):
                assert req < Dh or req >= Dh + P
                tok = int(p.qo_indptr[req])
                assert t0 <= tok < t1
                covered[tok] += 1
                seen.append(req)
            for req, start, cnt in nb.items.tolist():
                assert Dh <= req < Dh + P and t0 <= start and start + cnt <= t1
                assert p.qo_indptr[req] <= start and start + cnt <= p.qo_indptr[req + 1]
                covered[start:start + cnt] += 1
        assert (covered == 1).all()
        assert sorted(seen) == list(range(Dh)) + list(range(Dh + P, B))
        if Dt and Dh:
            mixed += 1
            last0 = gbs - nano[-1]
            assert Dh <= last0 and T - Dt >= last0
            if T == gbs and len(nano) == 2 and Dt < min(D, T - last0) and Dt > max(0, D - last0):
                # unclamped: the tail is the shortest suffix of the decode requests that reaches the share
                ctx = np.concatenate([p.positions[:Dh], p.positions[T - Dt:]]).astype(np.int64) + 1
                tail_sum, total = ctx[Dh:].sum(), ctx.sum()
                assert tail_sum >= frac * total > tail_sum - ctx[Dh]
    assert mixed > 5 or frac == 1.0


def test_online_release_is_identical_on_ranks_with_skewed_clocks():
    """Two replicas of request manager + scheduler (two tensor-parallel ranks) whose wall clocks run at
    different speeds admit the same requests in the same cycle once both release by rank 0's clock."""
    import threading

    import torch.distributed as dist

    from nanoflow_b200.serving.frontend import SharedReleaseClock

    store = dist.HashStore()
    store.set_timeout(__import__("datetime").timedelta(seconds=20))
    arrivals = np.cumsum(np.random.default_rng(3).exponential(0.05, size=60))
    cycles = 80
    results = {}

    def replica(rank, tick):
        now = [0.0]

        def clock():              # every read advances this rank's private clock
            now[0] += tick
            return now[0]

        rm = RequestManager(vocab_size=1000, random_ids=True, seed=0, clock=clock)
        for a in arrivals:
            rm.add_request(40, 6, float(a))
        rm.finalize_stats()
        rm.release_clock = SharedReleaseClock(store, rank, 2, keep=8)
        pool = DistKVPool(2, 2, 64, 400, 16)
        s = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=64, nanobatch_sizes=[32, 32],
                      average_prefill_length=40, average_decode_length=6, group_size=2)
        rm.start_processing()
        sig, prev = [], None
        for _ in range(cycles):
            rm.issue()
            p = s.schedule()
            if prev is not None:
                s.process_outputs(prev, np.zeros(len(prev.sample_reqs), dtype=np.int32))
            prev = p
            sig.append(None if p is None else
                       (p.num_tokens, p.num_decode, tuple((r.req_idx, a, n) for r, a, n in p.prefill),
                        tuple(nb.token_count for nb in p.nano), p.kv_indices.tolist()))
        results[rank] = sig

    threads = [threading.Thread(target=replica, args=(0, 0.011)), threading.Thread(target=replica, args=(1, 0.017))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert set(results) == {0, 1}
    assert results[0] == results[1]
    assert sum(1 for x in results[0] if x is not None) > 10       # the trace was actually served
    assert store.num_keys() < cycles                               # keys that both ranks are past get deleted


def test_offload_manager_files_retired_requests_and_counts_what_left_the_gpu():
    """KVOffloadManager with a stand-in engine: requests retired in an iteration ride on its offload in page
    order, what does not fit the per-iteration staging is dropped (and counted), the host store evicts beyond
    its byte limit while the totals keep counting, and held pages are released once the copy has completed."""
    from types import SimpleNamespace
    import torch
    from nanoflow_b200.serving.offload import KVOffloadManager

    layers, cap, page_elems = 2, 8, 16
    host = torch.arange(layers * cap * page_elems, dtype=torch.float32).view(layers, cap, page_elems)
    engine = SimpleNamespace(offload_cap=cap, offloaded_pages=lambda: host)
    released = []
    sched = SimpleNamespace(release_held_pages=lambda it: released.append(it))
    page_bytes = layers * page_elems * 4
    mgr = KVOffloadManager(engine, max_host_bytes=5 * page_bytes)

    def req(idx, pages, seqlen):
        return SimpleNamespace(req_idx=idx, kv_cache=SimpleNamespace(num_pages=pages, seqlen=seqlen), offloaded=False)

    a, b, c = req(1, 3, 40), req(2, 4, 60), req(3, 2, 20)          # 3 + 4 fit the 8 staging pages, the third does not
    plan = SimpleNamespace(iteration=7, retired_reqs=[a, b, c])
    mgr.on_iteration(plan)
    mgr.on_complete(plan, sched)
    assert released == [7]
    assert a.offloaded and b.offloaded and not c.offloaded
    assert (mgr.total_requests, mgr.total_pages, mgr.dropped_requests) == (2, 7, 1)
    assert mgr.total_bytes == 7 * page_bytes
    # request 2's pages are the four staged behind request 1's three
    assert torch.equal(mgr.store[2].data, host[:, 3:7]) and mgr.store[2].seqlen == 60
    # the store holds at most five pages' worth: filing request 2 (4 pages) evicted request 1 (3 pages)
    assert 1 not in mgr.store and mgr.bytes == 4 * page_bytes
    # an iteration without retired requests still releases what it held
    empty = SimpleNamespace(iteration=8, retired_reqs=[])
    mgr.on_iteration(empty)
    mgr.on_complete(empty, sched)
    assert released == [7, 8] and mgr.total_requests == 2
