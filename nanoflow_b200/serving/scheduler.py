"""Iteration-level batch scheduler with asynchronous control flow.

Each call to :meth:`Scheduler.schedule` forms the dense batch of the *next* iteration while the GPU
is still running the previous one:

* running decode requests continue by length only (their newest token is still on the device and
  is fed back there; the host sees it one iteration late);
* unfinished prompts get their next chunk (chunked prefill), then new requests are admitted while
  there are idle tokens in the dense batch, request slots, and the *projected peak* KV page usage
  (every running request assumed to grow to the trace's average prompt + output length) leaves
  room for one more request;
* KV pages for every scheduled token are allocated here, before the iteration is launched;
* the dense batch is laid out decode tokens first, then prefill tokens, and cut into nano-batches
  at fixed token boundaries; a prompt chunk that straddles a boundary becomes attention work items
  on both sides.

:meth:`process_outputs` consumes the sampled tokens of an iteration when they reach the host. An
EOS seen there stops the request at the next ``schedule`` call, i.e. a request that emitted EOS in
iteration *i* is retired when iteration *i+2* is formed; the one or two surplus tokens are dropped.

Behavioural model: ``Scheduler.schedule_req`` / ``bench_text_gen`` in the reference
(pipeline/utils/serve_8B.py:177-203 future-page estimate, :212-343 admission + chunking, :348-569
the asynchronous iteration, :530-561 continuation by length). The per-token Python list building
there (:419-431) is replaced by NumPy array construction.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from .kv_cache import DistKVCache, DistKVPool, KVPoolExhausted
from .request import FlyRequestInfo, NewRequestInfo, NewRequestQueue


class WorkingSet:
    """A set of in-flight requests (API of the reference's ``WorkingSet``, serve_8B.py:66-99)."""

    def __init__(self) -> None:
        self._set: List[FlyRequestInfo] = []

    def put(self, req: FlyRequestInfo) -> None:
        self._set.append(req)

    def __getitem__(self, key):
        return self._set[key]

    def __iter__(self):
        return iter(self._set)

    def __len__(self):
        return len(self._set)

    @property
    def size(self) -> int:
        return len(self._set)


@dataclass
class NanoBatchPlan:
    token_start: int
    token_count: int
    dec_begin: int          # first decode request (index into the batch's request order)
    dec_count: int
    items: np.ndarray       # [n,3] int32 prefill work items (request, first token, token count)


@dataclass
class BatchPlan:
    iteration: int
    decode: List[FlyRequestInfo]
    prefill: List[Tuple[FlyRequestInfo, int, int]]      # (request, chunk start, chunk length)
    num_tokens: int
    num_decode: int                                     # decode requests in all (head + tail)
    host_ids: np.ndarray
    feedback_src: np.ndarray
    positions: np.ndarray
    token_req: np.ndarray
    qo_indptr: np.ndarray
    kv_indptr: np.ndarray
    kv_indices: np.ndarray
    kv_last_page_len: np.ndarray
    sample_rows: np.ndarray
    sample_reqs: List[FlyRequestInfo]
    nano: List[NanoBatchPlan]
    max_kv_pages: int = 0
    retired_pages: Optional[np.ndarray] = None          # pages of requests retired at this step (offload)
    retired_reqs: List[FlyRequestInfo] = field(default_factory=list)
    # Request order of the batch: ``num_decode - num_tail_decode`` decode requests, the prompt chunks, then
    # ``num_tail_decode`` decode requests whose tokens are the last of the batch (they fall into the last
    # nano-batch). ``decode`` lists head then tail.
    num_tail_decode: int = 0

    @property
    def num_requests(self) -> int:
        return len(self.decode) + len(self.prefill)


class Scheduler:
    def __init__(self, memory_pool: DistKVPool, request_queue: NewRequestQueue, *,
                 global_batch_size: int, nanobatch_sizes: Optional[Sequence[int]] = None,
                 max_batch_size: Optional[int] = None, average_prefill_length: int = 1024,
                 average_decode_length: int = 512, group_size: int = 8, eos_token_id: Optional[int] = None,
                 stop_on_eos: bool = False, hold_retired_pages: bool = False, prefill_ctas: int = 296,
                 decode_tail_fraction: float = 0.0):
        self._memory_pool = memory_pool
        self._request_queue = request_queue
        self.global_batch_size = int(global_batch_size)
        self.nanobatch_sizes = list(nanobatch_sizes) if nanobatch_sizes else [self.global_batch_size]
        if sum(self.nanobatch_sizes) != self.global_batch_size:
            raise ValueError("nano-batch sizes must sum to the dense batch size")
        self.max_batch_size = int(max_batch_size or global_batch_size)
        self.average_prefill_length = int(average_prefill_length)
        self.average_decode_length = int(average_decode_length)
        self.tile_tokens = max(1, 128 // group_size)    # query tokens per prefill work item
        self.prefill_ctas = int(prefill_ctas)           # persistent CTAs of the prefill attention kernel (two per SM)
        self.eos_token_id = eos_token_id
        self.stop_on_eos = stop_on_eos
        self.hold_retired_pages = hold_retired_pages
        # Share of the decode requests' context (KV tokens to read) that goes to the end of the batch, and
        # so into the last nano-batch, instead of the front. With all decode requests in the first
        # nano-batch its attention takes several times longer than the last one's, and under tensor
        # parallelism the collective of one nano-batch has to hide behind the other's compute.
        if not 0.0 <= decode_tail_fraction <= 1.0:
            raise ValueError("decode_tail_fraction must be within [0, 1]")
        self.decode_tail_fraction = float(decode_tail_fraction)

        self._decode_workset = WorkingSet()
        self._prefill_workset = WorkingSet()
        self._draining: List[FlyRequestInfo] = []       # stopped, last tokens still in flight
        self._held_pages: List[Tuple[int, FlyRequestInfo]] = []
        self.retired: List[FlyRequestInfo] = []
        self.iteration = 0
        self.preemptions = 0
        self.schedule_log: List[dict] = []
        self.keep_schedule_log = False

    # ---- admission control ----------------------------------------------------------------------
    def _usage_curve(self, cur: np.ndarray) -> np.ndarray:
        """Projected page usage over the next ``L`` iterations for requests of current lengths
        ``cur`` that each grow by one token per iteration until avg prompt + avg output length.

        usage(t) = sum_j [t < r_j] * ceil((c_j + t) / ps). Requests are bucketed by
        (c_j + ps - 1) mod ps and remaining steps r_j, which turns the double sum into
        O(ps * L) array work instead of O(requests * L)."""
        ps = self._memory_pool.page_size
        L = self.average_prefill_length + self.average_decode_length + 2
        if cur.size == 0:
            return np.zeros(L, dtype=np.int64)
        c = cur.astype(np.int64)
        r = np.clip(L - 1 - c, 1, L)
        a = c + ps - 1
        A, mm = a // ps, a % ps
        key = mm * (L + 1) + r
        cnt = np.bincount(key, minlength=ps * (L + 1)).reshape(ps, L + 1)
        sa = np.bincount(key, weights=A.astype(np.float64), minlength=ps * (L + 1)).reshape(ps, L + 1)
        # alive at time t  <=>  r > t : suffix sums over r, shifted by one
        n_alive = cnt[:, ::-1].cumsum(axis=1)[:, ::-1][:, 1:]
        a_alive = sa[:, ::-1].cumsum(axis=1)[:, ::-1][:, 1:]
        t = np.arange(L, dtype=np.int64)[None, :]
        extra = (np.arange(ps, dtype=np.int64)[:, None] + t) // ps
        return (a_alive + n_alive * extra).sum(axis=0).astype(np.int64)

    def projected_peak_pages(self, extra_new: int = 0) -> int:
        """Peak KV page usage if every running request grows to avg prompt + avg output length
        (the admission test of the reference, pipeline/utils/serve_8B.py:177-203)."""
        cur = [r.kv_cache.seqlen + 1 for r in self._decode_workset]
        cur += [self.average_prefill_length + 1] * (self._prefill_workset.size + extra_new)
        if not cur:
            return 0
        return int(self._usage_curve(np.asarray(cur)).max())

    def _admission_state(self):
        cur = np.fromiter((r.kv_cache.seqlen + 1 for r in self._decode_workset), dtype=np.int64,
                          count=self._decode_workset.size)
        base = self._usage_curve(np.concatenate([cur, np.full(self._prefill_workset.size,
                                                               self.average_prefill_length + 1)]))
        one = self._usage_curve(np.asarray([self.average_prefill_length + 1]))
        return base, one

    # ---- preemption -----------------------------------------------------------------------------
    def _preempt_one(self, exclude: Sequence[FlyRequestInfo]) -> bool:
        """Free the pages of the newest decode request and queue it for recomputation."""
        protected = {id(r) for r in exclude}
        victim = None
        for r in reversed(self._decode_workset._set):
            if id(r) not in protected and not r.preempted:
                victim = r
                break
        if victim is None:
            return False
        self._decode_workset._set.remove(victim)
        victim.preempted = True   # a token still in flight for it is dropped when it arrives
        victim.kv_cache.release()
        redo = NewRequestInfo()
        redo.req_idx = victim.req_idx
        redo.prompt = np.concatenate([victim.prompt, np.asarray(victim.output, dtype=np.int32)])
        redo.output_len = victim.output_len - len(victim.output)
        redo.start_time = victim.request_comein_time
        self._request_queue._queue.appendleft(redo)
        self.preemptions += 1
        return True

    def _alloc(self, req: FlyRequestInfo, n: int, protect: Sequence[FlyRequestInfo]) -> bool:
        while True:
            try:
                req.kv_cache.allocate_tokens(n)
                return True
            except KVPoolExhausted:
                if not self._preempt_one(list(protect) + [req]):
                    return False

    # ---- retirement -----------------------------------------------------------------------------
    def _stop(self, req: FlyRequestInfo, plan_retired: list) -> None:
        plan_retired.append(req)
        if self.hold_retired_pages:
            self._held_pages.append((self.iteration, req))
        else:
            req.kv_cache.release()
        if req.pending > 0:
            self._draining.append(req)
        else:
            self._retire(req)

    def _retire(self, req: FlyRequestInfo) -> None:
        req.finished = True
        if req.finish_time == 0.0:
            req.finish_time = time.perf_counter()
        self.retired.append(req)

    def release_held_pages(self, upto_iteration: int) -> None:
        """Free pages of requests stopped at or before ``upto_iteration`` (their offload is done)."""
        keep = []
        for it, req in self._held_pages:
            if it <= upto_iteration:
                req.kv_cache.release()
            else:
                keep.append((it, req))
        self._held_pages = keep

    def requeue_running(self) -> int:
        """Give up every request that is in flight: free its pages and put it back at the head of the
        request queue with the tokens it has produced so far folded into its prompt, so that whoever
        serves the queue next (this engine after the failure has been dealt with, or a new one at a
        smaller tensor-parallel degree) recomputes its KV and carries on where it stopped. Requests that
        had already stopped and were only waiting for their last tokens are retired with what they have.
        Returns the number of re-queued requests. Tokens of iterations still in flight are dropped."""
        redo_list = []
        for ws in (self._decode_workset, self._prefill_workset):
            for r in list(ws._set):
                if r.preempted:
                    continue
                r.preempted = True
                r.kv_cache.release()
                redo = NewRequestInfo()
                redo.req_idx = r.req_idx
                redo.prompt = np.concatenate([r.prompt, np.asarray(r.output, dtype=np.int32)])
                redo.output_len = r.output_len - len(r.output)
                redo.start_time = r.request_comein_time
                if redo.output_len > 0:
                    redo_list.append(redo)
                else:
                    self._retire(r)
            ws._set.clear()
        for r in self._draining:
            r.pending = 0
            self._retire(r)
        self._draining = []
        self.release_held_pages(self.iteration)
        for redo in sorted(redo_list, key=lambda q: q.req_idx, reverse=True):
            self._request_queue._queue.appendleft(redo)
        return len(redo_list)

    # ---- main entry -----------------------------------------------------------------------------
    @property
    def has_work(self) -> bool:
        return bool(self._decode_workset.size or self._prefill_workset.size or self._request_queue.size
                    or self._draining)

    @property
    def in_flight(self) -> int:
        return self._decode_workset.size + self._prefill_workset.size

    def schedule(self) -> Optional[BatchPlan]:
        gbs, ps = self.global_batch_size, self._memory_pool.page_size
        retired_now: List[FlyRequestInfo] = []

        # 1. decode requests that continue (by length; EOS seen one iteration late)
        decode: List[FlyRequestInfo] = []
        for req in list(self._decode_workset):
            if req.eos_seen or req.generated >= req.output_len:
                self._decode_workset._set.remove(req)
                self._stop(req, retired_now)
        for req in list(self._decode_workset):
            if req.preempted:                             # lost its pages to an earlier allocation
                continue
            if len(decode) >= min(gbs, self.max_batch_size):
                break
            if self._alloc(req, 1, decode):
                decode.append(req)

        # 2. prompts in progress, then 3. new admissions
        idle = gbs - len(decode)
        slots = self.max_batch_size - len(decode)
        prefill: List[Tuple[FlyRequestInfo, int, int]] = []
        for req in list(self._prefill_workset):
            if idle <= 0 or slots <= 0:
                break
            n = min(req.input_len - req.prefill_done, idle)
            if n > 0 and self._alloc(req, n, decode):
                prefill.append((req, req.prefill_done, n))
                idle -= n
                slots -= 1
        admitted = 0
        ps_need = (self.average_prefill_length + self.average_decode_length + ps) // ps
        curve, one = (self._admission_state() if (idle > 0 and slots > 0 and self._request_queue.size > 0)
                      else (None, None))
        while idle > 0 and slots > 0 and self._request_queue.size > 0 and \
                self._memory_pool.capacity - int(curve.max()) > ps_need:
            curve = curve + one
            new = self._request_queue.get()
            req = FlyRequestInfo(req_idx=new.req_idx, prompt=np.asarray(new.prompt, dtype=np.int32),
                                 output_len=new.output_len, kv_cache=DistKVCache(self._memory_pool),
                                 request_comein_time=new.start_time)
            n = min(req.input_len, idle)
            try:
                req.kv_cache.allocate_tokens(n)
            except KVPoolExhausted:
                self._request_queue._queue.appendleft(new)
                break
            req.chunked_prefill = n < req.input_len
            self._prefill_workset.put(req)
            prefill.append((req, 0, n))
            idle -= n
            slots -= 1
            admitted += 1

        D = len(decode)
        T = D + sum(n for _, _, n in prefill)
        if T == 0:
            self._finish_retire_log(retired_now)
            return None

        # 4. arrays. Request (and token) order: head decode requests, prompt chunks, tail decode requests.
        P = len(prefill)
        B = D + P
        Dt = self._tail_decode_count(decode, T)
        Dh = D - Dt
        host_ids = np.zeros(T, dtype=np.int32)
        feedback = np.full(T, -1, dtype=np.int32)
        positions = np.empty(T, dtype=np.int32)
        token_req = np.empty(T, dtype=np.int32)
        qo_indptr = np.zeros(B + 1, dtype=np.int32)

        def fill_decode(reqs, tok0, req0):
            n = len(reqs)
            if n == 0:
                return
            # Newest token still on the device (launched last iteration, not yet seen by the host):
            # feed it back there. A request that sat out an iteration has it on the host already.
            feedback[tok0:tok0 + n] = np.fromiter((r.slot if r.pending > 0 else -1 for r in reqs), dtype=np.int32, count=n)
            host_ids[tok0:tok0 + n] = np.fromiter((r.output[-1] if (r.pending == 0 and r.output) else 0 for r in reqs),
                                                  dtype=np.int32, count=n)
            positions[tok0:tok0 + n] = np.fromiter((r.kv_cache.seqlen - 1 for r in reqs), dtype=np.int32, count=n)
            token_req[tok0:tok0 + n] = np.arange(req0, req0 + n, dtype=np.int32)
            qo_indptr[req0 + 1:req0 + n + 1] = np.arange(tok0 + 1, tok0 + n + 1, dtype=np.int32)

        head, tail = decode[:Dh], decode[Dh:]
        fill_decode(head, 0, 0)
        t = Dh
        sample_rows = list(range(Dh))
        sample_reqs = list(head)
        for j, (req, s, n) in enumerate(prefill):
            host_ids[t:t + n] = req.prompt[s:s + n]
            positions[t:t + n] = np.arange(s, s + n, dtype=np.int32)
            token_req[t:t + n] = Dh + j
            t += n
            qo_indptr[Dh + j + 1] = t
            if s + n == req.input_len:
                sample_rows.append(t - 1)
                sample_reqs.append(req)
        fill_decode(tail, t, Dh + P)
        sample_rows.extend(range(t, t + Dt))
        sample_reqs.extend(tail)
        kvs = [r.kv_cache for r in head] + [r.kv_cache for r, _, _ in prefill] + [r.kv_cache for r in tail]
        counts = np.fromiter((kv.num_pages for kv in kvs), dtype=np.int32, count=B)
        kv_indptr = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(counts, out=kv_indptr[1:])
        kv_indices = np.concatenate([kv.indicies for kv in kvs]).astype(np.int32, copy=False)
        kv_last = np.fromiter((kv.last_page_offset for kv in kvs), dtype=np.int32, count=B)

        # 5. state transitions for the launched work
        for slot, req in enumerate(sample_reqs):
            req.slot = slot
            req.pending += 1
        for req, s, n in prefill:
            req.prefill_done = s + n
            if not req.in_prefill:
                self._prefill_workset._set.remove(req)
                self._decode_workset.put(req)

        # 6. nano-batches
        nano = self._cut_nanobatches(T, Dh, Dt, prefill, qo_indptr)

        plan = BatchPlan(iteration=self.iteration, decode=decode, prefill=prefill, num_tokens=T, num_decode=D,
                         host_ids=host_ids, feedback_src=feedback, positions=positions, token_req=token_req,
                         qo_indptr=qo_indptr, kv_indptr=kv_indptr, kv_indices=kv_indices,
                         kv_last_page_len=kv_last, sample_rows=np.asarray(sample_rows, dtype=np.int32),
                         sample_reqs=sample_reqs, nano=nano, max_kv_pages=int(counts.max()) if B else 0,
                         retired_reqs=retired_now, num_tail_decode=Dt)
        if self.hold_retired_pages and retired_now:
            plan.retired_pages = np.concatenate([r.kv_cache.indicies for r in retired_now]).astype(np.int32)
        self._finish_retire_log(retired_now, plan)
        self.iteration += 1
        return plan

    def _finish_retire_log(self, retired_now, plan: Optional[BatchPlan] = None) -> None:
        if self.keep_schedule_log:
            self.schedule_log.append(dict(
                iteration=self.iteration, time=time.perf_counter(),
                decode_tokens=plan.num_decode if plan else 0,
                prefill_tokens=(plan.num_tokens - plan.num_decode) if plan else 0,
                batch_size=plan.num_tokens if plan else 0,
                idle_tokens=self.global_batch_size - (plan.num_tokens if plan else 0),
                page_usage=self._memory_pool.num_used_pages / max(1, self._memory_pool.capacity),
                queue=self._request_queue.size, retired=len(retired_now)))

    def _balanced_order(self, cost: np.ndarray) -> np.ndarray:
        """Order in which the attention kernel's persistent CTAs (CTA c takes items c, c + G, ...)
        get near-equal total cost: items sorted by falling cost, dealt in rounds of G that alternate
        direction, so the CTA that drew the dearest item of one round draws the cheapest of the next."""
        G = max(1, self.prefill_ctas)
        order = np.argsort(-cost, kind="stable")
        for r in range(1, (order.size + G - 1) // G, 2):
            order[r * G:(r + 1) * G] = order[r * G:(r + 1) * G][::-1].copy()
        return order

    def _tail_decode_count(self, decode: List[FlyRequestInfo], T: int) -> int:
        """How many of the decode requests (the last ones of ``decode``) go to the end of the batch:
        enough to carry ``decode_tail_fraction`` of the context, within what keeps a single range of
        decode requests per nano-batch (no head request in the last nano-batch, no tail request
        outside it)."""
        D = len(decode)
        if self.decode_tail_fraction <= 0.0 or len(self.nanobatch_sizes) < 2 or D == 0:
            return 0
        last_start = self.global_batch_size - self.nanobatch_sizes[-1]
        hi = min(D, max(0, T - last_start))               # tail tokens must lie inside the last nano-batch
        lo = max(0, D - last_start)                       # head tokens must end before it
        if hi <= 0:
            return 0
        ctx = np.fromiter((r.kv_cache.seqlen for r in decode), dtype=np.int64, count=D)
        from_end = np.cumsum(ctx[::-1])
        want = int(np.searchsorted(from_end, self.decode_tail_fraction * float(from_end[-1]), side="left")) + 1
        return int(min(hi, max(lo, want)))

    def _cut_nanobatches(self, T: int, Dh: int, Dt: int, prefill, qo_indptr) -> List[NanoBatchPlan]:
        out = []
        start = 0
        tq = self.tile_tokens
        P = len(prefill)
        tail0 = T - Dt                                     # first tail decode token
        for size in self.nanobatch_sizes:
            t0, t1 = start, min(T, start + size)
            start += size
            if t1 <= t0:
                out.append(NanoBatchPlan(t0 if t0 < T else T, 0, min(Dh, t0), 0, np.zeros((0, 3), dtype=np.int32)))
                continue
            d0, d1 = min(Dh, t0), min(Dh, t1)              # head decode requests: request index = token index
            a0, a1 = max(t0, tail0), t1                    # tail decode tokens of this nano-batch
            if a1 > a0:
                if d1 > d0:
                    raise AssertionError("a nano-batch holds decode requests from both ends of the batch")
                d0 = Dh + P + (a0 - tail0)
                d1 = d0 + (a1 - a0)
            items, kv_ends = [], []
            for j, (req, s, n) in enumerate(prefill):
                q0, q1 = int(qo_indptr[Dh + j]), int(qo_indptr[Dh + j + 1])
                a, b = max(q0, t0), min(q1, t1)
                if b <= a:
                    continue
                starts = np.arange(a, b, tq, dtype=np.int32)
                cnt = np.minimum(tq, b - starts).astype(np.int32)
                items.append(np.stack([np.full_like(starts, Dh + j), starts, cnt], axis=1))
                kv_ends.append(s + (starts - q0) + cnt)     # context each item attends to = its cost
            it = np.concatenate(items) if items else np.zeros((0, 3), dtype=np.int32)
            if it.shape[0] > 1:
                it = it[self._balanced_order(np.concatenate(kv_ends))]
            out.append(NanoBatchPlan(t0, t1 - t0, d0, d1 - d0, it))
        return out

    # ---- results --------------------------------------------------------------------------------
    def process_outputs(self, plan: BatchPlan, tokens: Optional[np.ndarray], now: Optional[float] = None) -> None:
        """Record the sampled tokens of ``plan`` (``tokens[slot]`` per sampling request)."""
        now = time.perf_counter() if now is None else now
        for slot, req in enumerate(plan.sample_reqs):
            req.pending -= 1
            tok = int(tokens[slot]) if tokens is not None else 0
            stopped = req.preempted or req.eos_seen or len(req.output) >= req.output_len
            if not stopped:
                if not req.output:
                    req.first_token_time = now
                    req.decode_start_at = now
                req.output.append(tok)
                if self.stop_on_eos and self.eos_token_id is not None and tok == self.eos_token_id:
                    req.eos_seen = True
                if req.eos_seen or len(req.output) >= req.output_len:
                    req.finish_time = now
        still = []
        for req in self._draining:
            if req.pending <= 0:
                self._retire(req)
            else:
                still.append(req)
        self._draining = still

    def drain_retired(self) -> List[FlyRequestInfo]:
        out, self.retired = self.retired, []
        return out
