"""Trace reader and request release clock.

Trace CSV (header line, then one request per line): ``idx,input_len,output_len,arrival_s[,prompt]``.
``input_len == -1`` means "tokenise the prompt text" (needs a tokenizer); otherwise synthetic ids are
made up. Requests become available either by wall clock (:meth:`issue`) or by simulated time
(:meth:`simulate_issue`). Mirrors ``requestManager`` in the reference (pipeline/utils/frontend.py:23-91).
Synthetic prompts there are ``range(len)``; here they may also be uniform-random ids (seeded), which
is what the benchmark configs ask for.
"""
from __future__ import annotations

import time
from typing import Callable, Optional

import numpy as np

from .request import NewRequestInfo, NewRequestQueue


class RequestManager:
    def __init__(self, filename: Optional[str] = None, *, vocab_size: int = 32000, random_ids: bool = False,
                 seed: int = 0, tokenizer: Optional[Callable[[str], "np.ndarray"]] = None,
                 clock: Callable[[], float] = time.perf_counter):
        self.filename = filename
        self._clock = clock                  # wall clock of this process (tests inject skewed ones)
        self.release_clock = None            # SharedReleaseClock under tensor parallelism (see issue())
        self._issue_cycle = 0
        self.avaliable_request_queue = NewRequestQueue()   # spelling kept from the reference API
        self.full_request_queue = NewRequestQueue()
        self.start_time = 0.0
        self.passed_time = 0.0
        self.average_prefill_length = 0
        self.average_decode_length = 0
        self.pdr = 0.0
        self.start_idx = 0
        self.vocab_size = vocab_size
        self.random_ids = random_ids
        self._rng = np.random.default_rng(seed)
        self._tokenizer = tokenizer
        self.total_requests = 0

    @property
    def available_request_queue(self) -> NewRequestQueue:
        return self.avaliable_request_queue

    def _make_prompt(self, n: int) -> np.ndarray:
        if self.random_ids:
            return self._rng.integers(0, self.vocab_size, size=n, dtype=np.int32)
        return (np.arange(n, dtype=np.int64) % self.vocab_size).astype(np.int32)

    def add_request(self, input_len: int, output_len: int, arrival: float = 0.0, prompt=None, text=None):
        req = NewRequestInfo()
        req.req_idx = self.total_requests
        self.total_requests += 1
        req.output_len = int(output_len)
        req.start_time = float(arrival)
        if prompt is not None:
            req.prompt = np.asarray(prompt, dtype=np.int32)
        elif input_len == -1:
            if self._tokenizer is None:
                raise ValueError("trace row asks for tokenisation (input_len == -1) but no tokenizer was given")
            req.prompt = np.asarray(self._tokenizer(text), dtype=np.int32)
            req.text = text
        else:
            if input_len <= 0:
                raise ValueError(f"request {req.req_idx}: input_len must be positive or -1")
            req.prompt = self._make_prompt(int(input_len))
        if req.output_len <= 0:
            raise ValueError(f"request {req.req_idx}: output_len must be positive")
        self.full_request_queue.put(req)
        return req

    def read_request(self, model_name_or_path: Optional[str] = None) -> None:
        if self.filename is None:
            raise ValueError("no trace file")
        if model_name_or_path and self._tokenizer is None:
            self._tokenizer = _lazy_hf_tokenizer(model_name_or_path)
        with open(self.filename, "r") as f:
            first = True
            for lineno, line in enumerate(f):
                if first:
                    first = False
                    continue
                line = line.rstrip("\n")
                if not line.strip():
                    continue
                parts = line.split(",", 4)
                if len(parts) < 4:
                    raise ValueError(f"{self.filename}:{lineno + 1}: expected idx,input_len,output_len,arrival")
                try:
                    in_len, out_len, arrival = int(parts[1]), int(parts[2]), float(parts[3])
                except ValueError as e:
                    raise ValueError(f"{self.filename}:{lineno + 1}: {e}") from None
                self.add_request(in_len, out_len, arrival, text=parts[4] if len(parts) > 4 else None)
        self.finalize_stats()

    def finalize_stats(self) -> None:
        q = self.full_request_queue._queue
        if not q:
            raise ValueError("trace holds no requests")
        self.average_prefill_length = sum(int(r.prompt.size) for r in q) // len(q)
        self.average_decode_length = sum(r.output_len for r in q) // len(q)
        self.pdr = self.average_prefill_length / max(1, self.average_decode_length)

    @property
    def decode_batch_size(self) -> int:
        return int(2048 // (1 + self.pdr))

    def start_processing(self) -> None:
        self.start_time = self._clock()
        if self.avaliable_request_queue.size > 0:
            self.start_idx = self.avaliable_request_queue.peek().req_idx
        elif self.full_request_queue.size > 0:
            self.start_idx = self.full_request_queue.peek().req_idx
        else:
            self.start_idx = -1

    def release_request(self) -> None:
        """Move requests whose arrival time has passed to the available queue; their ``start_time``
        becomes the wall-clock release time (latencies are measured from it), as in the reference."""
        while self.full_request_queue.size > 0 and self.full_request_queue.peek().start_time <= self.passed_time:
            r = self.full_request_queue.get()
            r.start_time = self._clock()
            self.avaliable_request_queue.put(r)

    def simulate_issue(self, estimate_cycle_time: float = 0.175) -> None:
        self.passed_time += estimate_cycle_time
        self.release_request()

    def issue(self) -> None:
        """Release by wall clock. Every tensor-parallel rank runs its own copy of the scheduler and all
        copies must admit the same requests in the same cycle (the collectives move rows whose count
        each rank derives from its own plan), but no two processes read the same wall clock. With a
        ``release_clock`` the elapsed time that rank 0 measured for this cycle is the one every rank
        uses, so the copies stay identical; without one (a single rank) the local clock decides."""
        t = self._clock()
        self.passed_time += t - self.start_time
        self.start_time = t
        if self.release_clock is not None:
            self.passed_time = self.release_clock.passed(self._issue_cycle, self.passed_time)
        self._issue_cycle += 1
        self.release_request()


class SharedReleaseClock:
    """Rank 0's elapsed time, cycle by cycle, through the job's key-value store.

    Rank 0 publishes the elapsed serving time it measured at the top of cycle ``c`` under one key per
    cycle; the other ranks block on that key (the store's ``get`` waits until the key exists) and use
    the value instead of their own clock. Every follower counts the cycles it has consumed in a counter
    key; every ``keep`` cycles rank 0 reads those counters and deletes the keys that all followers are
    past (while the engine is busy the ranks are at most the iterations in flight apart, but in an idle
    stretch nothing else holds rank 0 back). The reference runs one scheduler in one process for all
    GPUs (pipeline/utils/serve_8B.py:687-696) and so never meets the problem."""

    def __init__(self, store, rank: int, world: int = 2, prefix: str = "nf_release", keep: int = 64):
        self.store, self.rank, self.world, self.prefix, self.keep = store, rank, world, prefix, max(1, keep)
        self._deleted = 0          # rank 0: keys of cycles [0, _deleted) are gone
        if rank != 0:
            self.store.add(f"{prefix}/ack/{rank}", 0)

    def passed(self, cycle: int, local_passed: float) -> float:
        import struct

        key = f"{self.prefix}/{cycle}"
        if self.rank == 0:
            self.store.set(key, struct.pack("<d", float(local_passed)))
            if cycle - self._deleted >= 2 * self.keep:
                seen = min((int(self.store.add(f"{self.prefix}/ack/{r}", 0)) for r in range(1, self.world)),
                           default=cycle)
                for c in range(self._deleted, min(seen, cycle)):
                    self.store.delete_key(f"{self.prefix}/{c}")
                self._deleted = max(self._deleted, min(seen, cycle))
            return float(local_passed)
        value = struct.unpack("<d", bytes(self.store.get(key)))[0]
        self.store.add(f"{self.prefix}/ack/{self.rank}", 1)
        return value


def _lazy_hf_tokenizer(name: str):
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name)
    return lambda s: np.asarray(tok(s)["input_ids"], dtype=np.int32)


requestManager = RequestManager  # reference spelling
