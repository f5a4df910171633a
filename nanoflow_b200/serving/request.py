"""Request records. Names follow the reference's ``pipeline/utils/request_info.py:2-57``."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .kv_cache import DistKVCache


@dataclass
class NewRequestInfo:
    """A request as read from the trace, before admission."""
    req_idx: int = 0
    prompt: Optional[np.ndarray] = None   # int32 token ids
    output_len: int = 0
    start_time: float = 0.0               # arrival (trace seconds, then wall clock once released)
    text: Optional[str] = None


class NewRequestQueue:
    def __init__(self) -> None:
        self._queue = deque()

    @property
    def size(self) -> int:
        return len(self._queue)

    def put(self, req: NewRequestInfo) -> None:
        self._queue.append(req)

    def get(self) -> NewRequestInfo:
        if not self._queue:
            raise IndexError("request queue is empty")
        return self._queue.popleft()

    def peek(self) -> NewRequestInfo:
        return self._queue[0]

    def clear(self) -> None:
        self._queue.clear()


@dataclass
class FlyRequestInfo:
    """A request in flight: prompt progress, generated tokens, KV pages, latency bookkeeping."""
    req_idx: int
    prompt: np.ndarray
    output_len: int
    kv_cache: DistKVCache
    request_comein_time: float = 0.0
    prefill_done: int = 0                       # prompt tokens already run
    output: List[int] = field(default_factory=list)
    pending: int = 0                            # tokens launched whose value the host has not seen
    decode_start_at: float = 0.0
    finish_time: float = 0.0
    first_token_time: float = 0.0
    chunked_prefill: bool = False
    finished: bool = False
    eos_seen: bool = False
    slot: int = -1                              # row of this request's newest token in the last sampled array
    offloaded: bool = False
    preempted: bool = False                     # pages taken back; the request was re-queued

    @property
    def input_len(self) -> int:
        return int(self.prompt.size)

    @property
    def in_prefill(self) -> bool:
        return self.prefill_done < self.prompt.size

    @property
    def generated(self) -> int:
        """Tokens generated so far, counting launched-but-unseen ones."""
        return len(self.output) + self.pending

    def finish(self) -> None:
        self.kv_cache.release()
        self.finished = True
