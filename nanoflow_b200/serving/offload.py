"""KV offload of retired requests to pinned host memory, and reload.

When a request stops, its KV pages are not returned to the pool at once: the next iteration gathers
them layer by layer on the copy stream and copies them to pinned host memory beside the layer's
compute (engine side: ``runtime/pipeline.py:offload_layer``); once that iteration has completed the
host copy is filed under the request id and the pages are released. ``restore`` puts a stored
request back into freshly allocated pages (host -> device copy + page scatter), e.g. to continue a
multi-round conversation without recomputing its prompt.

The reference emulates the traffic only (fixed sizes, identity indices, D2H immediately followed by
H2D; pipeline/src/pipeline.cu:37-61, :701-726, :915-931); this one moves the real pages.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .kv_cache import DistKVCache
from .request import FlyRequestInfo
from .scheduler import BatchPlan, Scheduler


@dataclass
class StoredKV:
    req_idx: int
    seqlen: int
    data: torch.Tensor          # [layers, n_pages, page_elems] on the host


class KVOffloadManager:
    def __init__(self, engine, max_host_bytes: int = 8 << 30):
        if getattr(engine, "offload_cap", 0) <= 0:
            raise ValueError("engine was built without offload (use a PLLM_OFFLOAD config)")
        self.engine = engine
        self.max_host_bytes = max_host_bytes
        self.store: Dict[int, StoredKV] = {}
        self.bytes = 0
        # totals since start (what left the GPU, whether or not the host store still keeps it)
        self.total_requests = 0
        self.total_pages = 0
        self.total_bytes = 0
        self.dropped_requests = 0               # retired beyond the per-iteration staging capacity
        self._pending: Dict[int, List] = {}     # iteration -> [(req, n_pages)] in page order

    # ---- hooks called by the serving loop --------------------------------------------------------
    def on_iteration(self, plan: BatchPlan) -> None:
        """Remember which retired requests ride on this iteration's offload (page order = request order)."""
        if not plan.retired_reqs:
            return
        cap, used, lst = self.engine.offload_cap, 0, []
        for req in plan.retired_reqs:
            n = req.kv_cache.num_pages
            if used + n > cap:
                self.dropped_requests += len(plan.retired_reqs) - len(lst)
                break                              # beyond the per-iteration staging: dropped, not offloaded
            lst.append((req, used, n, req.kv_cache.seqlen))
            used += n
        self._pending[plan.iteration] = lst

    def on_complete(self, plan: BatchPlan, scheduler: Scheduler) -> None:
        lst = self._pending.pop(plan.iteration, [])
        if lst:
            host = self.engine.offloaded_pages()
            for req, off, n, seqlen in lst:
                data = host[:, off:off + n].clone()
                nbytes = data.numel() * data.element_size()
                while self.store and self.bytes + nbytes > self.max_host_bytes:
                    _, old = self.store.popitem()
                    self.bytes -= old.data.numel() * old.data.element_size()
                self.store[req.req_idx] = StoredKV(req.req_idx, seqlen, data)
                self.bytes += nbytes
                self.total_requests += 1
                self.total_pages += n
                self.total_bytes += nbytes
                req.offloaded = True
        scheduler.release_held_pages(plan.iteration)

    # ---- reload ------------------------------------------------------------------------------------
    def restore(self, req_idx: int, kv: DistKVCache) -> int:
        """Copy a stored request into the pages of ``kv`` (which must hold exactly its length).
        Returns the restored sequence length. Runs eagerly on the current stream."""
        from .. import ops

        st = self.store[req_idx]
        if kv.seqlen != st.seqlen or kv.num_pages != st.data.shape[1]:
            raise ValueError("target KV cache must be allocated for the stored sequence length")
        dev = self.engine.device
        ids = torch.from_numpy(np.ascontiguousarray(kv.indicies)).to(dev)
        for l, pool in enumerate(self.engine.bufs.kv_pool):
            staging = st.data[l].to(dev, non_blocking=True)
            ops.kv_move_pages(pool, staging, ids, to_staging=False, status=self.engine.bufs.status)
        return st.seqlen
