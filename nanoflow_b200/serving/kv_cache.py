"""Paged KV-cache bookkeeping (page ids only; the memory lives in the engine's device pool).

Same roles and names as the reference's ``pipeline/utils/kv_cache.py``: :class:`DistKVPool` (free
pages, identical on every GPU because attention is head-parallel, kv_cache.py:20-65),
:class:`DistKVCache` (page list + sequence length of one request, :67-105) and
:class:`BatchedDistKVCache` (flattens a batch into ``kv_indices / kv_indptr / kv_last_page_len``,
decode requests first, :107-158). Differences: the free list is a NumPy stack (O(1) bulk
alloc/free, deterministic order so replicated schedulers on all ranks agree), running out of pages
raises :class:`KVPoolExhausted` instead of tripping an ``assert``, and batch flattening is vectorised.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np


class KVPoolExhausted(RuntimeError):
    """Raised when an allocation asks for more pages than are free."""


class DistKVPool:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, capacity: int, page_size: int,
                 num_devices: int = 1):
        if num_devices > 0 and num_kv_heads % num_devices:
            raise ValueError("num_kv_heads must be divisible by num_devices")
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.capacity, self.page_size, self.num_devices = int(capacity), int(page_size), num_devices
        # stack of free ids; pop from the end. Lowest ids come out first.
        self._free = np.arange(self.capacity - 1, -1, -1, dtype=np.int32)
        self._nfree = self.capacity
        self._is_free = np.ones(self.capacity, dtype=bool)

    @property
    def num_free_pages(self) -> int:
        return self._nfree

    @property
    def num_used_pages(self) -> int:
        return self.capacity - self._nfree

    def alloc_pages(self, n: int) -> np.ndarray:
        if n < 0 or n > self._nfree:
            raise KVPoolExhausted(f"need {n} pages, {self._nfree} free of {self.capacity}")
        out = self._free[self._nfree - n:self._nfree][::-1].copy()
        self._nfree -= n
        self._is_free[out] = False
        return out

    def alloc_page(self) -> int:
        return int(self.alloc_pages(1)[0])

    def free_pages(self, ids) -> None:
        ids = np.asarray(ids, dtype=np.int32)
        if ids.size == 0:
            return
        if (ids < 0).any() or (ids >= self.capacity).any() or self._is_free[ids].any() or \
                np.unique(ids).size != ids.size:
            raise ValueError("free_pages: invalid or already-free page id")
        self._free[self._nfree:self._nfree + ids.size] = ids[::-1]
        self._nfree += ids.size
        self._is_free[ids] = True

    def free_page(self, idx: int) -> None:
        self.free_pages([idx])


class DistKVCache:
    """Page list and length of one request. ``allocate_tokens`` grows it, ``release`` frees it."""

    __slots__ = ("_pool", "_pages", "_npages", "_seqlen")

    def __init__(self, pool: DistKVPool):
        self._pool = pool
        self._pages = np.empty(8, dtype=np.int32)
        self._npages = 0
        self._seqlen = 0

    @property
    def seqlen(self) -> int:
        return self._seqlen

    @property
    def indicies(self) -> np.ndarray:  # spelling kept from the reference API
        return self._pages[:self._npages]

    indices = indicies

    @property
    def num_pages(self) -> int:
        return self._npages

    @property
    def last_page_offset(self) -> int:
        return (self._seqlen - 1) % self._pool.page_size + 1

    def pages_needed(self, num_tokens: int) -> int:
        ps = self._pool.page_size
        return (self._seqlen + num_tokens + ps - 1) // ps - self._npages

    def allocate_tokens(self, num_tokens: int) -> None:
        if num_tokens <= 0:
            raise ValueError("allocate_tokens needs a positive token count")
        need = self.pages_needed(num_tokens)
        if need > 0:
            new = self._pool.alloc_pages(need)
            if self._npages + need > self._pages.size:
                grown = np.empty(max(2 * self._pages.size, self._npages + need), dtype=np.int32)
                grown[:self._npages] = self._pages[:self._npages]
                self._pages = grown
            self._pages[self._npages:self._npages + need] = new
            self._npages += need
        self._seqlen += num_tokens

    def release(self) -> None:
        self._pool.free_pages(self._pages[:self._npages])
        self._npages = 0
        self._seqlen = 0


class BatchedDistKVCache:
    """Flatten the page tables of a batch, decode requests first, then prefill requests."""

    def __init__(self, decode_kvs: Sequence[DistKVCache], prefill_kvs: Sequence[DistKVCache]):
        kvs: List[DistKVCache] = list(decode_kvs) + list(prefill_kvs)
        counts = np.fromiter((kv.num_pages for kv in kvs), dtype=np.int32, count=len(kvs))
        self.kv_indptr = np.zeros(len(kvs) + 1, dtype=np.int32)
        np.cumsum(counts, out=self.kv_indptr[1:])
        self.kv_indices = (np.concatenate([kv.indicies for kv in kvs]).astype(np.int32, copy=False)
                           if kvs else np.zeros(0, dtype=np.int32))
        self.kv_last_page_len = np.fromiter((kv.last_page_offset for kv in kvs), dtype=np.int32,
                                            count=len(kvs))
        self.seqlens = np.fromiter((kv.seqlen for kv in kvs), dtype=np.int32, count=len(kvs))

    def toCPUPinned(self):
        """Pinned torch copies of the three arrays (the reference's hand-off format)."""
        import torch

        pin = torch.cuda.is_available()
        mk = lambda a: (torch.from_numpy(a.copy()).pin_memory() if pin else torch.from_numpy(a.copy()))
        self.pinned_kv_indices, self.pinned_kv_indptr = mk(self.kv_indices), mk(self.kv_indptr)
        self.pinned_kv_last_page_len = mk(self.kv_last_page_len)
        return self.pinned_kv_indices, self.pinned_kv_indptr, self.pinned_kv_last_page_len
