"""Guard words around activation buffers (debug aid for out-of-bounds writes).

Every buffer handed out by :class:`GuardedArena` sits between two guard regions filled with a fixed
bit pattern. ``check()`` compares the guards with the pattern and names the buffers whose neighbour
bytes changed, and on which side: a kernel that writes past the rows or columns it was given shows
up after the iteration that did it, without a memory-checking tool attached. The engine turns this
on with ``debug_guards`` in the pipeline configuration and checks after every iteration.

The reference has nothing comparable: its bump allocator hands out adjacent ranges of one scratch
buffer (pipeline/include/allocManager.cuh:26-61), so an overrun lands silently in the next tensor.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

GUARD_BYTES = 512
PATTERN = 0x5A


@dataclass
class _Entry:
    name: str
    raw: torch.Tensor        # uint8: [guard | payload (padded to 16 B) | guard]
    payload_bytes: int


class GuardedArena:
    def __init__(self, device, guard_bytes: int = GUARD_BYTES):
        if guard_bytes <= 0 or guard_bytes % 16:
            raise ValueError("guard_bytes must be a positive multiple of 16")
        self.device = torch.device(device)
        self.guard_bytes = guard_bytes
        self._entries: List[_Entry] = []
        self._names: Dict[str, int] = {}

    def zeros(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A zero-filled tensor of ``shape`` whose storage is fenced by guard bytes on both sides."""
        n = 1
        for s in shape:
            n *= int(s)
        esz = torch.empty((), dtype=dtype).element_size()
        payload = (n * esz + 15) // 16 * 16
        g = self.guard_bytes
        raw = torch.zeros(g + payload + g, dtype=torch.uint8, device=self.device)
        raw[:g] = PATTERN
        raw[g + n * esz:] = PATTERN          # padding bytes after the last element belong to the rear guard
        count = self._names.get(name, 0)
        self._names[name] = count + 1
        self._entries.append(_Entry(name if count == 0 else f"{name}#{count}", raw, n * esz))
        return raw[g:g + n * esz].view(dtype).view(*shape)

    def check(self) -> List[Tuple[str, str, int]]:
        """``(buffer, "front" | "rear", first corrupted byte offset within that guard)`` per damaged guard."""
        bad: List[Tuple[str, str, int]] = []
        g = self.guard_bytes
        for e in self._entries:
            for side, region in (("front", e.raw[:g]), ("rear", e.raw[g + e.payload_bytes:])):
                wrong = region != PATTERN
                if bool(wrong.any()):
                    bad.append((e.name, side, int(torch.nonzero(wrong)[0, 0])))
        return bad

    def restore(self) -> None:
        """Rewrite all guards (after a reported corruption, so the next check starts clean)."""
        g = self.guard_bytes
        for e in self._entries:
            e.raw[:g] = PATTERN
            e.raw[g + e.payload_bytes:] = PATTERN

    def __len__(self) -> int:
        return len(self._entries)
