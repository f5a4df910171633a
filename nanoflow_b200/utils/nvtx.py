"""NVTX ranges around scheduler phases and engine calls (visible in Nsight Systems), as no-ops when
CUDA is absent. The reference wraps the same phases in ``torch.profiler.record_function``
(pipeline/utils/serve_8B.py:213-523)."""
from __future__ import annotations

import contextlib


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch

        on = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        on = False
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
