"""Named ranges around scheduler phases and engine calls: an NVTX range (visible in Nsight Systems)
when CUDA is present plus a ``torch.profiler.record_function`` range (visible in the Chrome trace that
``serve --profile_mode`` writes). The reference wraps the same phases in ``record_function``
(pipeline/utils/serve_8B.py:213-523)."""
from __future__ import annotations

import contextlib


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch
        from torch.profiler import record_function

        on = torch.cuda.is_available()
    except ImportError:  # pragma: no cover
        yield
        return
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        with record_function(name):
            yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
