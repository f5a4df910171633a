"""Logging helpers: a per-rank file logger and a tensor dumper.

The reference has a global spdlog logger plus one file logger per rank (``log_<rank>.txt``,
pipeline/src/pipeline.cu:15-19) and ``log_tensor`` (pipeline/include/tensorLogger.cuh:24-67), which
synchronises, copies a window of a tensor to the host and prints it. Same two tools here.
"""
from __future__ import annotations

import logging
import os
from typing import Optional

_LOGGERS = {}


def rank_logger(rank: int = 0, directory: str = ".", level=logging.INFO, to_stderr: bool = False) -> logging.Logger:
    """Logger writing to ``<directory>/log_<rank>.txt`` (created once per rank)."""
    key = (rank, os.path.abspath(directory))
    if key in _LOGGERS:
        return _LOGGERS[key]
    lg = logging.getLogger(f"nanoflow_b200.rank{rank}")
    lg.setLevel(level)
    lg.propagate = False
    os.makedirs(directory, exist_ok=True)
    fh = logging.FileHandler(os.path.join(directory, f"log_{rank}.txt"), mode="w")
    fh.setFormatter(logging.Formatter("%(asctime)s [%(levelname)s] %(message)s"))
    lg.addHandler(fh)
    if to_stderr:
        lg.addHandler(logging.StreamHandler())
    _LOGGERS[key] = lg
    return lg


def log_tensor(logger: logging.Logger, tensor, name: str, rows: int = 4, cols: int = 8,
               row0: int = 0, col0: int = 0) -> str:
    """Synchronise, copy a [rows, cols] window of a 1-D / 2-D tensor to the host and log it with
    shape, dtype, min / max / mean and a NaN count. Returns the logged text."""
    import torch

    t = tensor.detach()
    if t.is_cuda:
        torch.cuda.synchronize(t.device)
    t2 = t.reshape(1, -1) if t.dim() == 1 else t.reshape(t.shape[0], -1)
    win = t2[row0:row0 + rows, col0:col0 + cols].float().cpu()
    f = t2.float()
    text = (f"{name}: shape={tuple(t.shape)} dtype={t.dtype} min={f.min().item():.5g} max={f.max().item():.5g} "
            f"mean={f.mean().item():.5g} nan={int(torch.isnan(f).sum())}\n{win}")
    logger.info(text)
    return text
