"""Request traces in the CSV format the frontend reads: ``idx,input_len,output_len,arrival_s[,prompt]``.

Workloads of the reference (datasets/utils/generate_fix_trace.sh:8-21, generate_real_trace.sh:11-52,
datasets/utils/utils.py:37-72, :93-96):

* fixed lengths: 512-512, 1024-512, 512-1024, 128-1024, 512-2, all requests available at t = 0;
* real lengths: (input, output) pairs from a length file such as the Splitwise / LMSYS-Chat-1M /
  ShareGPT tables (``TIMESTAMP,ContextTokens,GeneratedTokens``), filtered to input <= 3072,
  output <= 1024, input + output <= 4096, with exponential inter-arrival times (seed 420) at a
  requested rate, or all at t = 0 for offline runs (rate 0);
* synthetic log-normal lengths (median / sigma per side, clipped), the stand-in when no length file
  is available.

The length tables themselves are data, not code, and are not shipped here; ``real_trace`` takes any
CSV with those three columns.
"""
from __future__ import annotations

import csv
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np

FIXED_WORKLOADS = {"512-512": (512, 512), "1024-512": (1024, 512), "512-1024": (512, 1024),
                   "128-1024": (128, 1024), "512-2": (512, 2)}
ARRIVAL_SEED = 420


def poisson_arrivals(n: int, rate: float, seed: int = ARRIVAL_SEED) -> np.ndarray:
    """Arrival times with exponential gaps of mean 1/rate (rate <= 0: everything at t = 0)."""
    if rate <= 0:
        return np.zeros(n)
    rng = np.random.default_rng(seed)
    return np.cumsum(rng.exponential(1.0 / rate, size=n))


def fixed_trace(input_len: int, output_len: int, n: int, rate: float = 0.0) -> List[Tuple[int, int, float]]:
    t = poisson_arrivals(n, rate)
    return [(input_len, output_len, float(t[i])) for i in range(n)]


def filter_lengths(pairs: Iterable[Tuple[int, int]], max_in: int = 3072, max_out: int = 1024,
                   max_total: int = 4096) -> List[Tuple[int, int]]:
    return [(i, o) for i, o in pairs if 0 < i <= max_in and 0 < o <= max_out and i + o <= max_total]


def read_length_csv(path: str) -> List[Tuple[int, int]]:
    """``TIMESTAMP,ContextTokens,GeneratedTokens`` (header optional) -> [(input, output)]."""
    out = []
    with open(path) as f:
        for row in csv.reader(f):
            if len(row) < 3:
                continue
            try:
                out.append((int(float(row[1])), int(float(row[2]))))
            except ValueError:
                continue   # header
    return out


def real_trace(pairs: Sequence[Tuple[int, int]], n: int, rate: float = 0.0, shuffle_seed: Optional[int] = 0):
    pairs = filter_lengths(pairs)
    if not pairs:
        raise ValueError("no request survives the length filter")
    idx = np.arange(len(pairs))
    if shuffle_seed is not None:
        np.random.default_rng(shuffle_seed).shuffle(idx)
    t = poisson_arrivals(n, rate)
    return [(pairs[idx[i % len(idx)]][0], pairs[idx[i % len(idx)]][1], float(t[i])) for i in range(n)]


def lognormal_lengths(n: int, in_median: float = 600, in_sigma: float = 0.9, in_clip=(16, 4096),
                      out_median: float = 250, out_sigma: float = 0.9, out_clip=(1, 2048), seed: int = 0):
    """Synthetic variable-length stream: log-normal prompt / output lengths, clipped."""
    rng = np.random.default_rng(seed)
    ins = np.clip(np.rint(rng.lognormal(np.log(in_median), in_sigma, n)), *in_clip).astype(int)
    outs = np.clip(np.rint(rng.lognormal(np.log(out_median), out_sigma, n)), *out_clip).astype(int)
    return list(zip(ins.tolist(), outs.tolist()))


def write_trace(path: str, rows: Sequence[Tuple[int, int, float]]) -> None:
    with open(path, "w") as f:
        f.write("idx,input_len,output_len,arrival\n")
        for i, (a, b, t) in enumerate(rows):
            f.write(f"{i},{a},{b},{t}\n")
