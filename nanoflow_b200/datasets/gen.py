"""Generate the standard trace files (the role of datasets/gen.sh in the reference).

    python -m nanoflow_b200.datasets.gen --out traces/ [--n 20000] [--lengths splitwise.csv ...]
        [--rates 0 5 10 20 ...]

Writes ``fixed-<in>-<out>.csv`` for the five fixed workloads, ``lognormal-<rate>.csv`` for the synthetic
variable-length stream and, for every length file given, ``<name>-<rate>.csv``.
"""
from __future__ import annotations

import argparse
import os

from .traces import (FIXED_WORKLOADS, fixed_trace, lognormal_lengths, poisson_arrivals, read_length_csv, real_trace,
                     write_trace)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--n", type=int, default=20000)
    ap.add_argument("--lengths", nargs="*", default=[])
    ap.add_argument("--rates", nargs="*", type=float, default=[0.0])
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    for name, (i, o) in FIXED_WORKLOADS.items():
        write_trace(os.path.join(a.out, f"fixed-{name}.csv"), fixed_trace(i, o, a.n))
    pairs = lognormal_lengths(a.n)
    for rate in a.rates:
        t = poisson_arrivals(a.n, rate)
        write_trace(os.path.join(a.out, f"lognormal-{rate:g}.csv"), [(p[0], p[1], float(t[k])) for k, p in enumerate(pairs)])
        for path in a.lengths:
            base = os.path.splitext(os.path.basename(path))[0]
            write_trace(os.path.join(a.out, f"{base}-{rate:g}.csv"), real_trace(read_length_csv(path), a.n, rate))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
