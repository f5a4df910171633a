"""Per-iteration op timeline: CUDA-event timestamps of every op of the graph, aggregated by op kind
and exportable as a Chrome / Perfetto trace (one track per stream class).

The reference times whole iterations with ``cudaEventElapsedTime`` and prints them
(pipeline/src/pipeline.cu:765-779) and wraps scheduler phases in ``torch.profiler.record_function``
(pipeline/utils/serve_8B.py:213-523); op-level timelines there need Nsight Systems.
"""
from __future__ import annotations

import json
import re
from collections import defaultdict
from typing import Dict, Iterable, List, Tuple

Event = Tuple[str, str, float, float]   # (op name, stream class, start_us, end_us)


def op_kind(name: str) -> str:
    """``L12.nb1.gate_up`` -> ``gate_up``; ``lm_head`` -> ``lm_head``."""
    return name.split(".")[-1]


def aggregate(events: Iterable[Event]) -> Dict[str, Dict[str, float]]:
    """Sum of (end - start) per op kind. Note: an op's interval includes time it spent queued behind
    other work on its stream only when events are recorded without gaps; treat sums as upper bounds."""
    agg: Dict[str, Dict[str, float]] = defaultdict(lambda: {"count": 0, "total_us": 0.0})
    for name, _stream, a, b in events:
        k = op_kind(name)
        agg[k]["count"] += 1
        agg[k]["total_us"] += b - a
    span = 0.0
    ev = list(events)
    if ev:
        span = max(e[3] for e in ev) - min(e[2] for e in ev)
    out = {k: {"count": int(v["count"]), "total_us": round(v["total_us"], 1),
               "share": round(v["total_us"] / span, 4) if span else 0.0} for k, v in agg.items()}
    out["_iteration"] = {"count": 1, "total_us": round(span, 1), "share": 1.0}
    return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_us"]))


def to_chrome_trace(events: Iterable[Event], pid: int = 0) -> dict:
    tids = {}
    out = []
    for name, stream, a, b in events:
        tid = tids.setdefault(stream, len(tids))
        out.append({"name": name, "cat": op_kind(name), "ph": "X", "ts": a, "dur": max(b - a, 0.001),
                    "pid": pid, "tid": tid})
    for stream, tid in tids.items():
        out.append({"name": "thread_name", "ph": "M", "pid": pid, "tid": tid, "args": {"name": f"stream:{stream}"}})
    return {"traceEvents": out, "displayTimeUnit": "ms"}


def dump(events: List[Event], path: str, pid: int = 0) -> None:
    with open(path, "w") as f:
        json.dump({"aggregate": aggregate(events), **to_chrome_trace(events, pid)}, f)


def dump_ranks(per_rank: List[List[Event]], path: str) -> Dict[str, Dict[str, float]]:
    """One trace file with a process per rank, plus per rank the busy time of its compute stream and the
    total time of its collectives: on the ranks that reach a collective early its duration contains the
    wait for the last rank, so a rank whose collectives are short and whose compute stream is busiest
    is the one the others wait for."""
    events: List[dict] = []
    summary: Dict[str, Dict[str, float]] = {}
    for rank, ev in enumerate(per_rank):
        tr = to_chrome_trace(ev, pid=rank)
        events.extend(tr["traceEvents"])
        events.append({"name": "process_name", "ph": "M", "pid": rank, "args": {"name": f"rank {rank}"}})
        span = (max(e[3] for e in ev) - min(e[2] for e in ev)) if ev else 0.0
        summary[f"rank{rank}"] = {
            "iteration_us": round(span, 1),
            "compute_stream_busy_us": round(sum(b - a for _n, st, a, b in ev if st == "gemm"), 1),
            "collectives_us": round(sum(b - a for n, _st, a, b in ev if op_kind(n).startswith(("ar_", "ag_"))), 1)}
    with open(path, "w") as f:
        json.dump({"ranks": summary, "aggregate": aggregate(per_rank[0]) if per_rank else {},
                   "traceEvents": events, "displayTimeUnit": "ms"}, f)
    return summary
