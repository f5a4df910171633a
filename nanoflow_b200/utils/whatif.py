"""What-if replay of an op graph with given op durations.

``simulate`` walks the ops in issue order, starts each one when its stream is free and its
dependencies have ended, and returns start / end times, the length of the iteration, how long every
stream was busy and the chain of ops that determines the end (critical path). It knows nothing about
SMs, links or clocks: kernels that share the GPU in reality slow each other down, here a duration is
what it is given. Its use is to take the durations measured in one timeline
(``bench.py --timeline``) and ask what the same kernels would add up to under another schedule: a
second network stream, decode requests spread over the nano-batches, another nano-batch split.

    python -m nanoflow_b200.utils.whatif tl8.json --tp 8 --nano 4096,4096 [--net-streams 2]
        [--attn-overlap] [--cross-layer] [--scale attn_decode.nb0=0.5 attn_decode.nb1=+167]

The reference's only schedule tooling plots per-cycle batch sizes after the fact
(pipeline/utils/plotSchedule.py:1-52); it has no model of the per-layer op schedule.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from typing import Dict, List, Optional, Sequence, Tuple

from ..runtime.graph import OpGraph


def simulate(graph: OpGraph, durations: Sequence[float], single_stream: bool = False) -> dict:
    """``durations[i]`` in microseconds for op i. ``after_start`` edges delay an op until the named op
    has started."""
    n = len(graph.ops)
    if len(durations) != n:
        raise ValueError("one duration per op")
    start, end = [0.0] * n, [0.0] * n
    why: List[Optional[int]] = [None] * n          # the op whose end (or the stream predecessor) set the start
    free: Dict[str, Tuple[float, Optional[int]]] = {}
    for i, op in enumerate(graph.ops):
        s = "all" if single_stream else op.stream
        t, src = free.get(s, (0.0, None))
        for d in op.deps:
            if end[d] > t:
                t, src = end[d], d
        for d in op.after_start:
            if start[d] > t:
                t, src = start[d], d
        e = t + float(durations[i])
        for d in getattr(op, "gated", ()):        # fed row block by row block: done no earlier than its feeder
            if end[d] > e:
                e = end[d]
        start[i], end[i], why[i] = t, e, src
        free[s] = (end[i], i)
    last = max(range(n), key=lambda i: end[i]) if n else None
    path = []
    i = last
    while i is not None:
        path.append(i)
        i = why[i]
    busy: Dict[str, float] = {}
    for i, op in enumerate(graph.ops):
        busy[op.stream] = busy.get(op.stream, 0.0) + float(durations[i])
    return {"makespan": end[last] if n else 0.0, "start": start, "end": end, "busy": busy, "critical_path": path[::-1]}


def stream_gaps(graph: OpGraph, sim: dict, stream: str) -> float:
    """Idle time on ``stream`` between its first op's start and its last op's end."""
    ops = [i for i, op in enumerate(graph.ops) if op.stream == stream]
    if not ops:
        return 0.0
    span = max(sim["end"][i] for i in ops) - min(sim["start"][i] for i in ops)
    return span - sum(sim["end"][i] - sim["start"][i] for i in ops)


def durations_from_timeline(graph: OpGraph, events: Sequence[dict], default_us: float = 3.0,
                            launch_gap_us: float = 0.0) -> List[float]:
    """Durations by op name from a Chrome-trace event list (``ph == "X"``, ``dur`` in microseconds).
    Ops without an event get ``default_us``; ``launch_gap_us`` is added to every op (the distance between
    consecutive launches on a stream)."""
    by_name = {e["name"]: float(e["dur"]) for e in events if e.get("ph") == "X"}
    return [by_name.get(op.name, default_us) + launch_gap_us for op in graph.ops]


def scale_durations(graph: OpGraph, durations: Sequence[float], rules: Dict[str, str]) -> List[float]:
    """``rules``: "<op kind>.nb<k>" or "<op kind>" -> "0.5" (factor) or "+167" / "-20" (microseconds added),
    applied to every layer's op of that kind (the name's last component) and nano-batch."""
    out = list(durations)
    for i, op in enumerate(graph.ops):
        kind = op.name.split(".")[-1]
        for key in (f"{kind}.nb{op.nano}", kind):
            if key in rules:
                r = rules[key]
                out[i] = max(0.0, out[i] + float(r)) if r[0] in "+-" else out[i] * float(r)
                break
    return out


def structural_graph(tp: int, nano: Sequence[int], layers: int, pipeline_type: str = "", net_streams: int = 1,
                     prefill_beside_decode: bool = True, attn_overlap: bool = False,
                     cross_layer: bool = False) -> OpGraph:
    """The op graph of a pipeline with the tiny model's tensors on the CPU: op names, streams and
    dependencies are those of any model with the same layer count, tensor-parallel degree and
    nano-batch count."""
    import torch

    from ..config import builtin_config
    from ..models import random_full_weights, shard_weights
    from ..parallel.collectives import TpCollectives
    from ..runtime.pipeline import Buffers, IoSpec, build_graph

    tp = 2 if tp > 1 else 1      # the structure is the same for every degree above one; the tiny model shards two ways
    gbs = 16 * len(nano) * 3
    sizes = [gbs // len(nano)] * len(nano)
    ptype = pipeline_type or ("PLLM" if tp > 1 else ("LOCAL" if len(nano) > 1 else "NON_OVERLAP_LOCAL"))
    cfg = builtin_config("tiny", gpu_num=tp, global_batch_size=gbs, pipeline_type=ptype,
                         nanobatch_sizes=sizes if len(nano) > 1 else None, run_layer=layers)
    m, e = cfg.model, cfg.engine
    e.max_batch_size, e.net_streams, e.prefill_beside_decode = gbs, net_streams, prefill_beside_decode
    e.attn_overlap = attn_overlap
    e.cross_layer_pipeline = cross_layer
    w = shard_weights(random_full_weights(m, seed=0), m, 0, tp, dtype=torch.bfloat16)
    coll = TpCollectives.for_analysis(0, tp) if tp > 1 else None
    bf = torch.bfloat16
    z = lambda *s, dtype=bf: torch.zeros(*s, dtype=dtype)
    sym = (lambda *s, dtype=bf: coll.alloc(s, dtype)) if coll else z
    T = B = gbs
    meta_dev = torch.zeros(8 * T + 8 * B + 4096, dtype=torch.int32)
    names = ["host_ids", "feedback_src", "positions", "token_req", "qo_indptr", "kv_indptr", "kv_last_page_len",
             "sample_rows", "kv_indices"]
    meta = {nm: meta_dev[i * (T + 8):(i + 1) * (T + 8)] for i, nm in enumerate(names)}
    x0 = z(T, m.hidden_size)
    pools = [z(16, 2, m.kv_heads_local, 16, m.head_dim) for _ in range(m.run_layers)]
    bufs = Buffers(x=[x0, sym(T + 8 * len(sizes), m.hidden_size) if tp > 1 else x0], h=sym(T, m.hidden_size),
                   qkv=z(T, m.qkv_size_local), q_rot=z(T, m.q_size_local), attn_out=z(T, m.q_size_local),
                   act=z(T, m.ffn_local), sample_h=z(B, m.hidden_size), sample_hn=z(B, m.hidden_size),
                   logits=z(B, w.lm_head.shape[0]), cand_val=sym(tp, B, dtype=torch.float32),
                   cand_idx=sym(tp, B, dtype=torch.int32), sampled=z(B, dtype=torch.int32), kv_pool=pools,
                   inv_freq=torch.zeros(m.head_dim // 2), status=torch.zeros(1, dtype=torch.int32),
                   decode_ws=torch.zeros(1024), meta=meta,
                   nano_items=[torch.zeros(s + 2, 3, dtype=torch.int32) for s in sizes],
                   gemm_ws=torch.zeros(1 << 16))
    g = build_graph(m, e, w, bufs, coll, IoSpec(meta_dev, 4 * T, 8 * T))
    g._keep = (bufs, w, coll, meta_dev)      # parameter blocks point into these
    return g


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("timeline", help="Chrome trace written by bench.py --timeline")
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--nano", default="4096,4096")
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--pipeline", default="")
    ap.add_argument("--net-streams", type=int, default=1)
    ap.add_argument("--serial-attention", action="store_true")
    ap.add_argument("--attn-overlap", action="store_true")
    ap.add_argument("--cross-layer", action="store_true", help="software pipeline across layers (skewed under TP)")
    ap.add_argument("--launch-gap", type=float, default=2.7, help="microseconds between launches on a stream")
    ap.add_argument("--scale", nargs="*", default=[], help="<kind>[.nb<k>]=<factor | +us | -us>")
    ap.add_argument("--pid", type=int, default=0)
    a = ap.parse_args(argv)
    with open(a.timeline) as f:
        d = json.load(f)
    events = [e for e in (d["traceEvents"] if isinstance(d, dict) else d) if e.get("pid", 0) == a.pid]
    nano = [int(x) for x in a.nano.split(",")]
    g = structural_graph(a.tp, nano, a.layers, a.pipeline, a.net_streams, not a.serial_attention, a.attn_overlap,
                         a.cross_layer)
    dur = durations_from_timeline(g, events, launch_gap_us=a.launch_gap)
    rules = dict(r.split("=", 1) for r in a.scale)
    dur = scale_durations(g, dur, rules)
    sim = simulate(g, dur)
    kinds: Dict[str, float] = {}
    for i in sim["critical_path"]:
        k = re.sub(r"^L\d+\.", "", g.ops[i].name)
        kinds[k] = kinds.get(k, 0.0) + dur[i]
    print(json.dumps({"iteration_ms": round(sim["makespan"] / 1e3, 2),
                      "busy_ms": {s: round(v / 1e3, 2) for s, v in sim["busy"].items()},
                      "compute_stream_idle_ms": round(stream_gaps(g, sim, "gemm") / 1e3, 2),
                      "critical_path_ms": {k: round(v / 1e3, 2) for k, v in sorted(kinds.items(), key=lambda x: -x[1])}},
                     indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
