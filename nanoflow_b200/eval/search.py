"""Parameter search for an overlapped pipeline: nano-batch split, CTA budget of the collectives, share of
the decode requests scheduled into the last nano-batch.

    python -m nanoflow_b200.eval.search --gpus 8 --model llama2-70B --out tuned/ \
        [--splits 0.40 0.45 0.50 0.55 0.60] [--comm-ctas 64 96 128] [--decode-tail 0 0.25 0.5] [--rounds 2]
        [--nano-counts 2 4] [--switch attn-overlap=0,1 net-streams=1,2]

Every point is one run of the repository's ``bench.py`` (steady-state offline throughput, device timed,
maximum over ranks); the value searched is its tokens/s. The search is coordinate descent: one
parameter is swept while the others stay at their best known values, parameters in turn, for
``--rounds`` rounds or until a round changes nothing; points already measured are not run again. The
result is the four-section configuration of the best point (``<out>/best.json``, loadable by
``nanoflow_b200.serve`` and ``test_compute``) and a log of all points (``<out>/search.csv``).

The reference publishes its nano-batch sizes and block counts as constants in its shipped configs and
source (pipeline/config_all/llama2-70B/2048.json:37-47, pipeline/src/pipeline.cu:677-732) and names an
offline search that is not in the repository; this is that tool for this engine.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import subprocess
import sys
from typing import Callable, Dict, List, Optional, Sequence, Tuple

Point = Tuple[float, int, float]          # (first nano-batch's share of the dense batch, comm CTAs, decode tail share)
Runner = Callable[[Dict], float]

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def split_sizes(gbs: int, share: float, granule: int = 128, count: int = 2) -> List[int]:
    """Nano-batch sizes for a first-nano-batch share, all multiples of ``granule`` (one GEMM M tile) and
    at least one granule. With ``count`` > 2 the rest of the batch is cut into ``count - 1`` equal parts
    (the last one takes the remainder)."""
    if count < 2 or gbs < count * granule:
        raise ValueError("dense batch too small to split")
    first = int(round(gbs * share / granule)) * granule
    first = min(max(first, granule), gbs - (count - 1) * granule)
    if count == 2:
        return [first, gbs - first]
    part = max(granule, (gbs - first) // (count - 1) // granule * granule)
    sizes = [first] + [part] * (count - 2)
    return sizes + [gbs - sum(sizes)]


def coordinate_descent(axes: Dict[str, Sequence], start: Dict, measure: Callable[[Dict], float], rounds: int = 2,
                       log: Optional[List[Dict]] = None, pair_moves: bool = False) -> Tuple[Dict, float]:
    """Maximise ``measure`` over the grid ``axes`` (name -> candidate values) starting from ``start``.
    Returns the best point and its value; ``log`` collects every distinct point measured."""
    cache: Dict[Tuple, float] = {}

    def value(pt: Dict) -> float:
        key = tuple(pt[k] for k in sorted(pt))
        if key not in cache:
            cache[key] = float(measure(dict(pt)))
            if log is not None:
                log.append(dict(pt, value=cache[key]))
        return cache[key]

    best = dict(start)
    best_v = value(best)
    names = list(axes)
    for _ in range(max(1, rounds)):
        changed = False
        for name in names:
            for c in axes[name]:
                if c == best[name]:
                    continue
                trial = dict(best, **{name: c})
                v = value(trial)
                if v > best_v:
                    best, best_v, changed = trial, v, True
        if not changed and pair_moves:
            # Parameters that only pay off together (more nano-batches with the attention overlap, say)
            # are invisible to single moves: when those are exhausted, try changing two at once.
            for i, a in enumerate(names):
                for b in names[i + 1:]:
                    for ca in axes[a]:
                        for cb in axes[b]:
                            if ca == best[a] or cb == best[b]:
                                continue
                            trial = dict(best, **{a: ca, b: cb})
                            v = value(trial)
                            if v > best_v:
                                best, best_v, changed = trial, v, True
        if not changed:
            break
    return best, best_v


def bench_runner(gpus: int, model: str, steps: int, warmup: int, extra: Sequence[str] = (), port: int = 29560) -> Runner:
    """Measure one point by running ``bench.py`` and reading its JSON line."""
    bench = os.path.join(ROOT, "bench.py")

    def run(pt: Dict) -> float:
        args = ["--gpus", str(gpus), "--model", model, "--steps", str(steps), "--warmup", str(warmup), *extra]
        if pt.get("nano"):
            args += ["--nano", ",".join(str(n) for n in pt["nano"])]
        if pt.get("comm_ctas"):
            args += ["--comm-ctas", str(pt["comm_ctas"])]
        if pt.get("decode_tail"):
            args += ["--decode-tail", str(pt["decode_tail"])]
        for flag, v in (pt.get("switches") or {}).items():      # bench.py switches: True -> bare flag, else its value
            if v is True:
                args.append(f"--{flag}")
            elif v not in (False, None, 0):
                args += [f"--{flag}", str(v)]
        if gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), bench, *args]
        else:
            cmd = [sys.executable, bench, *args]
        res = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT)
        for line in reversed(res.stdout.strip().splitlines()):
            if line.startswith("{"):
                out = json.loads(line)
                run.last = out
                return float(out["value"])
        raise RuntimeError(f"bench.py printed no result line:\n{res.stdout[-1000:]}\n{res.stderr[-2000:]}")

    run.last = None
    return run


def search(gbs: int, splits: Sequence[float], comm_ctas: Sequence[int], decode_tail: Sequence[float], runner: Runner,
           rounds: int = 2, start: Optional[Point] = None, nano_counts: Sequence[int] = (2,),
           switches: Optional[Dict[str, Sequence]] = None) -> Tuple[Dict, float, List[Dict]]:
    """Search for a dense batch of ``gbs`` tokens over the first nano-batch's share, the number of
    nano-batches, the collectives' CTA budget, the decode-tail share and any further ``bench.py`` switches
    (``switches``: flag name -> candidate values, ``True`` / ``False`` for bare flags). ``runner`` gets
    ``{"nano": [...], "comm_ctas": c, "decode_tail": f, "switches": {...}}`` and returns tokens/s."""
    log: List[Dict] = []
    switches = dict(switches or {})
    axes = {"share": list(splits), "count": list(nano_counts), "comm_ctas": list(comm_ctas),
            "decode_tail": list(decode_tail)}
    axes.update({f"sw:{k}": list(v) for k, v in switches.items()})
    s0 = start or (min(splits, key=lambda s: abs(s - 0.5)), comm_ctas[0], decode_tail[0])
    first = {"share": s0[0], "count": nano_counts[0], "comm_ctas": s0[1], "decode_tail": s0[2]}
    first.update({f"sw:{k}": v[0] for k, v in switches.items()})

    def share_of(pt: Dict) -> float:          # "half" means an equal split whatever the number of nano-batches
        return pt["share"] * 2.0 / pt["count"]

    def measure(pt: Dict) -> float:
        return runner({"nano": split_sizes(gbs, share_of(pt), count=pt["count"]), "comm_ctas": pt["comm_ctas"],
                       "decode_tail": pt["decode_tail"],
                       "switches": {k[3:]: v for k, v in pt.items() if k.startswith("sw:")}})

    best, v = coordinate_descent(axes, first, measure, rounds, log, pair_moves=len(axes) > 4 or len(nano_counts) > 1)
    for row in log + [best]:
        row["nano"] = split_sizes(gbs, share_of(row), count=row["count"])
        row["switches"] = {k[3:]: row[k] for k in list(row) if k.startswith("sw:")}
    return best, v, log


def write_results(out_dir: str, model: str, gpus: int, gbs: int, pipeline_type: str, best: Dict, value: float,
                  log: List[Dict]) -> List[str]:
    from ..config import make_config

    os.makedirs(out_dir, exist_ok=True)
    cfg = make_config(model, gpu_num=gpus, global_batch_size=gbs, pipeline_type=pipeline_type,
                      nanobatch_sizes=list(best["nano"]))
    cfg["pipeline_configs"].setdefault("sm_budget", {})["comm"] = int(best["comm_ctas"])
    cfg["pipeline_configs"]["decode_tail_fraction"] = float(best["decode_tail"])
    for flag, v in (best.get("switches") or {}).items():        # bench.py flag names -> configuration keys
        key = {"attn-overlap": "attn_overlap", "net-streams": "net_streams", "decode-stages": "decode_stages",
               "fuse-rs": "fuse_gemm_rs", "fuse-rs-staged": "gemm_rs_staged"}.get(flag)
        if key:
            cfg["pipeline_configs"][key] = v
    cfg["pipeline_configs"]["searched"] = {"tokens_per_s": value, "points": len(log),
                                           "switches": best.get("switches") or {}}
    files = [os.path.join(out_dir, "best.json"), os.path.join(out_dir, "search.csv")]
    with open(files[0], "w") as f:
        json.dump(cfg, f, indent=2)
    with open(files[1], "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["nanobatches", "comm_ctas", "decode_tail", "switches", "tokens_per_s"])
        for row in log:
            w.writerow(["+".join(str(n) for n in row["nano"]), row["comm_ctas"], row["decode_tail"],
                        " ".join(f"{k}={v}" for k, v in sorted((row.get("switches") or {}).items())), row["value"]])
    return files


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--model", default="llama2-70B")
    ap.add_argument("--out", required=True)
    ap.add_argument("--splits", nargs="*", type=float, default=[0.40, 0.45, 0.50, 0.55, 0.60])
    ap.add_argument("--comm-ctas", nargs="*", type=int, default=[64, 96, 128])
    ap.add_argument("--decode-tail", nargs="*", type=float, default=[0.0, 0.25, 0.5])
    ap.add_argument("--nano-counts", nargs="*", type=int, default=[2], help="numbers of nano-batches to try")
    ap.add_argument("--switch", nargs="*", default=[], metavar="FLAG=V1,V2",
                    help="further bench.py switches to sweep, e.g. attn-overlap=0,1 net-streams=1,2 ar-wide=0,1 "
                         "(0 / 1 for bare flags)")
    ap.add_argument("--rounds", type=int, default=2)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pipeline", default="", help="default: PLLM on several GPUs, LOCAL on one")
    a = ap.parse_args(argv)
    a.pipeline = a.pipeline or ("PLLM" if a.gpus > 1 else "LOCAL")
    extra = ["--pipeline", a.pipeline]
    runner = bench_runner(a.gpus, a.model, a.steps, a.warmup, extra)
    # one run with the defaults tells the dense batch bench.py picks for this model and GPU count
    base = runner({})
    gbs = int(runner.last["config"]["global_batch"])
    print(f"defaults: {base:.1f} tokens/s at dense batch {gbs}", flush=True)
    bare = {"attn-overlap", "ar-wide", "fuse-rs", "fuse-rs-staged", "serial-attention", "no-fuse-norm"}
    switches: Dict[str, List] = {}
    for item in a.switch:
        flag, _, vals = item.partition("=")
        switches[flag] = [(v not in ("0", "", "false")) if flag in bare else int(v) for v in vals.split(",")]
    best, v, log = search(gbs, a.splits, a.comm_ctas, a.decode_tail, runner, a.rounds, nano_counts=a.nano_counts,
                          switches=switches)
    files = write_results(a.out, a.model, a.gpus, gbs, a.pipeline, best, v, log)
    print(json.dumps({"best": best, "tokens_per_s": v, "defaults_tokens_per_s": base, "points": len(log),
                      "files": files}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
