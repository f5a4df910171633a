"""Experiment runner: spawns ``python -m nanoflow_b200.serve`` once per experiment point and collects
``<prefix>.stat.csv`` files into one results JSON. Finished points are skipped on re-run (their
result file exists), so an interrupted sweep resumes where it stopped.

    python -m nanoflow_b200.eval.harness fixed-offline --model llama2-70B --gpus 8 --out results/
    python -m nanoflow_b200.eval.harness real-offline  --model llama2-70B --gpus 8 --traces traces/ --out results/
    python -m nanoflow_b200.eval.harness online        --model llama3-70B --gpus 8 --rates 5 10 20 40 60 --out results/
    python -m nanoflow_b200.eval.harness ablation      --model llama2-70B --gpus 8 --out results/
    python -m nanoflow_b200.eval.harness summarize     --out results/
    python -m nanoflow_b200.eval.harness merge         --model llama2-70B --out results/   # pllm.json, the reference's layout
    python -m nanoflow_b200.eval.harness plot          --out results/                      # figures from pllm.json

Experiment families and defaults follow the reference (pipeline/eval/eval-fix-offline/run.py:42-50:
empty weights, skip cycles then 1500 run cycles; pipeline/eval/eval-real-online-2048/run.py:45-49,
:86-95: request-rate sweep per dense batch size; pipeline/eval/eval-ablation/run.py:20, :49-57:
non-overlap / nanobatch-only / full / offload; pipeline/eval/summarize.py:76-176).
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import subprocess
import sys
from typing import Dict, List, Optional

from ..config import CONFIG_DIR, make_config, shipped_variants
from ..datasets.traces import FIXED_WORKLOADS, fixed_trace, lognormal_lengths, poisson_arrivals, write_trace
from .baseline_data import OFFLINE_FIXED, OPTIMAL_LLAMA2_70B_A100, speedup_table


def _serve_cmd(gpus: int, args: List[str], port: int = 29540) -> List[str]:
    if gpus > 1:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
                "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "nanoflow_b200.serve", *args]
    return [sys.executable, "-m", "nanoflow_b200.serve", *args]


def run_point(name: str, out_dir: str, config: Dict, trace_rows, *, gpus: int, run_cycles: int, skip_cycles: int,
              online: bool = False, est_cycle_time: float = 0.1, backend: str = "gpu", dry_run: bool = False) -> Optional[Dict]:
    os.makedirs(out_dir, exist_ok=True)
    prefix = os.path.join(out_dir, name)
    if os.path.exists(prefix + ".stat.csv"):
        return read_stat(prefix + ".stat.csv")              # resume: point already done
    cfg_path, trace_path = prefix + ".config.json", prefix + ".trace.csv"
    with open(cfg_path, "w") as f:
        json.dump(config, f, indent=1)
    write_trace(trace_path, trace_rows)
    args = ["-t", trace_path, "-c", cfg_path, "-r", str(run_cycles), "-s", str(skip_cycles), "--empty_weight", "True",
            "--est_cycle_time", str(est_cycle_time), "-o", prefix, "--backend", backend]
    if online:
        args += ["--online", "True", "--until_empty", "True"]
    cmd = _serve_cmd(gpus, args)
    if dry_run:
        print(" ".join(cmd))
        return None
    res = subprocess.run(cmd, capture_output=True, text=True)
    with open(prefix + ".log", "w") as f:
        f.write(res.stdout + res.stderr)
    if res.returncode != 0 or not os.path.exists(prefix + ".stat.csv"):
        raise RuntimeError(f"experiment {name} failed, see {prefix}.log")
    return read_stat(prefix + ".stat.csv")


def read_stat(path: str) -> Dict[str, float]:
    with open(path) as f:
        rows = list(csv.DictReader(f))
    return {k: float(v) for k, v in rows[0].items()}


def _n_requests(gbs: int, cycles: int, in_len: int, out_len: int) -> int:
    return int(cycles * gbs / (in_len + out_len)) + 4 * gbs // max(1, out_len) + 64


def fixed_offline(a) -> Dict:
    out = {}
    for wl, (i, o) in FIXED_WORKLOADS.items():
        if a.workloads and wl not in a.workloads:
            continue
        cfg = make_config(a.model, gpu_num=a.gpus, global_batch_size=a.batch)
        rows = fixed_trace(i, o, _n_requests(a.batch, a.skip_cycles + a.run_cycles, i, o))
        out[wl] = run_point(f"fixed-{a.model}-{wl}", a.out, cfg, rows, gpus=a.gpus, run_cycles=a.run_cycles,
                            skip_cycles=a.skip_cycles, backend=a.backend, dry_run=a.dry_run)
    return out


def real_offline(a) -> Dict:
    from ..datasets.traces import read_length_csv, real_trace

    out = {}
    sources = {}
    if a.traces and os.path.isdir(a.traces):
        for fn in sorted(os.listdir(a.traces)):
            if fn.endswith(".csv"):
                sources[os.path.splitext(fn)[0]] = read_length_csv(os.path.join(a.traces, fn))
    if not sources:
        sources["lognormal"] = lognormal_lengths(50000)
    for name, pairs in sources.items():
        cfg = make_config(a.model, gpu_num=a.gpus, global_batch_size=a.batch)
        rows = real_trace(pairs, _n_requests(a.batch, a.skip_cycles + a.run_cycles, 600, 250))
        out[name] = run_point(f"real-{a.model}-{name}", a.out, cfg, rows, gpus=a.gpus, run_cycles=a.run_cycles,
                              skip_cycles=a.skip_cycles, backend=a.backend, dry_run=a.dry_run)
    return out


def online(a) -> Dict:
    out = {}
    pairs = lognormal_lengths(a.requests)
    for rate in a.rates:
        t = poisson_arrivals(a.requests, rate)
        rows = [(p[0], p[1], float(t[k])) for k, p in enumerate(pairs)]
        cfg = make_config(a.model, gpu_num=a.gpus, global_batch_size=a.batch,
                          pipeline_type="PLLM_OFFLOAD" if a.offload and a.gpus > 1 else None)
        out[f"{rate:g}"] = run_point(f"online-{a.model}-b{a.batch}-r{rate:g}", a.out, cfg, rows, gpus=a.gpus,
                                     run_cycles=a.run_cycles, skip_cycles=0, online=True, backend=a.backend,
                                     dry_run=a.dry_run)
    return out


def ablation(a) -> Dict:
    out = {}
    variants = shipped_variants(a.model)
    for name in ("non-overlap", "nanobatch-only", "2048", "pllm-offload"):
        if name not in variants:
            continue
        cfg = variants[name]
        cfg["model_configs"]["gpu_num"] = a.gpus
        cfg["serve_configs"]["actual_gpu_num"] = a.gpus
        rows = fixed_trace(1024, 512, _n_requests(2048, a.skip_cycles + a.run_cycles, 1024, 512))
        out[name] = run_point(f"ablation-{a.model}-{name}", a.out, cfg, rows, gpus=a.gpus, run_cycles=a.run_cycles,
                              skip_cycles=a.skip_cycles, backend=a.backend, dry_run=a.dry_run)
    return out


def summarize(a) -> Dict:
    """Collect every ``*.stat.csv`` under --out into results.json with speed-ups against the
    published numbers where the workload matches."""
    res: Dict[str, Dict] = {}
    for fn in sorted(os.listdir(a.out)):
        if fn.endswith(".stat.csv"):
            name = fn[:-len(".stat.csv")]
            st = read_stat(os.path.join(a.out, fn))
            res[name] = st
            for wl, row in OFFLINE_FIXED.items():
                if name.endswith(wl) and name.startswith("fixed-llama2-70B"):
                    st["speedup_vs_published"] = speedup_table(st["token_per_second_per_gpu"], wl)
                    st["fraction_of_a100_optimal"] = st["token_per_second_per_gpu"] / OPTIMAL_LLAMA2_70B_A100
    with open(os.path.join(a.out, "results.json"), "w") as f:
        json.dump(res, f, indent=1)
    return res


ABLATION_LABELS = {"non-overlap": "Non-overlap", "nanobatch-only": "Nanobatch-only", "2048": "Nanoflow",
                   "pllm-offload": "Nanoflow-offload"}


def merge(a) -> Dict:
    """Write ``pllm.json`` in the layout of the reference's merged results
    (pipeline/eval/merge_results.py:10-62 plus the ``ablation`` block pipeline/eval/plot_all.py:52-53
    reads): tokens/s/GPU per fixed and per real-length workload, request rate -> normalised latency per
    online sweep, tokens/s/GPU per ablation variant. Points that were not run are left out."""
    res = {"offline_throughput_const": {}, "offline_throughput_real_trace": {}, "online_throughput": {}, "ablation": {}}
    for fn in sorted(os.listdir(a.out)):
        if not fn.endswith(".stat.csv"):
            continue
        name = fn[:-len(".stat.csv")]
        st = read_stat(os.path.join(a.out, fn))
        kind, _, rest = name.partition("-")
        if not rest.startswith(a.model + "-"):
            continue
        tail = rest[len(a.model) + 1:]
        if kind == "fixed":
            res["offline_throughput_const"][tail] = st["token_per_second_per_gpu"]
        elif kind == "real":
            res["offline_throughput_real_trace"][tail] = st["token_per_second_per_gpu"]
        elif kind == "ablation":
            res["ablation"][ABLATION_LABELS.get(tail, tail)] = {"1024-512": st["token_per_second_per_gpu"]}
        elif kind == "online":
            batch, _, rate = tail.rpartition("-r")
            sweep = res["online_throughput"].setdefault(batch, {"request_rate": [], "normalized_latency": []})
            sweep["request_rate"].append(float(rate))
            sweep["normalized_latency"].append(st["average_normalize_latency"])
    for sweep in res["online_throughput"].values():
        order = sorted(range(len(sweep["request_rate"])), key=lambda i: sweep["request_rate"][i])
        sweep["request_rate"] = [sweep["request_rate"][i] for i in order]
        sweep["normalized_latency"] = [sweep["normalized_latency"][i] for i in order]
    with open(os.path.join(a.out, "pllm.json"), "w") as f:
        json.dump(res, f, indent=1)
    return res


def plot(a) -> Dict:
    """Figures from ``pllm.json`` (run ``merge`` first): offline throughput per workload beside the
    published numbers of the other systems, normalised latency over request rate, the ablation bars.
    PNG files with matplotlib; without it the same series as one text file of bar charts. The
    reference draws these with pipeline/eval/plot_all.py:62-326."""
    from .baseline_data import OFFLINE_REAL
    with open(os.path.join(a.out, "pllm.json")) as f:
        data = json.load(f)
    series = []          # (title, unit, [(label, value)])
    for title, block, published in (("Offline throughput, constant lengths", "offline_throughput_const", OFFLINE_FIXED),
                                    ("Offline throughput, real length distributions", "offline_throughput_real_trace",
                                     OFFLINE_REAL)):
        for wl, ours in data.get(block, {}).items():
            bars = [(f"{k} (published, A100)", float(v)) for k, v in published.get(wl, {}).items()]
            series.append((f"{title}: {wl}", "tokens/s/GPU", bars + [("this engine", float(ours))]))
    for batch, sweep in data.get("online_throughput", {}).items():
        series.append((f"Online, {batch}: normalised latency by request rate", "s/token",
                       [(f"{r:g} req/s", float(v)) for r, v in zip(sweep["request_rate"], sweep["normalized_latency"])]))
    if data.get("ablation"):
        series.append(("Ablation, 1024-512", "tokens/s/GPU",
                       [(k, float(v["1024-512"])) for k, v in data["ablation"].items()]))
    written = []
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        plt = None
    if plt is not None:
        for n, (title, unit, bars) in enumerate(series):
            fig, ax = plt.subplots(figsize=(8, 4))
            ax.bar([b[0] for b in bars], [b[1] for b in bars])
            ax.set_title(title)
            ax.set_ylabel(unit)
            ax.tick_params(axis="x", rotation=30)
            fig.tight_layout()
            path = os.path.join(a.out, f"figure_{n}.png")
            fig.savefig(path)
            plt.close(fig)
            written.append(path)
    else:
        path = os.path.join(a.out, "figures.txt")
        with open(path, "w") as f:
            for title, unit, bars in series:
                f.write(f"{title} [{unit}]\n")
                top = max([v for _, v in bars] + [1e-30])
                width = max(len(b[0]) for b in bars) if bars else 0
                for label, v in bars:
                    f.write(f"  {label:<{width}} {'#' * max(1, int(round(50 * v / top)))} {v:.6g}\n")
                f.write("\n")
        written.append(path)
    return {"figures": written, "series": len(series)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("family", choices=["fixed-offline", "real-offline", "online", "ablation", "summarize", "merge", "plot"])
    ap.add_argument("--model", default="llama2-70B")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--batch", type=int, default=2048)
    ap.add_argument("--out", required=True)
    ap.add_argument("--run_cycles", type=int, default=1500)
    ap.add_argument("--skip_cycles", type=int, default=2000)
    ap.add_argument("--workloads", nargs="*", default=[])
    ap.add_argument("--traces", default="")
    ap.add_argument("--rates", nargs="*", type=float, default=[5, 10, 20, 30, 40, 50, 60])
    ap.add_argument("--requests", type=int, default=2000)
    ap.add_argument("--offload", action="store_true")
    ap.add_argument("--backend", default="gpu")
    ap.add_argument("--dry_run", action="store_true")
    a = ap.parse_args(argv)
    fn = {"fixed-offline": fixed_offline, "real-offline": real_offline, "online": online, "ablation": ablation,
          "summarize": summarize, "merge": merge, "plot": plot}[a.family]
    print(json.dumps(fn(a), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
