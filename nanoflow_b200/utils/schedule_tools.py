"""Small command-line helpers around traces and scheduler logs.

    python -m nanoflow_b200.utils.schedule_tools gen-req "<prompt>" <decode_len> <rate> <out.csv> [--n N]
    python -m nanoflow_b200.utils.schedule_tools to-csv <cycle_log.txt> <out.csv>
    python -m nanoflow_b200.utils.schedule_tools plot <schedule.csv> [--out prefix]
    python -m nanoflow_b200.utils.schedule_tools trend <prefill_decode.csv>

``gen-req``  demo trace of identical prompts: ``idx,-1,decode_len,arrival, prompt`` per line (the text
             prompt is tokenised by the frontend), arrivals ``idx / rate`` apart (rate 0 = all at once).
             Reference: pipeline/utils/gen_req.py:1-19.
``to-csv``   turns a cycle log of ``------------------ Cycle N ------------------`` blocks with
             ``key: value`` lines (regular and skip cycles) into one CSV row per cycle. The serving loop
             of this package writes its ``.schedule`` file as CSV already; this reads the reference's
             text form. Reference: pipeline/utils/listToCSV.py:5-40.
``plot``     memory usage and decode / prefill batch size per cycle. With matplotlib the same four PNG
             files as the reference (pipeline/utils/plotSchedule.py:5-42); without it, a text summary
             (min / mean / max and a coarse character plot) per series.
``trend``    prefill and prefill+decode tokens per cycle from a two-column CSV
             (pipeline/utils/plot_trend.py:1-18), PNG or text as above.
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from typing import Dict, List, Optional, Sequence

CYCLE_RE = re.compile(r"-{6,} (Skip Cycle|Cycle) (\d+) -{6,}")

# column names of this package's .schedule CSV and of the reference's converted cycle log
SERIES = {
    "memory": ("page_usage", "memory usage %"),
    "decode": ("decode_tokens", "decode effective bsz"),
    "prefill": ("prefill_tokens", "prefill effective bsz"),
}
CYCLE_COLS = ("iteration", "Cycle")


def gen_req(prompt: str, decode_len: int, rate: float, path: str, n: int = 100000) -> int:
    interval = 0.0 if rate == 0 else 1.0 / rate
    with open(path, "w") as f:
        for i in range(n):
            f.write(f"{i},-1,{decode_len},{interval * i}, {prompt}\n")
    return n


def parse_cycle_log(text: str) -> List[Dict[str, str]]:
    rows: List[Dict[str, str]] = []
    marks = list(CYCLE_RE.finditer(text))
    for k, m in enumerate(marks):
        body = text[m.end():marks[k + 1].start() if k + 1 < len(marks) else len(text)]
        row: Dict[str, str] = {"Cycle": m.group(2), "is_skip_cycle": str(m.group(1) != "Cycle")}
        for line in body.strip().splitlines():
            if ":" in line:
                key, value = line.split(":", 1)
                row[key.strip()] = value.strip()
        rows.append(row)
    return rows


def cycle_log_to_csv(src: str, dst: str) -> int:
    with open(src) as f:
        rows = parse_cycle_log(f.read())
    fields = sorted({k for r in rows for k in r})
    with open(dst, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=fields)
        w.writeheader()
        w.writerows(rows)
    return len(rows)


def _read_columns(path: str) -> Dict[str, List[float]]:
    with open(path, newline="") as f:
        rd = csv.DictReader(f)
        cols: Dict[str, List[float]] = {k: [] for k in (rd.fieldnames or [])}
        for row in rd:
            for k, v in row.items():
                try:
                    cols[k].append(float(v))
                except (TypeError, ValueError):
                    cols[k].append(float("nan"))
    return cols


def _pick(cols: Dict[str, List[float]], names: Sequence[str]) -> Optional[List[float]]:
    for n in names:
        if n in cols:
            return cols[n]
    return None


def text_plot(values: Sequence[float], width: int = 64, height: int = 8) -> str:
    vals = [v for v in values if v == v]
    if not vals:
        return "(no data)"
    lo, hi = min(vals), max(vals)
    step = max(1, len(vals) // width)
    pts = [sum(vals[i:i + step]) / len(vals[i:i + step]) for i in range(0, len(vals), step)][:width]
    span = (hi - lo) or 1.0
    grid = [[" "] * len(pts) for _ in range(height)]
    for x, v in enumerate(pts):
        grid[height - 1 - min(height - 1, int((v - lo) / span * (height - 1) + 0.5))][x] = "*"
    lines = ["".join(r) for r in grid]
    return "\n".join(lines) + f"\nmin {lo:g}  mean {sum(vals) / len(vals):g}  max {hi:g}  n {len(vals)}"


def plot_schedule(path: str, out_prefix: Optional[str] = None) -> List[str]:
    """Returns the files written (PNG with matplotlib, else one ``.txt``)."""
    cols = _read_columns(path)
    x = _pick(cols, CYCLE_COLS) or list(range(len(next(iter(cols.values()), []))))
    series = {k: _pick(cols, names) for k, names in SERIES.items()}
    prefix = out_prefix or path
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        out = prefix + ".schedule_summary.txt"
        with open(out, "w") as f:
            for k, v in series.items():
                if v is not None:
                    f.write(f"== {k} per cycle ==\n{text_plot(v)}\n\n")
        return [out]
    files = []
    titles = {"memory": ("Memory Usage % Across Cycles", "memory_usage"),
              "decode": ("Decode Effective Batch Size Across Cycles", "decode_effective_bsz"),
              "prefill": ("Prefill Effective Batch Size Across Cycles", "prefill_effective_bsz")}
    for k, (title, suffix) in titles.items():
        if series[k] is None:
            continue
        plt.figure()
        plt.plot(x, series[k], marker="o", markersize=1, linestyle="-")
        plt.title(title)
        plt.xlabel("Cycle")
        plt.grid(True)
        files.append(f"{prefix}.{suffix}.png")
        plt.savefig(files[-1])
        plt.close()
    if series["decode"] is not None and series["prefill"] is not None:
        plt.figure()
        plt.plot(x, series["decode"], label="Decode Effective Batch Size")
        plt.plot(x, series["prefill"], label="Prefill Effective Batch Size")
        plt.legend()
        plt.grid(True)
        files.append(f"{prefix}.effective_bsz.png")
        plt.savefig(files[-1])
        plt.close()
    return files


def plot_trend(path: str) -> str:
    prefill, total = [], []
    with open(path, newline="") as f:
        for row in csv.reader(f):
            if len(row) >= 2:
                try:
                    p, d = float(row[0]), float(row[1])
                except ValueError:
                    continue
                prefill.append(p)
                total.append(p + d)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        out = path + ".trend.txt"
        with open(out, "w") as f:
            f.write(f"== prefill ==\n{text_plot(prefill)}\n\n== prefill + decode ==\n{text_plot(total)}\n")
        return out
    plt.figure()
    plt.plot(prefill, label="prefill")
    plt.plot(total, label="sum")
    plt.ylim(0, max(2100.0, max(total, default=0.0) * 1.05))
    plt.legend()
    plt.savefig(path + ".png")
    plt.close()
    return path + ".png"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gen-req")
    g.add_argument("prompt")
    g.add_argument("decode_len", type=int)
    g.add_argument("rate", type=float)
    g.add_argument("out")
    g.add_argument("--n", type=int, default=100000)
    c = sub.add_parser("to-csv")
    c.add_argument("src")
    c.add_argument("dst")
    p = sub.add_parser("plot")
    p.add_argument("schedule_csv")
    p.add_argument("--out", default=None)
    t = sub.add_parser("trend")
    t.add_argument("csv")
    a = ap.parse_args(argv)
    if a.cmd == "gen-req":
        print(gen_req(a.prompt, a.decode_len, a.rate, a.out, a.n), "requests ->", a.out)
    elif a.cmd == "to-csv":
        print(cycle_log_to_csv(a.src, a.dst), "cycles ->", a.dst)
    elif a.cmd == "plot":
        print("\n".join(plot_schedule(a.schedule_csv, a.out)))
    else:
        print(plot_trend(a.csv))
    return 0


if __name__ == "__main__":
    sys.exit(main())
