"""Result files of a serving run, in the reference's formats (pipeline/utils/serve_8B.py:755-797):

``<prefix>.stat``       human-readable summary
``<prefix>.stat.csv``   one row: total_time, token_per_second, token_per_second_per_gpu, total_cycle,
                        cycle_time, average_ttft, average_tpot, average_normalize_latency
``<prefix>.req_time``   per request: req_idx, input_len, output_len, req_comein_time, encode_latency,
                        decode_start_at, decode_latency
``<prefix>.req_tokens`` per request: generated token ids (``.req_words`` when a detokenizer is given)
``<prefix>.schedule``   per cycle: decode / prefill tokens, idle tokens, page usage, queue length

Throughput is counted as the reference counts it: retired requests x (average prompt + average
output length) over host wall-clock seconds, and per GPU by dividing by ``gpu_num``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

from .request import FlyRequestInfo

CSV_COLUMNS = ("total_time,token_per_second,token_per_second_per_gpu,total_cycle,cycle_time,"
               "average_ttft,average_tpot,average_normalize_latency")


@dataclass
class RunSummary:
    total_time: float
    token_per_second: float
    token_per_second_per_gpu: float
    total_cycle: int
    cycle_time: float
    average_ttft: float
    average_tpot: float
    average_normalize_latency: float
    retired: int

    def csv_row(self) -> str:
        return (f"{self.total_time},{self.token_per_second},{self.token_per_second_per_gpu},{self.total_cycle},"
                f"{self.cycle_time},{self.average_ttft},{self.average_tpot},{self.average_normalize_latency}")


def request_latencies(req: FlyRequestInfo) -> Dict[str, float]:
    """encode_latency = arrival -> first token; decode_latency = first -> last token."""
    first = req.first_token_time or req.finish_time
    enc = max(0.0, first - req.request_comein_time)
    dec = max(0.0, (req.finish_time or first) - first)
    return {"encode_latency": enc, "decode_start_at": first, "decode_latency": dec}


def summarize(retired: Sequence[FlyRequestInfo], wall_seconds: float, cycles: int, gpu_num: int,
              average_prefill_length: float, average_decode_length: float) -> RunSummary:
    n = len(retired)
    tps = n * (average_prefill_length + average_decode_length) / wall_seconds if wall_seconds > 0 else 0.0
    ttft = tpot = norm = 0.0
    for r in retired:
        lat = request_latencies(r)
        out_len = max(1, len(r.output))
        ttft += lat["encode_latency"]
        tpot += lat["decode_latency"] / max(1, out_len - 1)
        norm += (lat["decode_start_at"] + lat["decode_latency"] - r.request_comein_time) / out_len
    d = max(1, n)
    return RunSummary(total_time=wall_seconds, token_per_second=tps, token_per_second_per_gpu=tps / max(1, gpu_num),
                      total_cycle=cycles, cycle_time=wall_seconds / max(1, cycles), average_ttft=ttft / d,
                      average_tpot=tpot / d, average_normalize_latency=norm / d, retired=n)


def write_outputs(prefix: str, summary: RunSummary, retired: Sequence[FlyRequestInfo],
                  schedule_log: Optional[List[dict]] = None,
                  detokenize: Optional[Callable[[List[int]], str]] = None, output_idx: bool = False) -> List[str]:
    """``output_idx``: ``.req_words`` gets a ``Req <n>:`` line before every request, as the reference's
    flag of that name does (pipeline/utils/serve_8B.py:723-725). ``.req_tokens.uniq`` counts identical
    output sequences (the reference's ``sort | uniq -c``, serve_8B.py:731): identical prompts must give
    identical greedy outputs."""
    files = []
    with open(prefix + ".stat", "w") as f:
        f.write(f"TOTAL Time taken: {summary.total_time}\n")
        f.write(f"Token per second: {summary.token_per_second}\n")
        f.write(f"per GPU: {summary.token_per_second_per_gpu}\n")
        f.write(f"Total Cycle: {summary.total_cycle}\n")
        f.write(f"Cycle time taken: {summary.cycle_time}\n")
        f.write(f"Actual Retired request size: {summary.retired}\n")
        f.write(f"Average TTFT: {summary.average_ttft}\n")
        f.write(f"Average TPOT: {summary.average_tpot}\n")
        f.write(f"Average Normalize Latency: {summary.average_normalize_latency}\n")
    files.append(prefix + ".stat")
    with open(prefix + ".stat.csv", "w") as f:
        f.write(CSV_COLUMNS + "\n" + summary.csv_row() + "\n")
    files.append(prefix + ".stat.csv")
    with open(prefix + ".req_time", "w") as f:
        f.write("req_idx,input_len,output_len,req_comein_time,encode_latency,decode_start_at,decode_latency\n")
        for r in retired:
            lat = request_latencies(r)
            f.write(f"{r.req_idx},{r.input_len},{len(r.output)},{r.request_comein_time},{lat['encode_latency']},"
                    f"{lat['decode_start_at']},{lat['decode_latency']}\n")
    files.append(prefix + ".req_time")
    with open(prefix + ".req_tokens", "w") as f:
        for r in sorted(retired, key=lambda r: r.req_idx):
            f.write(f"{r.req_idx}: {' '.join(str(t) for t in r.output)}\n")
    files.append(prefix + ".req_tokens")
    counts: dict = {}
    for r in retired:
        key = " ".join(str(t) for t in list(r.prompt.tolist()) + list(r.output))
        counts[key] = counts.get(key, 0) + 1
    with open(prefix + ".req_tokens.uniq", "w") as f:
        for key in sorted(counts):
            f.write(f"{counts[key]:7d} {key}\n")
    files.append(prefix + ".req_tokens.uniq")
    if detokenize is not None:
        with open(prefix + ".req_words", "w") as f:
            for n, r in enumerate(sorted(retired, key=lambda r: r.req_idx)):
                if output_idx:
                    f.write(f"Req {n}:\n")
                f.write(f"{r.req_idx}: {detokenize(r.output)}\n")
        files.append(prefix + ".req_words")
    if schedule_log:
        with open(prefix + ".schedule", "w") as f:
            cols = ["iteration", "decode_tokens", "prefill_tokens", "batch_size", "idle_tokens", "page_usage",
                    "queue", "retired"]
            f.write(",".join(cols) + "\n")
            for row in schedule_log:
                f.write(",".join(str(row.get(c, "")) for c in cols) + "\n")
        files.append(prefix + ".schedule")
    return files
