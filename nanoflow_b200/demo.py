"""Two one-line entry points over the other command-line tools.

    python -m nanoflow_b200.demo serve [--model llama3-8B] [--prompt "The University of Washington is located"]
        [--decode-length 100] [--requests 64] [--gpus 1] [--backend gpu] [--out demo/]
    python -m nanoflow_b200.demo perf --model llama2-70B --gpus 8 --out results/ [--dry_run]

``serve`` writes a trace of identical prompts, serves it with the model's shipped configuration for up to
200 cycles and prints what the first request generated. With a tokenizer (a local ``hf_path`` in the
configuration) the prompt text is tokenised and the output detokenised; without one the prompt
becomes as many synthetic token ids as it has words and the output is printed as ids. ``perf``
generates the traces and runs every experiment family of the evaluation harness, then summarises,
merges and plots. They stand for the reference's ``serve.sh`` (interactive prompt and model choice ->
``gen_req.py`` -> ``serve_8B.py -r 200``, serve.sh:14-59) and ``perf.sh`` (datasets/gen.sh +
pipeline/eval/run_all.sh).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List

MODELS = ["llama2-70B", "llama3-70B", "llama3.1-70B", "llama3-8B", "llama3.1-8B", "qwen2-72B", "tiny"]


def _serve(a) -> int:
    from . import serve
    from .config import MODEL_ARCHS, make_config, shipped_variants
    from .datasets.traces import write_trace
    from .utils.schedule_tools import gen_req

    os.makedirs(a.out, exist_ok=True)
    if a.model not in MODEL_ARCHS:
        raise SystemExit(f"unknown model {a.model}; choose from {', '.join(m for m in MODELS if m in MODEL_ARCHS)}")
    if a.model == "tiny":
        cfg = make_config("tiny", gpu_num=a.gpus, global_batch_size=48)
    else:
        variants = shipped_variants(a.model)
        cfg = variants["1024" if "1024" in variants and MODEL_ARCHS[a.model]["hidden_size"] <= 4096 else "2048"]
        cfg["model_configs"]["gpu_num"] = a.gpus
        cfg["serve_configs"]["actual_gpu_num"] = a.gpus
    if a.hf_path:
        cfg["serve_configs"]["hf_path"] = a.hf_path
    cfg_path = os.path.join(a.out, "config.json")
    with open(cfg_path, "w") as f:
        json.dump(cfg, f, indent=1)
    trace = os.path.join(a.out, "trace.csv")
    have_tok = bool(cfg["serve_configs"].get("hf_path")) and os.path.isdir(cfg["serve_configs"]["hf_path"])
    if have_tok:
        gen_req(a.prompt, a.decode_length, 0, trace, n=a.requests)          # input_len -1: tokenise the text
    else:
        n_in = max(1, len(a.prompt.split()))
        write_trace(trace, [(n_in, a.decode_length, 0.0)] * a.requests)
    prefix = os.path.join(a.out, "demo")
    args = ["-t", trace, "-c", cfg_path, "-r", "200", "--backend", a.backend, "-o", prefix, "--random_ids", "false"]
    if a.backend == "cpu":
        args += ["--allocate_page_num", "256"]
    if a.gpus > 1 and a.backend == "gpu" and "RANK" not in os.environ:
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29570", "-m", "nanoflow_b200.serve", *args]
        rc = subprocess.run(cmd).returncode
    else:
        rc = serve.main(args)
    if rc == 0:
        words = prefix + ".req_words"
        shown = words if os.path.exists(words) else prefix + ".req_tokens"
        with open(shown) as f:
            first = f.readline().strip()
        print(f"prompt: {a.prompt}\nfirst request ({os.path.basename(shown)}): {first}")
    return rc


def _perf(a) -> int:
    from .datasets import gen
    from .eval import harness

    traces = os.path.join(a.out, "traces")
    if not a.dry_run:
        gen.main(["--out", traces, "--n", str(a.requests)])
    common = ["--model", a.model, "--gpus", str(a.gpus), "--out", a.out, "--backend", a.backend,
              "--run_cycles", str(a.run_cycles), "--skip_cycles", str(a.skip_cycles)]
    if a.batch:
        common += ["--batch", str(a.batch)]
    if a.dry_run:
        common.append("--dry_run")
    steps: List[List[str]] = [["fixed-offline", *common], ["real-offline", *common],
                              ["online", "--requests", str(a.requests), *common]]
    if a.gpus > 1:
        steps.append(["ablation", *common])
    for step in steps:
        rc = harness.main(step)
        if rc != 0:
            return rc
    if not a.dry_run:
        for step in (["summarize", "--out", a.out], ["merge", "--model", a.model, "--out", a.out], ["plot", "--out", a.out]):
            harness.main(step)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    s.add_argument("--model", default="llama3-8B", help=", ".join(MODELS))
    s.add_argument("--prompt", default="The University of Washington is located")
    s.add_argument("--decode-length", type=int, default=100)
    s.add_argument("--requests", type=int, default=64)
    s.add_argument("--gpus", type=int, default=1)
    s.add_argument("--backend", default="gpu", choices=["gpu", "cpu"])
    s.add_argument("--hf-path", default="", help="local Hugging Face snapshot (tokenizer, weights)")
    s.add_argument("--out", default="demo")
    p = sub.add_parser("perf")
    p.add_argument("--model", default="llama2-70B")
    p.add_argument("--gpus", type=int, default=8)
    p.add_argument("--batch", type=int, default=0)
    p.add_argument("--backend", default="gpu", choices=["gpu", "cpu"])
    p.add_argument("--out", required=True)
    p.add_argument("--requests", type=int, default=2000)
    p.add_argument("--run_cycles", type=int, default=1500)
    p.add_argument("--skip_cycles", type=int, default=2000)
    p.add_argument("--dry_run", action="store_true")
    a = ap.parse_args(argv)
    return _serve(a) if a.cmd == "serve" else _perf(a)


if __name__ == "__main__":
    sys.exit(main())
