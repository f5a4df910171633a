"""Serving / offline-throughput entry point.

    python -m nanoflow_b200.serve -t trace.csv -c nanoflow_b200/configs/llama3-8B/2048.json -r 200 \
        --empty_weight True -o out/run1

Flags follow the reference's ``serve_8B.py`` (pipeline/utils/serve_8B.py:584-596): ``-t`` trace CSV,
``-c`` config JSON, ``-r`` run cycles, ``-s`` skip cycles (scheduler-only warm-up to the steady batch
mix), ``--est_cycle_time`` (simulated seconds per cycle while skipping / in simulated-time mode),
``--empty_weight`` (random-init weights instead of converted checkpoints), ``-o`` output prefix,
``--allocate_page_num`` (KV pages per GPU; 0 = size from free memory). For tensor parallel runs launch
one process per GPU with ``python -m torch.distributed.run --nproc-per-node N -m nanoflow_b200.serve ...``.
Outputs: ``<prefix>.stat / .stat.csv / .req_time / .req_tokens / .req_tokens.uniq / .schedule`` (see
serving/stats.py), ``.req_words`` with a tokenizer, ``.trace.json.gz`` with ``--profile_mode``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def _bool(s: str) -> bool:
    return str(s).lower() in ("1", "true", "yes", "y")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-t", "--trace_path", type=str, required=True, help="request trace CSV")
    ap.add_argument("-r", "--run_cycles", type=int, default=20)
    ap.add_argument("-c", "--config_path", type=str, required=True, help="four-section config JSON")
    ap.add_argument("-s", "--skip_cycles", type=int, default=0)
    ap.add_argument("--est_cycle_time", type=float, default=0.175)
    ap.add_argument("-o", "--output_prefix", type=str, default="")
    ap.add_argument("--allocate_page_num", type=int, default=0)
    ap.add_argument("--empty_weight", type=_bool, default=False)
    ap.add_argument("--output_idx", type=_bool, default=False, help="number the requests in <prefix>.req_words")
    ap.add_argument("--profile_mode", type=_bool, default=False,
                    help="run 10 cycles under torch.profiler and write <prefix>.trace.json.gz (Chrome trace)")
    ap.add_argument("--online", type=_bool, default=False, help="release requests by wall clock (arrival times)")
    ap.add_argument("--random_ids", type=_bool, default=True, help="synthetic prompts use uniform-random token ids")
    ap.add_argument("--stop_on_eos", type=_bool, default=False)
    ap.add_argument("--backend", choices=["gpu", "cpu"], default="gpu")
    ap.add_argument("--until_empty", type=_bool, default=False, help="ignore -r and run until the trace is served")
    ap.add_argument("--heartbeat", type=_bool, default=False,
                    help="tensor parallel runs: check before every launch that all ranks are alive")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from .config import load_config
    from .models import random_full_weights, random_rank_weights, shard_weights
    from .models.weights import ensure_converted, load_rank_weights, load_weights
    from .serving import DistKVPool, RequestManager, Scheduler
    from .serving.loop import ServingLoop
    from .serving.stats import summarize, write_outputs

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = load_config(args.config_path, tp=world if world > 1 else None)
    model, eng_cfg = cfg.model, cfg.engine
    if world > 1 and world != model.tp:
        raise SystemExit(f"config is for tp={model.tp} but WORLD_SIZE={world}")

    # A tokenizer is used only when the config names a local directory that holds one (hf_path): trace
    # rows with input_len == -1 are tokenised with it and <prefix>.req_words is written with it.
    detok, tok_dir = None, None
    if eng_cfg.hf_path and os.path.isdir(eng_cfg.hf_path):
        try:
            from transformers import AutoTokenizer

            tk = AutoTokenizer.from_pretrained(eng_cfg.hf_path)
            detok, tok_dir = (lambda ids: tk.decode(list(ids), skip_special_tokens=True)), eng_cfg.hf_path
        except (OSError, ValueError, KeyError, ImportError) as e:   # no tokenizer files there: go on without
            print(f"no tokenizer under {eng_cfg.hf_path}: {e}", file=sys.stderr)
    rm = RequestManager(args.trace_path, vocab_size=model.vocab_size, random_ids=args.random_ids)
    rm.read_request(tok_dir)

    coll = None
    if args.backend == "gpu":
        from .runtime.engine import Engine

        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            import torch.distributed as dist
            from .parallel.collectives import TpCollectives

            dist.init_process_group("nccl", device_id=dev)
            coll = TpCollectives(rank, world, dev)
        have_files = False
        if not args.empty_weight and eng_cfg.weight_path:
            # converted per-rank files; written first from the Hugging Face snapshot if they are missing
            if rank == 0:
                have_files = ensure_converted(eng_cfg.weight_path, eng_cfg.hf_path, max(1, world))
            if world > 1:
                torch.distributed.barrier()
            have_files = ensure_converted(eng_cfg.weight_path, "", max(1, world))
        if not have_files:
            weights = random_rank_weights(model, rank, max(1, world), dev, o1=bool(eng_cfg.o_allgather_nanos))
        else:
            weights = load_rank_weights(eng_cfg.weight_path, model, rank, max(1, world), device=dev,
                                        o1=bool(eng_cfg.o_allgather_nanos))
        engine = Engine(cfg, weights, device=dev, collectives=coll, num_pages=args.allocate_page_num or None)
        num_pages = engine.num_pages
    else:
        from .runtime.cpu_backend import CpuEngine

        tp = model.tp
        num_pages = args.allocate_page_num or 4096
        if not args.empty_weight and eng_cfg.weight_path and ensure_converted(eng_cfg.weight_path, eng_cfg.hf_path, tp,
                                                                                dtype=torch.float32):
            shards = load_weights(tp, eng_cfg.weight_path, model, dtype=torch.float32)
        else:
            fw = random_full_weights(model, seed=0)
            shards = [shard_weights(fw, model, r, tp, dtype=torch.float32) for r in range(tp)]
        engine = CpuEngine(cfg, shards, num_pages=num_pages)

    pool = DistKVPool(model.run_layers, model.num_kv_heads, model.head_dim, num_pages, eng_cfg.page_size, model.tp)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=eng_cfg.global_batch_size,
                    nanobatch_sizes=eng_cfg.resolved_nanobatches(), max_batch_size=eng_cfg.max_batch_size,
                    average_prefill_length=rm.average_prefill_length, average_decode_length=rm.average_decode_length,
                    group_size=model.group_size, eos_token_id=model.eos_token_id, stop_on_eos=args.stop_on_eos,
                    hold_retired_pages=bool(eng_cfg.offload and args.backend == "gpu"),
                    decode_tail_fraction=eng_cfg.decode_tail_fraction)
    sch.keep_schedule_log = bool(args.output_prefix)
    offload = None
    if eng_cfg.offload and args.backend == "gpu":
        from .serving.offload import KVOffloadManager

        offload = KVOffloadManager(engine)
    health = None
    if args.heartbeat and world > 1:
        from torch.distributed.distributed_c10d import _get_default_store
        from .parallel.health import Heartbeat

        health = Heartbeat(_get_default_store(), rank, world)
    if args.online and world > 1:
        # all ranks release requests by rank 0's clock, so that the replicated schedulers stay identical
        from torch.distributed.distributed_c10d import _get_default_store
        from .serving.frontend import SharedReleaseClock

        rm.release_clock = SharedReleaseClock(_get_default_store(), rank, world)
    loop = ServingLoop(engine, sch, rm, simulated_time=not args.online, est_cycle_time=args.est_cycle_time,
                       offload=offload, health=health, trace_phases=args.profile_mode)
    log = None
    if args.output_prefix:
        # one log file per rank beside the outputs (the reference writes log_<rank>.txt, pipeline/src/pipeline.cu:15-19)
        from .utils.logging import rank_logger
        log = rank_logger(rank, os.path.dirname(os.path.abspath(args.output_prefix)) or ".")
        log.info("serving %s: %d GPUs, pipeline %s, dense batch %d, nano-batches %s, %d KV pages, trace %s",
                 eng_cfg.model_id or args.config_path, model.tp, eng_cfg.pipeline_type, eng_cfg.global_batch_size,
                 eng_cfg.resolved_nanobatches(), num_pages, args.trace_path)
    if args.skip_cycles:
        loop.skip_cycles(args.skip_cycles)
    rm.start_processing()
    t0 = time.perf_counter()
    if args.profile_mode:
        # the older serving loops of the reference export a Chrome trace of ten cycles this way
        # (pipeline/utils/scheduler.py:434-477)
        import gzip
        import tempfile
        from torch.profiler import ProfilerActivity, profile, record_function

        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if args.backend == "gpu" else [])
        with profile(activities=acts, record_shapes=True) as prof:
            with record_function("model_inference"):
                loop.run(max_cycles=10, until_empty=True)
        if rank == 0:
            out = (args.output_prefix or "serve") + ".trace.json.gz"
            os.makedirs(os.path.dirname(os.path.abspath(out)) or ".", exist_ok=True)
            with tempfile.TemporaryDirectory() as tmp:
                raw = os.path.join(tmp, "trace.json")
                prof.export_chrome_trace(raw)
                with open(raw, "rb") as fi, gzip.open(out, "wb") as fo:
                    fo.write(fi.read())
            print(f"profile written to {out}")
    else:
        loop.run(max_cycles=None if args.until_empty else args.run_cycles, until_empty=True)
    wall = time.perf_counter() - t0
    engine.check_status()
    st = loop.stats
    summary = summarize(st.retired, wall, st.cycles, model.tp, rm.average_prefill_length, rm.average_decode_length)
    if log is not None:
        log.info("done: %d cycles, %d requests retired, %.1f tokens/s, %.2f ms per cycle", st.cycles, summary.retired,
                 summary.token_per_second, summary.cycle_time * 1e3)
    if offload is not None:
        off_line = (f"KV offload: {offload.total_requests} requests, {offload.total_pages} pages, "
                    f"{offload.total_bytes / 1e6:.1f} MB per GPU to pinned host memory "
                    f"({offload.total_bytes / 1e6 / max(wall, 1e-9):.1f} MB/s per GPU), "
                    f"{offload.dropped_requests} requests beyond the per-iteration staging")
        if log is not None:
            log.info(off_line)
    if rank == 0:
        print(f"cycles {st.cycles}  retired {summary.retired}  tokens/s {summary.token_per_second:.1f} "
              f"(per GPU {summary.token_per_second_per_gpu:.1f})  cycle {summary.cycle_time * 1e3:.2f} ms")
        if offload is not None:
            print(off_line)
        if args.output_prefix:
            os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)) or ".", exist_ok=True)
            write_outputs(args.output_prefix, summary, st.retired, sch.schedule_log, output_idx=args.output_idx,
                          detokenize=detok)
    engine.finalize()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
