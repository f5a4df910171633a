#!/usr/bin/env python
"""Headline benchmark: Llama-2-70B offline serving throughput, 1024 input / 512 output tokens,
tensor parallel over N GPUs of one node (N = 1 runs the whole model on one B200).

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 3

A step is one serving iteration (one dense batch of prefill + decode tokens through all 80 layers,
sampling included). The scheduler is first advanced without GPU work to the steady-state batch mix
(the reference's ``--skip_cycles``, pipeline/utils/serve_8B.py:657-662), then W warm-up steps run,
then exactly K steps are timed twice:

* ``value``: CUDA events on the engine stream around the K steps (barrier + synchronize on both
  sides), max over ranks; tokens = dense-batch tokens executed in those steps, whole job.
* ``e2e``: the same K-step loop through the public serving API (``ServingLoop.step``) timed by host
  wall clock, including every step's scheduler work, the pinned-host -> device copy of the batch
  metadata / prompt token ids and the device -> host read of the sampled tokens.

Weights are random-init bf16 of the real architecture, prompts are uniform-random token ids
(synthetic; there is no network for checkpoints or datasets). The model (>= 17 GB of weights per
GPU) is far larger than L2, so no explicit L2 flush is needed between iterations.

``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REF_UNAVAILABLE = ("reference is not installable or buildable offline: its checkout has no setup.py/pyproject "
                   "(pip: 'Neither setup.py nor pyproject.toml found'); its CMake build needs the empty "
                   "3rdparty submodules (cutlass, flashinfer, mscclpp, spdlog) and targets sm_80 only")

BASELINE_TOK_S_PER_GPU = 1263.0   # NanoFlow, Llama-2-70B, 8xA100, in1024/out512 (published)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.rows:
            if t < t0 or t > t1 + 0.1:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama2-70B")
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--global-batch", type=int, default=0, help="dense tokens per iteration (0 = choose)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the result invalid)")
    ap.add_argument("--pipeline", default="", help="override pipeline_type")
    ap.add_argument("--nano", default="", help="comma-separated nano-batch sizes (must sum to the dense batch); "
                    "default: two halves for the overlapped pipelines")
    ap.add_argument("--comm-ctas", type=int, default=0)
    ap.add_argument("--mem-fraction", type=float, default=0.96, help="share of device memory the engine may use")
    ap.add_argument("--fuse-rs", action="store_true", help="K-split GEMMs push their partial rows to the owners "
                    "from the GEMM epilogue (fused GEMM -> reduce-scatter) instead of the collective pulling them")
    ap.add_argument("--fuse-rs-staged", action="store_true", help="with --fuse-rs: rows leave the epilogue through "
                    "shared memory and one 256-byte bulk copy per row and 128 columns")
    ap.add_argument("--no-fuse-norm", action="store_true", help="one GPU: separate RMSNorm launches after O / down")
    ap.add_argument("--serial-attention", action="store_true",
                    help="prefill attention after decode attention on one stream instead of beside it")
    ap.add_argument("--attn-overlap", action="store_true",
                    help="tensor-parallel overlapped pipelines: decode attention on its own stream under the GEMMs of "
                         "the other nano-batches (use with three or four nano-batches, e.g. --nano 2048,2048,2048,2048)")
    ap.add_argument("--gate-gemm", action="store_true",
                    help="tensor parallel: the GEMM behind an all-reduce + norm starts with the collective and waits per "
                         "128-row block for its input rows")
    ap.add_argument("--o-allgather", default="",
                    help="tensor parallel: comma-separated nano-batches whose O projection takes the all-gather form "
                         "(attention output gathered column-wise, N-split weight) instead of K-split weight + all-reduce")
    ap.add_argument("--cross-layer", action="store_true",
                    help="overlapped pipelines: software pipeline across layers (a nano-batch's attention of layer l+1 "
                         "under the other nano-batches' O / FFN GEMMs of layer l)")
    ap.add_argument("--prefill-impl", default="", choices=["", "ws", "tc", "mma"], help="prefill attention kernel")
    ap.add_argument("--decode-ctas", type=int, default=0, help="CTA budget of the decode attention kernel (0 = default)")
    ap.add_argument("--decode-impl", default="", choices=["", "tma"], help="decode attention kernel (tma: producer warp)")
    ap.add_argument("--gemm-smem-kb", type=int, default=0, help="with --attn-overlap: shared memory a GEMM CTA keeps")
    ap.add_argument("--decode-stages", type=int, default=0, choices=[0, 2, 3, 4],
                    help="decode attention pages in flight per warp (0: 3, or 2 with --attn-overlap)")
    ap.add_argument("--ar-wide", action="store_true", help="8 GPUs: all-reduce with twice the loads in flight per phase")
    ap.add_argument("--symm-backend", default="", choices=["", "auto", "ipc", "nvls"],
                    help="symmetric heap: nvls binds the ranks' heaps to an NVLink multicast object (all-reduce "
                         "through the switch), ipc is plain peer mappings; default auto (nvls when available)")
    ap.add_argument("--push-by-copy", action="store_true",
                    help="all-reduce + norm: the normed rows reach the peers by copy-engine copies instead of stores "
                         "from the kernel")
    ap.add_argument("--no-multimem", action="store_true", help="keep the peer-load all-reduce even on an nvls heap")
    ap.add_argument("--net-streams", type=int, default=1, choices=[1, 2],
                    help="2: the collectives of odd nano-batches run on a second network stream")
    ap.add_argument("--decode-tail", type=float, default=-1.0,
                    help="share of the decode requests' context scheduled into the last nano-batch (0 = all first; "
                         "default: 0.5 for the overlapped tensor-parallel pipeline, else 0)")
    ap.add_argument("--virtual-tp", type=int, default=0,
                    help="one GPU runs rank 0's share of a tensor-parallel job of this degree, collectives reduced "
                         "to their local part (development aid; the JSON line is marked invalid)")
    ap.add_argument("--fake-wire-us-per-row", type=float, default=0.0,
                    help="with --virtual-tp: every all-reduce is followed on its stream by a sleep of this many "
                         "microseconds per row of its nano-batch, standing in for the absent ranks")
    ap.add_argument("--skip-cycles", type=int, default=1600)
    ap.add_argument("--executor", default="auto", help="auto | native | graph (native executor, iterations "
                    "captured and launched as CUDA graphs) | python")
    ap.add_argument("--timeline", default="", help="after the timed regions, time every op of one iteration "
                    "with CUDA events and write the aggregate + Chrome trace to this file")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")

    import numpy as np
    import torch

    from nanoflow_b200.config import builtin_config
    from nanoflow_b200.models import random_rank_weights
    from nanoflow_b200.runtime.engine import Engine
    from nanoflow_b200.serving import DistKVPool, RequestManager, Scheduler
    from nanoflow_b200.serving.loop import ServingLoop

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    coll = None
    if world > 1:
        import torch.distributed as dist
        from nanoflow_b200.parallel.collectives import TpCollectives

        dist.init_process_group("nccl", device_id=dev)
        coll = TpCollectives(rank, world, dev, backend=args.symm_backend)
        coll.wide = bool(args.ar_wide)
        if args.no_multimem:
            coll.use_multimem = False
        coll.push_by_copy = bool(args.push_by_copy)

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    tp = world
    if args.virtual_tp > 1:
        if world != 1:
            raise SystemExit("--virtual-tp runs on one GPU")
        from nanoflow_b200.parallel.collectives import TpCollectives

        tp = args.virtual_tp
        coll = TpCollectives(0, 1, dev)
        coll.fake_wire_us_per_row = args.fake_wire_us_per_row
    # KV capacity decides how many requests fit, hence the steady-state dense batch: with 1024/512
    # requests a batch of T tokens holds T/3 decode requests of ~1280 tokens each.
    probe = builtin_config(args.model, gpu_num=tp, global_batch_size=2048)
    if args.layers:
        probe.model.num_layers = args.layers
        probe.model.run_layers = args.layers
    weight_bytes = probe.model.param_count() * 2 / tp + probe.model.vocab_size * probe.model.hidden_size * 2 * (1 - 1 / tp)
    total_mem = torch.cuda.get_device_properties(dev).total_memory
    kv_budget = total_mem * args.mem_fraction - weight_bytes - (4 << 30)
    tok_cap = kv_budget / probe.model.kv_bytes_per_token_local()
    avg_ctx = args.input_len + args.output_len / 2
    gbs = args.global_batch
    if gbs == 0:
        max_decode = tok_cap / (avg_ctx * 1.12)
        gbs = int(max_decode * (args.input_len + args.output_len) / args.output_len)
        gbs = max(256, min(8192, gbs // 64 * 64))
    # Measured on B200: with two ranks the all-reduces are short and splitting the batch costs more GEMM
    # efficiency than the overlap returns; from four ranks on the overlapped pipeline wins.
    ptype = args.pipeline or ("NON_OVERLAP_LOCAL" if tp == 1 else "NON_OVERLAP" if tp == 2 else "PLLM")
    if args.decode_tail < 0:
        # both nano-batches get decode requests, so that each attention front-end covers the other's all-reduce
        args.decode_tail = 0.5 if (tp > 2 and not ptype.startswith("NON")) else 0.0
    nano = None
    if args.nano:
        nano = [int(x) for x in args.nano.split(",")]
    elif not ptype.startswith("NON"):
        half = max(128, (gbs // 2) // 128 * 128)
        nano = [half, gbs - half]
    cfg = builtin_config(args.model, gpu_num=tp, global_batch_size=gbs, pipeline_type=ptype,
                         **({"nanobatch_sizes": nano} if nano else {}))
    if args.comm_ctas:
        cfg.engine.sm_budget["comm"] = args.comm_ctas
    cfg.engine.fuse_gemm_rs = bool(args.fuse_rs)
    cfg.engine.gemm_rs_staged = bool(args.fuse_rs_staged)
    cfg.engine.net_streams = args.net_streams
    cfg.engine.attn_overlap = bool(args.attn_overlap)
    cfg.engine.cross_layer_pipeline = bool(args.cross_layer)
    cfg.engine.gate_gemm = bool(args.gate_gemm)
    cfg.engine.o_allgather_nanos = [int(k) for k in args.o_allgather.split(",") if k != ""] if tp > 1 else []
    cfg.engine.prefill_impl = args.prefill_impl
    cfg.engine.decode_impl = args.decode_impl
    if args.gemm_smem_kb:
        from nanoflow_b200.runtime import pipeline as _pl
        _pl.GEMM_SMEM_KB_BESIDE_ATTENTION = args.gemm_smem_kb
    if args.decode_ctas:
        cfg.engine.sm_budget["attn_decode"] = args.decode_ctas
    cfg.engine.decode_stages = args.decode_stages
    cfg.engine.fuse_gemm_norm = not args.no_fuse_norm
    cfg.engine.prefill_beside_decode = not args.serial_attention
    if args.layers:
        cfg.model.num_layers = args.layers
        cfg.model.run_layers = args.layers
    cfg.engine.max_batch_size = gbs
    cfg.engine.gpu_mem_fraction = args.mem_fraction
    model = cfg.model

    t_load = time.perf_counter()
    weights = random_rank_weights(model, 0 if args.virtual_tp > 1 else rank, tp, dev, seed=0,
                                  o1=bool(cfg.engine.o_allgather_nanos))
    torch.cuda.synchronize()
    # One GPU: iterations go out as CUDA graphs (measured 45.5 against 47.1 ms per iteration); with
    # several ranks the launch gaps already hide under the other streams and plain launches are kept.
    executor = args.executor if args.executor != "auto" else ("graph" if world == 1 and args.virtual_tp <= 1 else "auto")
    eng = Engine(cfg, weights, device=dev, collectives=coll, executor=executor)
    load_s = time.perf_counter() - t_load

    # synthetic trace: constant-length requests, all available at t=0 (offline)
    n_req = int((args.skip_cycles + 4 * (args.warmup + args.steps) + 64) * gbs / (args.input_len + args.output_len)) + 512
    rm = RequestManager(vocab_size=model.vocab_size, random_ids=True, seed=0)
    for _ in range(n_req):
        rm.add_request(args.input_len, args.output_len, 0.0)
    rm.finalize_stats()
    pool = DistKVPool(model.run_layers, model.num_kv_heads, model.head_dim, eng.num_pages, cfg.engine.page_size, tp)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                    nanobatch_sizes=cfg.engine.resolved_nanobatches(), max_batch_size=gbs,
                    average_prefill_length=args.input_len, average_decode_length=args.output_len,
                    group_size=model.group_size, decode_tail_fraction=args.decode_tail)
    loop = ServingLoop(eng, sch, rm, simulated_time=True, est_cycle_time=1.0)
    loop.skip_cycles(args.skip_cycles)

    for _ in range(max(3, args.warmup)):
        loop.step()
    loop.drain()
    eng.check_status()

    # ---- timed region 1: device time (CUDA events), max over ranks --------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    launches0 = eng.native.launches if eng.native is not None else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    tw0 = time.perf_counter()
    e0.record(eng.stream)
    tok0 = loop.stats.tokens_processed
    for _ in range(args.steps):
        loop.step()
    loop.drain()
    e1.record(eng.stream)
    barrier()
    torch.cuda.synchronize()
    tw1 = time.perf_counter()
    dev_ms = e0.elapsed_time(e1)
    tokens_dev = loop.stats.tokens_processed - tok0
    launches = (eng.native.launches - launches0) if eng.native is not None else args.steps * eng.launches_per_iteration
    n_memcpy = sum(1 for op in eng.graph.ops if op.kernel == "nfk_memcpy_p")
    launches -= args.steps * n_memcpy

    # ---- timed region 2: end to end through the public API, host wall clock ------------------------
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tok1 = loop.stats.tokens_processed
    h2d = d2h = 0
    for _ in range(args.steps):
        loop.step()
        h2d += eng.h2d_bytes_last
        d2h += eng.d2h_bytes_last
    loop.drain()
    barrier()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    tokens_e2e = loop.stats.tokens_processed - tok1
    clocks = sampler.stop(tw0, time.perf_counter())
    eng.check_status()

    if args.timeline:
        from nanoflow_b200.utils import timeline as tl
        loop._release()
        plan = sch.schedule()
        eng.update(plan)
        eng.run_async(timed=True)
        toks = eng.run_async_wait()
        sch.process_outputs(plan, toks)
        ev = eng.timeline()
        per_rank = [ev]
        if world > 1:
            # every rank's timeline goes into the file: a collective's duration on a rank that reaches it
            # early contains the wait for the last rank, which only the comparison across ranks shows
            per_rank = [None] * world
            torch.distributed.all_gather_object(per_rank, [tuple(e) for e in ev])
        if rank == 0:
            if world > 1:
                print("timeline ranks:", json.dumps(tl.dump_ranks(per_rank, args.timeline)), file=sys.stderr)
            else:
                tl.dump(ev, args.timeline, pid=rank)
            agg = tl.aggregate(ev)
            print("timeline:", json.dumps({k: v for k, v in list(agg.items())[:14]}), file=sys.stderr)

    if world > 1:
        t = torch.tensor([dev_ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    else:
        e2e_ms = e2e_s * 1e3

    value = tokens_dev / (dev_ms / 1e3)
    e2e_value = tokens_e2e / (e2e_ms / 1e3)
    if rank == 0:
        out = {
            "metric": "Llama2-70B offline tokens/s (in1024/out512), whole job",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(dev_ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak",
            "scaling_note": "the dense batch per step grows with N (it is sized by the KV capacity left beside the "
                            "weights: 256 tokens on one GPU, 8192 on eight), so per-GPU work is not constant either; "
                            "compare tokens_per_s_per_gpu from N=2 on",
            "vs_baseline": round(value / world / BASELINE_TOK_S_PER_GPU, 3),
            "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)",
            "tokens_per_s_per_gpu": round(value / world, 1),
            "config": {"model": args.model, "global_batch": gbs, "seq_len": args.input_len + args.output_len,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "parallelism": f"tp{world}", "pipeline_type": ptype, "layers": model.run_layers,
                       "nanobatches": cfg.engine.resolved_nanobatches(), "fused_gemm_reduce_scatter": bool(cfg.engine.fuse_gemm_rs and tp > 1),
                       "collective_ctas": (next((op.params.num_ctas for op in eng.graph.ops
                                                 if op.kernel == "nfk_allreduce" and op.layer >= 0), 0) if tp > 1 else 0),
                       "prefill_beside_decode": bool(cfg.engine.prefill_beside_decode),
                       "decode_tail": args.decode_tail, "net_streams": cfg.engine.net_streams,
                       "attn_overlap": bool(cfg.engine.attn_overlap),
                       "cross_layer_pipeline": bool(cfg.engine.cross_layer_pipeline),
                       "gated_gemm_behind_all_reduce": bool(cfg.engine.gate_gemm and tp > 1),
                       "o_projection_all_gather_form_nanobatches": list(cfg.engine.o_allgather_nanos),
                       "prefill_impl": cfg.engine.prefill_impl or "default",
                       "decode_impl": cfg.engine.decode_impl or "default",
                       "normed_rows_pushed_by": ("copy engines" if getattr(coll, "push_by_copy", False) else "kernel") if world > 1 else "none",
                       "symm_heap": getattr(getattr(coll, "heap", None), "backend", "none") if world > 1 else "none",
                       "all_reduce": ("in-switch (multimem)" if getattr(coll, "use_multimem", False) else
                                      "peer loads") if world > 1 else "none",
                       "kv_pages": eng.num_pages, "tokens_per_step": round(tokens_dev / args.steps, 1),
                       "l2": "inputs larger than L2 (weights per GPU >> 126 MB); no flush",
                       "steady_state": f"{args.skip_cycles} scheduler-only cycles before warm-up",
                       "baseline": "1263 tok/s/GPU, NanoFlow on 8xA100 (published)"},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d // max(1, args.steps), "d2h_bytes_per_step": d2h // max(1, args.steps),
                    "ms_per_step": round(e2e_ms / args.steps, 3), "timer": "host wall clock"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "executor": ("python" if eng.native is None else
                         "native+cuda-graph %d launches, %d rebuilds" % eng.native.graph_stats
                         if eng.native.graph_stats[0] else "native"),
            "gemm_shapes": {k: {"pick": [v["best"][x] for x in ("tile_m", "tile_n", "cta_group", "split_k", "stream_k")],
                                "us": v["us"], "model_us": v["auto_us"]} for k, v in eng.gemm_tuning.items()},
            "load_seconds": round(load_s, 1),
        }
        if args.virtual_tp > 1:
            out["invalid"] = f"virtual tensor parallelism: rank 0's share of TP{tp} on one GPU, no communication"
        if args.layers:
            out["invalid"] = "reduced layer count (debug run)"
        print(json.dumps(out))
    eng.finalize()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
