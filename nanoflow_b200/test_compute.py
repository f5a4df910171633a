"""Standalone compute driver: one engine, random weights, a synthetic steady-state batch, a few timed
iterations.

    python -m nanoflow_b200.test_compute <config.json> [--iters 5] [--input-len 1024] [--output-len 512]
        [--layers N] [--skip-cycles 600]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m nanoflow_b200.test_compute <config.json>

Reads a pipeline configuration (the four-section JSON of ``nanoflow_b200/configs``), builds
random-init weights of that architecture for this rank, lets the scheduler reach the steady-state mix
of decode requests and prefill chunks for ``input-len`` / ``output-len`` requests without running the
model, then runs ``iters`` iterations and prints each one's device time. It is the install smoke test
and the quickest way to time a pipeline configuration.

Reference: ``test_compute <config.json>`` (pipeline/src/computeMain.cu:16-148: random weights,
``createUpdateData(..., 1024, 512)``, init -> config -> update -> run x5 -> finalize, per-iteration
milliseconds), run by the reference's installer as its smoke test. ``--virtual-tp`` is the reference's
``vnranks`` (pipeline/include/pipeline.h:34-35, pipeline/src/computeMain.cu:34-35): shapes of an
8-GPU job computed on fewer GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="run only the first N layers (0 = all)")
    ap.add_argument("--skip-cycles", type=int, default=600,
                    help="scheduler-only cycles before the first real iteration (reaches the steady-state mix)")
    ap.add_argument("--pages", type=int, default=0, help="KV pages (0 = from free memory)")
    ap.add_argument("--virtual-tp", type=int, default=0,
                    help="on one GPU, run rank 0's share of a tensor-parallel job of this degree with the "
                         "collectives reduced to their local part (times per-GPU work without the other GPUs)")
    a = ap.parse_args(argv)

    import torch

    from .config import load_config
    from .models import random_rank_weights
    from .runtime.engine import Engine
    from .serving import DistKVPool, RequestManager, Scheduler
    from .serving.loop import ServingLoop

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    coll = None
    if world > 1:
        import torch.distributed as dist

        from .parallel.collectives import TpCollectives

        dist.init_process_group("nccl", device_id=dev)
        coll = TpCollectives(rank, world, dev)
    tp = world
    if a.virtual_tp > 1:
        if world != 1:
            raise SystemExit("--virtual-tp runs on one GPU")
        from .parallel.collectives import TpCollectives

        tp = a.virtual_tp
        coll = TpCollectives(0, 1, dev)
    cfg = load_config(a.config, tp=tp)
    m, e = cfg.model, cfg.engine
    if a.layers:
        m.num_layers = m.run_layers = a.layers
    gbs = e.global_batch_size
    e.max_batch_size = max(e.max_batch_size, gbs)
    w = random_rank_weights(m, rank, tp, dev)
    eng = Engine(cfg, w, collectives=coll, num_pages=a.pages or None)
    n_req = int((a.skip_cycles + 4 * a.iters + 64) * gbs / (a.input_len + a.output_len)) + 256
    rm = RequestManager(vocab_size=m.vocab_size, random_ids=True, seed=0)
    for _ in range(n_req):
        rm.add_request(a.input_len, a.output_len, 0.0)
    rm.finalize_stats()
    pool = DistKVPool(m.run_layers, m.num_kv_heads, m.head_dim, eng.num_pages, e.page_size, tp)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs, nanobatch_sizes=e.resolved_nanobatches(),
                    max_batch_size=e.max_batch_size, average_prefill_length=a.input_len,
                    average_decode_length=a.output_len, group_size=m.group_size,
                    decode_tail_fraction=e.decode_tail_fraction)
    loop = ServingLoop(eng, sch, rm, simulated_time=True, est_cycle_time=1.0)
    loop.skip_cycles(a.skip_cycles)
    loop.step()
    loop.drain()                                   # one untimed iteration (first-launch costs)
    times = []
    for i in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tok0 = loop.stats.tokens_processed
        torch.cuda.synchronize()
        e0.record(eng.stream)
        loop.step()
        loop.drain()
        e1.record(eng.stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = t.item()
        times.append(ms)
        if rank == 0:
            print(f"iteration {i}: {ms:.3f} ms, {loop.stats.tokens_processed - tok0} tokens", flush=True)
    eng.check_status()
    if rank == 0:
        print(json.dumps({"config": a.config, "gpus": world, "tp": tp, "pipeline": e.pipeline_type, "dense_batch": gbs,
                          "nanobatches": e.resolved_nanobatches(), "kv_pages": eng.num_pages,
                          "ms_per_iteration": [round(t, 3) for t in times]}))
    eng.finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
