"""Interference micro-benchmark: a GEMM and an all-reduce run alone and then side by side.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 -m nanoflow_b200.parallel.overlap_bench

For each GEMM shape and each CTA budget of the collective it prints the GEMM time alone, the
all-reduce time alone, both times when launched together on two streams, and the makespan. These
are the numbers an SM-budget search needs (the reference ships the result of such a search as
``nanobatch_1_size`` / block counts in its JSON configs, not the search itself). All times are CUDA
events, max over ranks.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from nanoflow_b200 import ops
from nanoflow_b200.parallel.collectives import TpCollectives
from nanoflow_b200.runtime.pipeline import GEMM_SMEM_KB_SHARED_SM


def _t(e0, e1):
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    coll = TpCollectives(rank, world, dev, heap_bytes=512 << 20)
    rows, hidden = 3776, 8192
    buf = coll.alloc((rows, hidden), torch.bfloat16)
    hout = coll.alloc((rows, hidden), torch.bfloat16)
    wn = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    ws = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)
    s_g, s_c = torch.cuda.Stream(), torch.cuda.Stream()
    shapes = [("qkv", rows, 10240 // world, 8192, False), ("gate_up", rows, 28672 // world, 8192, True),
              ("down", rows, 8192, 28672 // world, False), ("o", rows, 8192, 8192 // world, False)]
    for name, M, N, K, swiglu in shapes:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        w2 = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 if swiglu else None
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

        def gemm():
            if swiglu:
                ops.gemm_swiglu(a, w, w2, out=out, workspace=ws, smem_budget_kb=GEMM_SMEM_KB_SHARED_SM)
            else:
                ops.gemm(a, w, out=out, workspace=ws, smem_budget_kb=GEMM_SMEM_KB_SHARED_SM)

        for ctas in (32, 64, 148, 296, 444):
            def ar():
                coll.all_reduce_(buf, norm_w=wn, norm_out=hout, num_ctas=ctas)

            res = {"gemm": name, "M": M, "N": N, "K": K, "ar_ctas": ctas, "world": world}
            for mode in ("gemm_alone", "ar_alone", "together_ar_first", "together_gemm_first"):
                times = []
                for it in range(5):
                    torch.cuda.synchronize(); dist.barrier()
                    e = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
                    e[0].record()
                    s_g.wait_event(e[0]); s_c.wait_event(e[0])
                    if mode in ("gemm_alone", "together_gemm_first"):
                        with torch.cuda.stream(s_g):
                            e[1].record(); gemm(); e[2].record()
                    if mode != "gemm_alone":
                        with torch.cuda.stream(s_c):
                            e[3].record(); ar(); e[4].record()
                    if mode == "together_ar_first":
                        with torch.cuda.stream(s_g):
                            e[1].record(); gemm(); e[2].record()
                    torch.cuda.current_stream().wait_stream(s_g)
                    torch.cuda.current_stream().wait_stream(s_c)
                    e[5].record()
                    torch.cuda.synchronize()
                    row = {"span": _t(e[0], e[5])}
                    if mode != "ar_alone":
                        row["gemm"] = _t(e[1], e[2])
                    if mode != "gemm_alone":
                        row["ar"] = _t(e[3], e[4])
                    if it >= 2:
                        times.append(row)
                res[mode] = {k: round(min(t[k] for t in times), 1) for k in times[0]}
            if rank == 0:
                print(json.dumps(res), flush=True)
    coll.check_status()
    coll.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
