"""Multi-GPU test worker, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 tests/mp_worker.py {collectives|collectives_wide|collectives_nvls|fused|engine|engine_nvls|engine_gate|engine_gate_nvls|engine_copy|engine_copy_nvls|engine_o1|engine_o1_nvls|timeout}

Prints ``MP_WORKER_OK <case>`` from rank 0 on success; any rank's assertion failure exits non-zero.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nanoflow_b200.ops import reference as ref  # noqa: E402
from nanoflow_b200.parallel.collectives import TpCollectives  # noqa: E402


def case_collectives(rank, world, dev, wide=False, backend="ipc"):
    coll = TpCollectives(rank, world, dev, heap_bytes=512 << 20, backend=backend)
    if backend == "nvls":
        assert coll.heap.mc_base != 0, "NVLS heap without a multicast address"
        coll.use_multimem = True            # also with two ranks, where the engine would keep the peer-load form
    if rank == 0:
        print(f"symmetric heap: {coll.heap.backend}, all-reduce through the switch: {coll.use_multimem}", flush=True)
    coll.wide = wide        # 8 ranks: the all-reduce form with twice the loads in flight (same results)
    # exact integer pattern (the reference's comm_test.cu:15 uses (i*rank)%101, exact in fp16; here
    # values < 101 * world stay exact in bf16 only when small, so use (i*(rank+1)) % 13)
    for rows, cols in [(64, 1024), (37, 8192), (1, 256), (0, 512), (300, 4096)]:
        full = coll.alloc((max(rows, 1), cols), torch.bfloat16)
        buf = full[:rows]
        idx = torch.arange(rows * cols, device=dev).reshape(rows, cols)
        buf.copy_(((idx * (rank + 1)) % 13).to(torch.bfloat16))
        want = sum(((idx * (r + 1)) % 13).float() for r in range(world))
        torch.cuda.synchronize(); dist.barrier()
        coll.all_reduce_(full, rows=rows)      # rows == 0 still takes part in the handshakes
        torch.cuda.synchronize()
        coll.check_status()
        assert torch.equal(buf.float(), want), f"all-reduce mismatch {rows}x{cols} on rank {rank}"
    # random data + fused RMSNorm against the fp32 restatement
    rows, cols = 203, 8192
    g = torch.Generator(device="cpu").manual_seed(7)
    parts = [torch.randn(rows, cols, generator=g).bfloat16() for _ in range(world)]
    wnorm = (1 + 0.1 * torch.randn(cols, generator=g)).bfloat16().to(dev)
    buf = coll.alloc((rows, cols), torch.bfloat16)
    out = coll.alloc((rows, cols), torch.bfloat16)
    buf.copy_(parts[rank].to(dev))
    torch.cuda.synchronize(); dist.barrier()
    coll.all_reduce_(buf, norm_w=wnorm, norm_out=out, eps=1e-5)
    torch.cuda.synchronize()
    coll.check_status()
    total = sum(p.float() for p in parts).to(dev)
    assert torch.allclose(buf.float(), total, atol=3e-2, rtol=1e-2)
    want_n = ref.rmsnorm(buf, wnorm, 1e-5)
    assert torch.allclose(out.float(), want_n, atol=3e-2, rtol=2e-2)
    # sharded-residual form: owners add their residual rows, keep the sum locally, push only the norm
    buf.copy_(parts[rank].to(dev))
    resid = torch.randn(rows, cols, generator=g).bfloat16().to(dev)      # same on every rank
    x_loc = resid.clone()
    out.zero_()
    torch.cuda.synchronize(); dist.barrier()
    coll.all_reduce_(buf, norm_w=wnorm, norm_out=out, eps=1e-5, resid=x_loc, sum_out=x_loc, push_sum=False)
    torch.cuda.synchronize()
    coll.check_status()
    mine = torch.arange(rank, rows, world, device=dev)
    want_x = (total + resid.float())
    assert torch.allclose(x_loc[mine].float(), want_x[mine], atol=4e-2, rtol=1e-2)
    others = torch.tensor([i for i in range(rows) if i % world != rank], device=dev)
    assert torch.equal(x_loc[others], resid[others])                      # rows of other owners untouched
    assert torch.equal(buf, parts[rank].to(dev))                          # partials not overwritten
    assert torch.allclose(out.float(), ref.rmsnorm(want_x.bfloat16(), wnorm, 1e-5), atol=4e-2, rtol=3e-2)
    buf.copy_(total.bfloat16())
    # every rank holds bit-identical results (deterministic reduction order)
    gathered = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf.contiguous())
    assert all(torch.equal(gathered[0], t) for t in gathered)
    # all-gather + barrier
    ag = coll.alloc((world, 4096), torch.int32)
    ag.zero_(); ag[rank] = torch.arange(4096, device=dev, dtype=torch.int32) + 1000 * rank
    torch.cuda.synchronize(); dist.barrier()
    coll.all_gather_(ag)
    coll.barrier_()
    torch.cuda.synchronize()
    coll.check_status()
    want = torch.stack([torch.arange(4096, dtype=torch.int32) + 1000 * r for r in range(world)]).to(dev)
    assert torch.equal(ag, want)
    # column-wise all-gather: rank r owns column block r of every row (also as a view into a wider tensor)
    for rows_c, w, pad in [(37, 64, 0), (1, 256, 0), (300, 1024, 128)]:
        wide = coll.alloc((rows_c, world * w + 2 * pad), torch.bfloat16)
        wide.fill_(-2.0)
        cg = wide[:, pad:pad + world * w]
        pat = lambda r: ((torch.arange(rows_c * w, device=dev).reshape(rows_c, w) * (r + 3)) % 251).to(torch.bfloat16)
        cg[:, rank * w:(rank + 1) * w] = pat(rank)
        torch.cuda.synchronize(); dist.barrier()
        coll.all_gather_columns_(cg)
        coll.barrier_()
        torch.cuda.synchronize()
        coll.check_status()
        assert torch.equal(cg, torch.cat([pat(r) for r in range(world)], dim=1)), f"column all-gather {rows_c}x{w}"
        if pad:
            assert bool((wide[:, :pad] == -2.0).all()) and bool((wide[:, pad + world * w:] == -2.0).all())
    # reduce-scatter: the owners' rows of the sum land in a local tensor, nothing else is written
    rows, cols = 203, 1024
    parts = [torch.randn(rows, cols, generator=g).bfloat16() for _ in range(world)]
    buf = coll.alloc((rows, cols), torch.bfloat16)
    buf.copy_(parts[rank].to(dev))
    got = torch.full((rows, cols), -1.0, dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize(); dist.barrier()
    coll.reduce_scatter_(buf, got)
    coll.barrier_()
    torch.cuda.synchronize()
    coll.check_status()
    total = sum(p.float() for p in parts).to(dev)
    mine = torch.arange(rank, rows, world, device=dev)
    others = torch.tensor([i for i in range(rows) if i % world != rank], device=dev)
    assert torch.allclose(got[mine].float(), total[mine], atol=3e-2, rtol=1e-2)
    assert bool((got[others] == -1.0).all()) and torch.equal(buf, parts[rank].to(dev))
    # the same two collectives through the copy engines (one peer-to-peer copy per destination)
    ag2 = coll.alloc((world, 3, 1000), torch.float32)
    ag2.zero_(); ag2[rank] = torch.arange(3000, device=dev, dtype=torch.float32).reshape(3, 1000) + 10000 * rank
    torch.cuda.synchronize(); dist.barrier()
    coll.all_gather_copy_(ag2)
    torch.cuda.synchronize()
    coll.check_status()
    want = torch.stack([torch.arange(3000, dtype=torch.float32).reshape(3, 1000) + 10000 * r for r in range(world)])
    assert torch.equal(ag2, want.to(dev))
    n = 4096
    ar = torch.arange(n, device=dev)
    partial = torch.stack([((ar * (rank + 1) + r) % 7).to(torch.bfloat16) for r in range(world)])
    scratch = coll.alloc((world, n), torch.bfloat16)
    red = torch.empty(n, dtype=torch.bfloat16, device=dev)
    for _ in range(2):                      # twice: the second round reuses the scratch rows
        coll.reduce_scatter_copy_(partial, scratch, red)
        torch.cuda.synchronize()
        coll.check_status()
        want = sum(((ar * (s_ + 1) + rank) % 7).float() for s_ in range(world))
        assert torch.equal(red.float(), want), "copy-engine reduce-scatter"
    # bandwidth (device-timed, max over ranks)
    rows, cols = 2048, 8192
    buf = coll.alloc((rows, cols), torch.bfloat16)
    for ctas in (8, 16, 32, 64, 128):
        for _ in range(3):
            coll.all_reduce_(buf, num_ctas=ctas)
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            coll.all_reduce_(buf, num_ctas=ctas)
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            nbytes = rows * cols * 2
            busbw = 2 * (world - 1) / world * nbytes / (t.item() * 1e-3) / 1e9
            print(f"allreduce {rows}x{cols} bf16 ctas={ctas}: {t.item()*1e3:.1f} us, bus bw {busbw:.0f} GB/s", flush=True)
    # the form the engine uses: owners keep the sum (+ residual) locally and push only the normed rows
    rows, cols = 4096, 8192
    buf = coll.alloc((rows, cols), torch.bfloat16)
    hout = coll.alloc((rows, cols), torch.bfloat16)
    x_loc = torch.zeros(rows, cols, dtype=torch.bfloat16, device=dev)
    wn = torch.ones(cols, dtype=torch.bfloat16, device=dev)
    buf.normal_()
    for ctas in (32, 64, 96, 148):
        for _ in range(3):
            coll.all_reduce_(buf, norm_w=wn, norm_out=hout, resid=x_loc, sum_out=x_loc, push_sum=False, num_ctas=ctas)
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            coll.all_reduce_(buf, norm_w=wn, norm_out=hout, resid=x_loc, sum_out=x_loc, push_sum=False, num_ctas=ctas)
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            # Bytes on one GPU's links, busier direction. Pull form: in = the other ranks' partial rows of the
            # rows it owns + the other owners' normed rows (out is the mirror image). In-switch form: out =
            # its partial rows of ALL rows (the switch reads every rank's copy of every row) + its normed
            # rows once; in = the sums of its rows + the other owners' normed rows.
            own = rows // world * cols * 2
            wire = (world * own + own) if coll.use_multimem else 2 * (world - 1) * own
            print(f"allreduce+norm {rows}x{cols} bf16 ctas={ctas}: {t.item()*1e3:.1f} us "
                  f"({wire / 770e9 * 1e6:.0f} us at 770 GB/s per direction)", flush=True)
    coll.check_status()
    coll.close()


def case_fused(rank, world, dev):
    """GEMM with the reduce-scatter epilogue (partial rows pushed to their owners from the epilogue)
    followed by the slab-reading reduce + residual + norm + all-gather, against plain PyTorch."""
    import ctypes
    from nanoflow_b200 import ops
    from nanoflow_b200.ops import GemmParams

    coll = TpCollectives(rank, world, dev, heap_bytes=256 << 20)
    for M, N, K in [(300, 512, 256), (1000, 8192, 1024), (77, 256, 128), (2048, 8192, 3584 // 2 * 2)]:
        g = torch.Generator(device="cpu").manual_seed(11)
        A = [torch.randn(M, K, generator=g).bfloat16() for _ in range(world)]
        W = [(torch.randn(N, K, generator=g) * 0.05).bfloat16() for _ in range(world)]
        resid = torch.randn(M, N, generator=g).bfloat16()
        wn = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16().to(dev)
        a, w = A[rank].to(dev), W[rank].to(dev)
        cap = (M + world - 1) // world
        part = coll.alloc((world * cap, N), torch.bfloat16)
        hout = coll.alloc((M, N), torch.bfloat16)
        x_loc = resid.to(dev).clone()
        slot = coll.rs_slot(part, 0, cap)
        for rep in range(4):                      # repeated: flags carry the epoch, counters reset themselves;
            epoch = coll._next_epoch()            # the last two rounds use the staged (bulk-copy) epilogue
            p = GemmParams()
            p.rs_staged = 1 if rep >= 2 else 0
            p.A, p.B, p.D = a.data_ptr(), w.data_ptr(), 0
            p.lda, p.ldb, p.ldd = K, K, N
            p.M, p.N, p.K, p.epilogue = M, N, K, 2
            for r, base in enumerate(slot["heap"]):
                p.rs_heap[r] = base
            p.rs_rank, p.rs_nranks, p.rs_rows_cap = rank, world, cap
            p.rs_slab_off, p.rs_flag_off, p.rs_epoch = slot["slab_off"], slot["flag_off"], epoch
            p.status = coll.status.data_ptr()
            x_loc.copy_(resid.to(dev)); hout.zero_()
            torch.cuda.synchronize(); dist.barrier()
            rc = ops.lib().nfk_gemm_bf16(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0, rc
            from nanoflow_b200.parallel.collectives import AllReduceParams
            q = AllReduceParams()
            q.ctx = coll.ctx()
            q.buf_off, q.flag_off, q.src_mode, q.slab_rows = slot["slab_off"], slot["flag_off"], 1, cap
            q.rows, q.cols, q.ld, q.epoch, q.num_ctas = M, N, N, epoch, 64
            q.norm_w, q.norm_out_off, q.norm_ld, q.eps = wn.data_ptr(), coll.heap.offset_of(hout), N, 1e-5
            q.resid, q.resid_ld, q.sum_out, q.sum_ld, q.push_sum = x_loc.data_ptr(), N, x_loc.data_ptr(), N, 0
            q.status = coll.status.data_ptr()
            rc = ops.lib().nfk_allreduce(ctypes.byref(q), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0, rc
            torch.cuda.synchronize()
            coll.check_status()
            want_x = sum((A[r].float() @ W[r].float().t()).bfloat16().float() for r in range(world)) + resid.float()
            mine = torch.arange(rank, M, world)
            tol = 4e-2 * (K / 64) ** 0.5
            assert torch.allclose(x_loc[mine.to(dev)].float().cpu(), want_x[mine], atol=tol, rtol=2e-2), (M, N, K, rep)
            want_h = ref.rmsnorm(want_x.bfloat16(), wn.cpu(), 1e-5)
            assert torch.allclose(hout.float().cpu(), want_h, atol=6e-2, rtol=4e-2), (M, N, K, rep)
    coll.close()


def case_engine(rank, world, dev, backend="ipc", gate=False, by_copy=False, o1=False):
    from nanoflow_b200.config import builtin_config
    from nanoflow_b200.models import ReferenceLlama, random_full_weights, shard_weights
    from nanoflow_b200.runtime.engine import Engine
    from nanoflow_b200.serving import DistKVPool, RequestManager, Scheduler
    from nanoflow_b200.serving.loop import ServingLoop

    for ptype, nano, fuse in (("NON_OVERLAP", None, False), ("PLLM", [16, 32], False), ("PLLM", [16, 32], True),
                              ("NON_OVERLAP", None, True)):
        gbs = 48
        # two KV heads shard over two ranks; more ranks take the variant with eight KV heads
        arch = "tiny" if world <= 2 else "tiny8"
        cfg = builtin_config(arch, gpu_num=world, global_batch_size=gbs, pipeline_type=ptype, nanobatch_sizes=nano)
        cfg.engine.max_batch_size = gbs
        cfg.engine.fuse_gemm_rs = fuse
        cfg.engine.gate_gemm = gate and not fuse     # QKV / gate-up start with the all-reduce that feeds them
        if o1:
            if fuse:
                continue
            # the all-gather form of the O projection: for the first nano-batch beside the all-reduce form of the
            # second (the reference's mix), and for the only nano-batch of the in-line pipeline
            cfg.engine.o_allgather_nanos = [0]
        fw = random_full_weights(cfg.model, seed=0, std=0.05)
        for lay in fw.layers:
            for k, v in vars(lay).items():
                if v is not None:
                    setattr(lay, k, v.bfloat16().float())
        fw.embed, fw.norm, fw.lm_head = fw.embed.bfloat16().float(), fw.norm.bfloat16().float(), fw.lm_head.bfloat16().float()
        oracle = ReferenceLlama(builtin_config(arch).model, fw)
        rng = np.random.default_rng(0)
        prompts = [rng.integers(0, 1024, size=32, dtype=np.int32) for _ in range(4)]
        rm = RequestManager(vocab_size=1024)
        for p in prompts:
            rm.add_request(32, 16, 0.0, prompt=p)
        rm.finalize_stats()
        pool = DistKVPool(2, cfg.model.num_kv_heads, 64, 64, 16, world)
        sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                        nanobatch_sizes=cfg.engine.resolved_nanobatches(), average_prefill_length=32,
                        average_decode_length=16, group_size=2)
        coll = TpCollectives(rank, world, dev, heap_bytes=64 << 20, backend=backend)
        if backend == "nvls":
            coll.use_multimem = True
        coll.push_by_copy = by_copy          # normed rows delivered by copy-engine copies + a closing barrier
        eng = Engine(cfg, shard_weights(fw, cfg.model, rank, world, device=dev, o1=o1), device=dev, collectives=coll,
                     num_pages=64)
        if o1:
            assert any(op.name.endswith(".o1") for op in eng.graph.ops)
        st = ServingLoop(eng, sch, rm, est_cycle_time=1.0).run()
        eng.check_status(); coll.check_status()
        eng.finalize()
        assert len(st.retired) == 4
        outs = {r.req_idx: r.output for r in st.retired}
        # all ranks agree on every sampled token
        flat = torch.tensor([t for i in sorted(outs) for t in outs[i]], device=dev)
        gathered = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree on sampled tokens"
        for i, out in outs.items():
            seq = torch.tensor(prompts[i].tolist() + out[:-1])
            logits, _ = oracle.forward(seq)
            steps = logits[31:]
            gap = steps.max(dim=-1).values - steps[torch.arange(16), torch.tensor(out)]
            assert gap.max().item() < 0.05 * steps.abs().max().item(), f"{ptype}: token far from oracle arg-max"
        coll.close()
        dist.barrier()


def case_timeout(rank, world, dev):
    """A collective whose peers never arrive ends by itself with a status code; the context stays usable.
    Rank 0 alone calls the all-reduce (nobody else signals), then everyone proves the GPU still works."""
    coll = TpCollectives(rank, world, dev, heap_bytes=16 << 20, backend="ipc")   # nothing bound in the switch
    buf = coll.alloc((8, 256), torch.bfloat16)
    spare = coll.new_flags()
    torch.cuda.synchronize(); dist.barrier()
    spare2 = coll.new_flags()
    if rank == 0:
        coll.all_reduce_(buf, flag_off=spare, epoch=1)
        # a second collective behind the one that timed out gives up at once: the status word is already
        # set, so a dead peer costs one time limit per iteration, not one per collective
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        coll.all_reduce_(buf, flag_off=spare2, epoch=1)
        e1.record()
        torch.cuda.synchronize()
        assert e0.elapsed_time(e1) < 500.0, f"second collective waited {e0.elapsed_time(e1):.0f} ms"
        try:
            coll.check_status()
            raise AssertionError("expected a peer-flag timeout")
        except RuntimeError as e:
            assert "0x500" in str(e)
    dist.barrier()
    x = torch.ones(4, device=dev)
    dist.all_reduce(x)
    assert x[0].item() == world
    coll.close()


if __name__ == "__main__":
    case = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        {"collectives": case_collectives, "collectives_wide": lambda r, w, d: case_collectives(r, w, d, wide=True),
         "collectives_nvls": lambda r, w, d: case_collectives(r, w, d, backend="nvls"),
         "engine": case_engine, "engine_nvls": lambda r, w, d: case_engine(r, w, d, backend="nvls"),
         "engine_copy": lambda r, w, d: case_engine(r, w, d, by_copy=True),
         "engine_copy_nvls": lambda r, w, d: case_engine(r, w, d, backend="nvls", by_copy=True),
         "engine_o1": lambda r, w, d: case_engine(r, w, d, o1=True),
         "engine_o1_nvls": lambda r, w, d: case_engine(r, w, d, backend="nvls", o1=True),
         "engine_gate": lambda r, w, d: case_engine(r, w, d, gate=True),
         "engine_gate_nvls": lambda r, w, d: case_engine(r, w, d, backend="nvls", gate=True),
         "timeout": case_timeout, "fused": case_fused}[case](rank, world, dev)
    except BaseException:
        import traceback
        print(f"MP_WORKER_FAIL rank {rank}\n" + traceback.format_exc(), flush=True)
        raise
    dist.barrier()
    if rank == 0:
        print(f"MP_WORKER_OK {case}", flush=True)
    dist.destroy_process_group()
