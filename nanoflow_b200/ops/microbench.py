"""Per-kernel micro-benchmarks: ``python -m nanoflow_b200.ops.microbench [gemm|swiglu|smallm|decode|prefill|norm|hostlink|budget|library|interference|all]``
(JSON lines; ``... table rows.jsonl`` turns them into a markdown table).

Each case is timed with CUDA events on the launching stream after warm-up, with an L2 flush (a
write larger than the 126 MB L2) between timed launches, and reported against the measured peaks
in ``MEASURED_PEAKS.json`` at the repository root (copy bandwidth, cuBLAS bf16 throughput) when that
file exists. This is the counterpart of the reference's NVBench drivers
(gemv/src/bench_batch_decode.cu:222-249, gemv/src/bench_batch_prefill.cu:142-151) and of
``CutlassGEMMWrapper::profile`` (pipeline/include/cutlassGemmWrapperImpl.cuh:378-418).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from nanoflow_b200 import ops

_FLUSH = None


def peaks():
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_ms(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemm(shapes=None, swiglu=False, tile_ns=(0,), num_ctas=0):
    _, tf_peak, how = peaks()
    shapes = shapes or [
        # Llama-2-70B TP8 per-GPU shapes (M = dense batch 2048 and nano-batches)
        (2048, 1280, 8192), (2048, 8192, 1024), (2048, 8192, 3584), (640, 1280, 8192),
        (1408, 8192, 3584), (4096, 8192, 3584),
        # TP1 shapes
        (2048, 10240, 8192), (2048, 8192, 8192), (2048, 8192, 28672), (256, 8192, 8192),
        # Llama-3-8B TP1
        (2048, 6144, 4096), (2048, 4096, 4096), (2048, 4096, 14336), (8192, 8192, 8192),
    ]
    rows = []
    for (M, N, K) in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        w2 = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 if swiglu else None
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ws = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")
        for tn in tile_ns:
            if swiglu:
                fn = lambda: ops.gemm_swiglu(a, w, w2, out=out, tile_n=tn, num_ctas=num_ctas, workspace=ws)
                flops = 4.0 * M * N * K
            else:
                fn = lambda: ops.gemm(a, w, out=out, tile_n=tn, num_ctas=num_ctas, workspace=ws)
                flops = 2.0 * M * N * K
            med, best = time_ms(fn)
            ref_fn = (lambda: torch.matmul(a, w.t(), out=out))
            rmed, _ = time_ms(ref_fn)
            rflops = 2.0 * M * N * K
            rows.append(dict(op="swiglu" if swiglu else "gemm", M=M, N=N, K=K, tile_n=tn,
                             ms=round(med, 4), tflops=round(flops / med / 1e9, 1),
                             frac_of_peak=round(flops / med / 1e9 / tf_peak, 3), peak=how,
                             cublas_ms=round(rmed, 4), cublas_tflops=round(rflops / rmed / 1e9, 1)))
            print(json.dumps(rows[-1]), flush=True)
    return rows


def _paged(batch, ctx, kv_heads, hd, qo_len=1):
    page = 16
    np_ = (ctx + page - 1) // page
    total = batch * np_
    pool = torch.randn(total, 2, kv_heads, page, hd, device="cuda", dtype=torch.bfloat16)
    kv_indptr = torch.arange(0, batch + 1, dtype=torch.int32, device="cuda") * np_
    kv_indices = torch.randperm(total, device="cuda").int()
    last = torch.full((batch,), (ctx - 1) % page + 1, dtype=torch.int32, device="cuda")
    qo = torch.arange(0, batch + 1, dtype=torch.int32, device="cuda") * qo_len
    return pool, qo, kv_indptr, kv_indices, last


def bench_decode():
    bw_peak, _, how = peaks()
    for (batch, ctx, kv_heads, group, ctas) in [(2731, 1280, 1, 8, 0), (683, 1280, 1, 8, 0), (683, 1280, 1, 8, 64),
                                                 (256, 1280, 8, 8, 0), (1024, 1280, 8, 4, 0), (64, 4096, 8, 8, 0)]:
        hd = 128
        q_heads = kv_heads * group
        pool, qo, kvp, kvi, last = _paged(batch, ctx, kv_heads, hd)
        q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        fn = lambda: ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0,
                                     req_count=batch, num_ctas=ctas)
        med, best = time_ms(fn)
        nbytes = batch * ctx * kv_heads * hd * 2 * 2 + 2 * q.numel() * 2
        print(json.dumps(dict(op="attn_decode", batch=batch, ctx=ctx, kv_heads=kv_heads, group=group,
                              num_ctas=ctas, ms=round(med, 4), gbs=round(nbytes / med / 1e6, 1),
                              frac_of_peak=round(nbytes / med / 1e6 / bw_peak, 3), peak=how)), flush=True)


def bench_prefill():
    _, tf_peak, how = peaks()
    for (batch, ctx, kv_heads, group) in [(2, 1024, 1, 8), (4, 1024, 1, 8), (2, 1024, 8, 8), (8, 1024, 8, 4), (1, 4096, 8, 8)]:
        hd = 128
        q_heads = kv_heads * group
        pool, qo, kvp, kvi, last = _paged(batch, ctx, kv_heads, hd, qo_len=ctx)
        q = torch.randn(batch * ctx, q_heads * hd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        tq = 128 // group
        items = torch.tensor([[b, b * ctx + t, min(tq, ctx - t)] for b in range(batch)
                              for t in range(0, ctx, tq)], dtype=torch.int32, device="cuda")
        flops = 4.0 * batch * q_heads * hd * ctx * ctx / 2
        for impl in ("ws", "tc", "mma"):
            fn = lambda: ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=q_heads, impl=impl)
            med, best = time_ms(fn)
            print(json.dumps(dict(op="attn_prefill_" + impl, batch=batch, ctx=ctx, kv_heads=kv_heads, group=group,
                                  ms=round(med, 4), tflops=round(flops / med / 1e9, 1),
                                  frac_of_peak=round(flops / med / 1e9 / tf_peak, 3), peak=how)), flush=True)


def bench_library_attention():
    """Same-box comparison rows: this package's decode / prefill attention kernels and the installed
    ``flashinfer`` library's on the same paged KV pool (HND layout, page 16, bf16, head_dim 128). A comparator
    only: nothing on the serving path calls the library. Its kernels are compiled on first use (or found in
    its cache directory, FLASHINFER_WORKSPACE_BASE); a form that cannot be built or run here gives a row with
    ``unavailable`` and the first line of the reason. The reference links a FlashInfer fork for the same two
    kernels (gemv/include/attention/decode.cuh, prefill.cuh)."""
    bw_peak, tf_peak, how = peaks()
    hd, page = 128, 16

    def row(**kw):
        print(json.dumps(kw), flush=True)

    def guarded(op, shape, make, rate):
        try:
            fn = make()
            med, _ = time_ms(fn)
            row(op=op, **shape, ms=round(med, 4), **rate(med), peak=how)
        except Exception as e:      # a missing compiler, cache or kernel image is a result here, not an error
            row(op=op, **shape, unavailable=(str(e).strip().splitlines() or [type(e).__name__])[0][:200])

    try:
        import flashinfer
    except Exception as e:
        row(op="flashinfer", unavailable=str(e)[:200])
        return
    fws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
    for (batch, ctx, kv_heads, group) in [(2731, 1280, 1, 8), (683, 1280, 1, 8), (256, 1280, 8, 8)]:
        q_heads = kv_heads * group
        pool, qo, kvp, kvi, last = _paged(batch, ctx, kv_heads, hd)
        q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        shape = dict(batch=batch, ctx=ctx, kv_heads=kv_heads, group=group)
        nbytes = batch * ctx * kv_heads * hd * 2 * 2 + 2 * q.numel() * 2
        rate = lambda med: dict(gbs=round(nbytes / med / 1e6, 1), frac_of_peak=round(nbytes / med / 1e6 / bw_peak, 3))
        guarded("attn_decode", shape, lambda: (lambda: ops.attn_decode(
            q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch)), rate)

        def fa2():
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(fws, "HND", use_tensor_cores=True)
            w.plan(kvp, kvi, last, q_heads, kv_heads, hd, page, q_data_type=torch.bfloat16,
                   kv_data_type=torch.bfloat16)
            q3 = q.view(batch, q_heads, hd)
            o3 = w.run(q3, pool)
            want = torch.empty_like(q)
            ops.attn_decode(q, want, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch)
            torch.cuda.synchronize()
            err = (o3.reshape(batch, -1).float() - want.float()).abs().max().item()
            if err > 0.05:
                raise RuntimeError(f"library result differs from this package's by {err:.3f}")
            return lambda: w.run(q3, pool)
        guarded("attn_decode_flashinfer_fa2", shape, fa2, rate)

        def trtllm():
            npages = (ctx + page - 1) // page
            tables = kvi.view(batch, npages).contiguous()
            lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
            ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
            q3 = q.view(batch, q_heads, hd)
            call = lambda: flashinfer.decode.trtllm_batch_decode_with_kv_cache(
                q3, pool, ws, tables, lens, ctx, hd ** -0.5, 1.0, kv_layout="HND")
            o3 = call()
            want = torch.empty_like(q)
            ops.attn_decode(q, want, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch)
            torch.cuda.synchronize()
            err = (o3.reshape(batch, -1).float() - want.float()).abs().max().item()
            if err > 0.05:
                raise RuntimeError(f"library result differs from this package's by {err:.3f}")
            return call
        guarded("attn_decode_flashinfer_trtllm_gen", shape, trtllm, rate)
        del pool

    for (batch, ctx, kv_heads, group) in [(4, 1024, 1, 8), (8, 1024, 8, 4), (1, 4096, 8, 8)]:
        q_heads = kv_heads * group
        pool, qo, kvp, kvi, last = _paged(batch, ctx, kv_heads, hd, qo_len=ctx)
        q = torch.randn(batch * ctx, q_heads * hd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        tq = 128 // group
        items = torch.tensor([[b, b * ctx + t, min(tq, ctx - t)] for b in range(batch)
                              for t in range(0, ctx, tq)], dtype=torch.int32, device="cuda")
        flops = 4.0 * batch * q_heads * hd * ctx * ctx / 2
        shape = dict(batch=batch, ctx=ctx, kv_heads=kv_heads, group=group)
        rate = lambda med: dict(tflops=round(flops / med / 1e9, 1), frac_of_peak=round(flops / med / 1e9 / tf_peak, 3))
        guarded("attn_prefill_ws", shape, lambda: (lambda: ops.attn_prefill(
            q, out, pool, qo, kvp, kvi, last, items, q_heads=q_heads, impl="ws")), rate)

        def fa2p():
            w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(fws, "HND")
            w.plan(qo, kvp, kvi, last, q_heads, kv_heads, hd, page, causal=True, q_data_type=torch.bfloat16,
                   kv_data_type=torch.bfloat16)
            q3 = q.view(batch * ctx, q_heads, hd)
            o3 = w.run(q3, pool)
            ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=q_heads, impl="ws")
            torch.cuda.synchronize()
            err = (o3.reshape(batch * ctx, -1).float() - out.float()).abs().max().item()
            if err > 0.05:
                raise RuntimeError(f"library result differs from this package's by {err:.3f}")
            return lambda: w.run(q3, pool)
        guarded("attn_prefill_flashinfer_fa2", shape, fa2p, rate)

        def trtllm_p():
            npages = (ctx + page - 1) // page
            tables = kvi.view(batch, npages).contiguous()
            lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
            ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
            q3 = q.view(batch * ctx, q_heads, hd)
            call = lambda: flashinfer.prefill.trtllm_batch_context_with_kv_cache(
                q3, pool, ws, tables, lens, ctx, ctx, hd ** -0.5, 1.0, batch, qo, qo, kv_layout="HND")
            o3 = call()
            ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=q_heads, impl="ws")
            torch.cuda.synchronize()
            err = (o3.reshape(batch * ctx, -1).float() - out.float()).abs().max().item()
            if err > 0.05:
                raise RuntimeError(f"library result differs from this package's by {err:.3f}")
            return call
        guarded("attn_prefill_flashinfer_trtllm_gen", shape, trtllm_p, rate)
        del pool


def bench_interference():
    """A GEMM beside a collective kernel that moves local data only: the all-reduce + residual + RMSNorm kernel
    with one rank (every load and store local, 268 MB through HBM per call) on a second stream beside the TP8
    per-GPU GEMMs of Llama-2-70B at M = 4096, for several CTA counts of the collective; then pinned tile shapes
    with the tiles dealt statically to persistent CTAs (stream_k = 2) and one work unit per CTA dealt by the
    hardware block scheduler (stream_k = 3). Separates what sharing SMs with a collective's CTAs costs from
    what the collective's NVLink traffic costs (which needs the other GPUs: ``parallel/overlap_bench.py``)."""
    from nanoflow_b200.parallel.collectives import TpCollectives
    dev = torch.device("cuda", torch.cuda.current_device())
    coll = TpCollectives(0, 1, dev, heap_bytes=768 << 20)
    rows, hidden = 4096, 8192
    buf = coll.alloc((rows, hidden), torch.bfloat16)
    buf.normal_()
    hout = coll.alloc((rows, hidden), torch.bfloat16)
    resid = torch.randn(rows, hidden, device=dev, dtype=torch.bfloat16)
    xout = torch.empty_like(resid)
    wn = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    ws = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)
    s_g, s_c = torch.cuda.Stream(), torch.cuda.Stream()

    def timed(fn_g, fn_c=None, reps_c=1, iters=8):
        ts = []
        for _ in range(3 + iters):
            flush_l2()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if fn_c is not None:
                with torch.cuda.stream(s_c):
                    c0.record()
                    for _ in range(reps_c):
                        fn_c()
                    c1.record()
            with torch.cuda.stream(s_g):
                e0.record()
                fn_g()
                e1.record()
            torch.cuda.synchronize()
            ts.append((e0.elapsed_time(e1) * 1e3, c0.elapsed_time(c1) * 1e3 if fn_c is not None else 0.0))
        ts = sorted(ts[3:])
        return ts[len(ts) // 2]

    def collective(ctas):
        return lambda: coll.all_reduce_(buf, norm_w=wn, norm_out=hout, num_ctas=ctas, resid=resid, sum_out=xout,
                                        push_sum=False)

    for name, M, N, K in [("qkv", 4096, 1280, 8192), ("o", 4096, 8192, 1024), ("down", 4096, 8192, 3584)]:
        a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        g = lambda: ops.gemm(a, w, out=out, workspace=ws, smem_budget_kb=200)
        alone = timed(g)[0]
        for ctas in (16, 32, 96, 148):
            ar_alone = timed(collective(ctas))[0]
            both = timed(g, collective(ctas), reps_c=2)     # two calls, so that the collective outlasts the GEMM
            print(json.dumps(dict(op="gemm_beside_local_collective", gemm=name, gemm_alone_us=round(alone, 1),
                                  ar_ctas=ctas, ar_alone_us=round(ar_alone, 1), gemm_beside_us=round(both[0], 1),
                                  two_ars_beside_us=round(both[1], 1))), flush=True)
        for tn, cg, sk in [(256, 2, 0), (128, 2, 0), (256, 1, 0), (128, 1, 0), (256, 2, 2), (128, 2, 2)]:
            try:
                for mode in (2, 3):
                    gg = lambda: ops.gemm(a, w, out=out, workspace=ws, smem_budget_kb=200, tile_n=tn, cta_group=cg,
                                          split_k=sk, stream_k=mode)
                    al = timed(gg)[0]
                    both = timed(gg, collective(32), reps_c=2)
                    print(json.dumps(dict(op="gemm_tile_deal", gemm=name, tile_n=tn, cta_group=cg, split_k=sk,
                                          stream_k=mode, alone_us=round(al, 1), beside_us=round(both[0], 1),
                                          two_ars_us=round(both[1], 1))), flush=True)
            except RuntimeError as e:       # e.g. split-K partial sums larger than the workspace
                print(json.dumps(dict(op="gemm_tile_deal", gemm=name, tile_n=tn, cta_group=cg, split_k=sk,
                                      error=str(e)[:100])), flush=True)
    coll.check_status()
    coll.close()


def bench_budget():
    """Decode attention against its CTA budget, alone and beside back-to-back GEMMs on a second stream:
    the table an SM-budget search needs (the reference sweeps ``sm_blk`` the same way,
    gemv/src/bench_batch_decode.cu:222-249, and ships only the chosen numbers in its configs).

    Shapes are one GPU's share of Llama-2-70B at TP8 in the 1024/512 steady state: 2731 decode requests x
    one KV head, ~1280 tokens of context; the GEMM is the gate/up projection of a 2048-row nano-batch."""
    bw_peak, tf_peak, how = peaks()
    batch, ctx, kv_heads, group, hd = 2731, 1280, 1, 8, 128
    q_heads = kv_heads * group
    pool, qo, kvp, kvi, last = _paged(batch, ctx, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    nbytes = batch * ctx * kv_heads * hd * 2 * 2 + 2 * q.numel() * 2
    M, F, K = 2048, 3584, 8192
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.02
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.02
    act = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")
    gflop = 4.0 * M * F * K
    s_a, s_g = torch.cuda.Stream(), torch.cuda.Stream()
    n_gemm = 3

    def run(ctas, stages, smem_kb, mode, impl=""):
        """mode: 'decode', 'gemm' or 'both'. Returns (decode us, gemm us per launch, span us), best of 5."""
        best = None
        for it in range(7):
            flush_l2()
            torch.cuda.synchronize()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
            e[0].record()
            s_a.wait_event(e[0]); s_g.wait_event(e[0])
            if mode in ("gemm", "both"):
                with torch.cuda.stream(s_g):
                    e[1].record()
                    for _ in range(n_gemm):
                        ops.gemm_swiglu(a, wg, wu, out=act, workspace=ws, smem_budget_kb=smem_kb)
                    e[2].record()
            if mode in ("decode", "both"):
                with torch.cuda.stream(s_a):
                    e[3].record()
                    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                                    num_ctas=ctas, stages=stages, impl=impl)
                    e[4].record()
            torch.cuda.current_stream().wait_stream(s_a)
            torch.cuda.current_stream().wait_stream(s_g)
            e[5].record()
            torch.cuda.synchronize()
            row = (e[3].elapsed_time(e[4]) * 1e3 if mode != "gemm" else 0.0,
                   e[1].elapsed_time(e[2]) * 1e3 / n_gemm if mode != "decode" else 0.0,
                   e[0].elapsed_time(e[5]) * 1e3)
            if it >= 2 and (best is None or row[2] < best[2]):
                best = row
        return best

    for smem_kb in (0, 200, 160, 130, 128, 96):
        _, g_us, _ = run(0, 0, smem_kb, "gemm")
        print(json.dumps(dict(op="budget_gemm_alone", M=M, F=F, K=K, smem_kb=smem_kb, us=round(g_us, 1),
                              tflops=round(gflop / g_us / 1e6, 1), peak=how)), flush=True)
    # (kernel, pages in flight per warp, shared memory a GEMM CTA may keep beside one such CTA)
    for impl, stages, smem_kb in (("", 3, 128), ("", 2, 160), ("tma", 2, 160), ("tma", 3, 128), ("tma", 4, 96)):
        for ctas in (16, 32, 48, 64, 96, 148, 296):
            if ctas > 148 and stages == 4:
                continue
            d_us, _, _ = run(ctas, stages, 0, "decode", impl)
            row = dict(op="budget_decode", impl=impl or "cp.async", num_ctas=ctas, stages=stages, alone_us=round(d_us, 1),
                       alone_frac_of_peak=round(nbytes / d_us / 1e3 / bw_peak, 3), peak=how)
            if ctas <= 148:
                d2, g2, span = run(ctas, stages, smem_kb, "both", impl)
                row.update(beside_gemm_smem_kb=smem_kb, beside_us=round(d2, 1), gemm_beside_us=round(g2, 1),
                           span_us=round(span, 1))
            print(json.dumps(row), flush=True)


def bench_norm():
    bw_peak, _, how = peaks()
    for rows, cols in [(2048, 8192), (16384, 8192), (2048, 4096)]:
        x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(cols, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(x)
        med, _ = time_ms(lambda: ops.rmsnorm(x, w, 1e-5, out=out))
        nbytes = 2 * x.numel() * 2
        print(json.dumps(dict(op="rmsnorm", rows=rows, cols=cols, ms=round(med, 4),
                              gbs=round(nbytes / med / 1e6, 1),
                              frac_of_peak=round(nbytes / med / 1e6 / bw_peak, 3), peak=how)), flush=True)


def small_case(which: str):
    """A few launches of one kernel on inputs larger than L2 (for a profiler capture)."""
    if which == "gemm":
        M, N, K = 4096, 8192, 8192
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(4):
            ops.gemm(a, w, out=out)
    elif which == "gemm_m256":
        # the one-GPU dense batch: every weight byte is streamed once per call (134 MB, larger than L2)
        M, N, K = 256, 8192, 8192
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ws = torch.zeros(160 << 20, dtype=torch.uint8, device="cuda")
        for _ in range(4):
            ops.gemm(a, w, out=out, workspace=ws)
    elif which == "gemm_shapes":
        # one launch per kernel shape: CTA pair 256 wide, CTA pair 128 wide, single CTA 256 wide
        M, N, K = 4096, 8192, 8192
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for cg, tn in ((2, 256), (2, 128), (1, 256)):
            ops.gemm(a, w, out=out, tile_n=tn, tile_m=1, cta_group=cg)
    elif which == "swiglu":
        M, N, K = 4096, 7168, 8192
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        w2 = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(4):
            ops.gemm_swiglu(a, w, w2, out=out)
    elif which == "decode":
        pool, qo, kvp, kvi, last = _paged(512, 1280, 8, 128)
        q = torch.randn(512, 64 * 128, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        for _ in range(4):
            ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=64, req_begin=0, req_count=512)
    elif which == "prefill_tc":
        pool, qo, kvp, kvi, last = _paged(4, 1024, 8, 128, qo_len=1024)
        q = torch.randn(4096, 64 * 128, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        items = torch.tensor([[b, b * 1024 + t, 16] for b in range(4) for t in range(0, 1024, 16)],
                             dtype=torch.int32, device="cuda")
        for _ in range(3):
            ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=64, impl="tc")
    elif which == "prefill_ws":
        pool, qo, kvp, kvi, last = _paged(4, 1024, 8, 128, qo_len=1024)
        q = torch.randn(4096, 64 * 128, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        items = torch.tensor([[b, b * 1024 + t, 16] for b in range(4) for t in range(0, 1024, 16)],
                             dtype=torch.int32, device="cuda")
        for _ in range(3):
            ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=64, impl="ws")
    elif which == "decode_tma":
        pool, qo, kvp, kvi, last = _paged(512, 1280, 8, 128)
        q = torch.randn(512, 64 * 128, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        for _ in range(4):
            ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=64, req_begin=0, req_count=512, impl="tma")
    elif which == "prefill":
        pool, qo, kvp, kvi, last = _paged(4, 1024, 8, 128, qo_len=1024)
        q = torch.randn(4096, 64 * 128, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        items = torch.tensor([[b, b * 1024 + t, 16] for b in range(4) for t in range(0, 1024, 16)],
                             dtype=torch.int32, device="cuda")
        for _ in range(4):
            ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=64, impl="mma")
    torch.cuda.synchronize()
    print("small case done:", which)


def bench_hostlink():
    """Pinned host <-> device copy bandwidth (the per-iteration metadata upload, the sampled tokens and
    the KV offload go over this link). Counterpart in the reference: pipeline/src/pythonProfiling.py,
    which measures pinned H2D / D2H bandwidth before compressing its traces."""
    for mb in (1, 16, 256):
        n = mb << 20
        host = torch.empty(n, dtype=torch.uint8).pin_memory()
        dev = torch.empty(n, dtype=torch.uint8, device="cuda")
        for name, fn in (("h2d", lambda: dev.copy_(host, non_blocking=True)),
                         ("d2h", lambda: host.copy_(dev, non_blocking=True))):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            print(json.dumps(dict(op=f"hostlink_{name}", mbytes=mb, ms=round(ms, 4), gbs=round(n / ms / 1e6, 1))),
                  flush=True)


def table(path: str) -> str:
    """Markdown table from the JSON lines this module prints (``... all > rows.jsonl``)."""
    hbm, tf, how = peaks()
    out = ["| op | shape | ms | TFLOP/s or GB/s | of " + how + " peak | cuBLAS TFLOP/s (same shape) |", "|---|---|---|---|---|---|"]
    for line in open(path):
        line = line.strip()
        if not line.startswith("{"):
            continue
        d = json.loads(line)
        shape = " ".join(f"{k}={d[k]}" for k in ("M", "N", "F", "K", "batch", "ctx", "kv_heads", "group", "rows", "cols",
                                                  "mbytes", "tile_m", "tile_n", "split_k", "num_ctas") if k in d)
        if "tflops" in d:
            rate, frac = f"{d['tflops']} TFLOP/s", d.get("frac_of_peak", round(d["tflops"] / tf, 3))
        else:
            rate = f"{d.get('gbs', '')} GB/s"
            frac = d.get("frac_of_peak", d.get("frac_of_bw", round(d["gbs"] / hbm, 3) if "gbs" in d else ""))
        out.append(f"| {d['op']} | {shape} | {d.get('ms', '')} | {rate} | {frac} | {d.get('cublas_tflops', '')} |")
    return "\n".join(out)


def main(argv):
    what = argv[1] if len(argv) > 1 else "all"
    if what == "table":
        print(table(argv[2]))
        return
    if what.startswith("small_"):
        small_case(what[len("small_"):])
        return
    if what == "smallm":
        ws = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
        bw_peak = peaks()[0]
        for (M, N, K) in [(256, 10240, 8192), (256, 8192, 8192), (256, 8192, 28672), (128, 8192, 28672),
                          (512, 8192, 28672), (256, 1280, 8192), (256, 8192, 3584), (85, 32000, 8192)]:
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            for (tm, tn, sk) in [(0, 0, 0), (2, 256, 1), (2, 256, 4), (2, 224, 3), (2, 224, 4), (2, 192, 3), (2, 128, 2),
                                 (1, 128, 1)]:
                try:
                    med, _ = time_ms(lambda: ops.gemm(a, w, out=out, tile_m=tm, tile_n=tn, split_k=sk, workspace=ws))
                except RuntimeError:
                    continue
                gbs = (N * K * 2 + M * K * 2 + M * N * 2) / med / 1e6
                print(json.dumps(dict(op="gemm_smallm", M=M, N=N, K=K, tile_m=tm, tile_n=tn, split_k=sk,
                                      ms=round(med, 4), gbs=round(gbs, 1), frac_of_bw=round(gbs / bw_peak, 3))), flush=True)
            med, _ = time_ms(lambda: torch.matmul(a, w.t(), out=out))
            print(json.dumps(dict(op="cublas", M=M, N=N, K=K, ms=round(med, 4),
                                  gbs=round((N * K * 2 + M * K * 2 + M * N * 2) / med / 1e6, 1))), flush=True)
        for (M, F, K) in [(256, 28672, 8192), (256, 3584, 8192)]:
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.02
            w2 = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.02
            out = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
            for (tm, tn) in [(0, 0), (2, 256), (2, 224), (2, 192), (1, 256)]:
                med, _ = time_ms(lambda: ops.gemm_swiglu(a, w, w2, out=out, tile_m=tm, tile_n=tn, workspace=ws))
                gbs = (2 * F * K * 2) / med / 1e6
                print(json.dumps(dict(op="swiglu_smallm", M=M, F=F, K=K, tile_m=tm, tile_n=tn, ms=round(med, 4),
                                      gbs=round(gbs, 1), frac_of_bw=round(gbs / bw_peak, 3))), flush=True)
        return
    if what in ("gemm", "all"):
        bench_gemm()
    if what in ("swiglu", "all"):
        bench_gemm(shapes=[(2048, 3584, 8192), (640, 3584, 8192), (2048, 28672, 8192), (2048, 14336, 4096)],
                   swiglu=True)
    if what in ("decode", "all"):
        bench_decode()
    if what in ("prefill", "all"):
        bench_prefill()
    if what == "budget":
        bench_budget()
    if what == "library":
        bench_library_attention()
    if what == "interference":
        bench_interference()
    if what in ("norm", "all"):
        bench_norm()
    if what in ("hostlink", "all"):
        bench_hostlink()


if __name__ == "__main__":
    main(sys.argv)
