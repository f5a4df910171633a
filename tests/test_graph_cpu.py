"""Static checks of the op graph on CPU: every pipeline variant builds, dependencies only point
backwards, and no two ops that touch the same bytes (one of them writing) are left unordered."""
import pytest
import torch

from nanoflow_b200.config import builtin_config
from nanoflow_b200.models import random_full_weights, shard_weights
from nanoflow_b200.parallel.collectives import TpCollectives
from nanoflow_b200.runtime.pipeline import Buffers, IoSpec, build_graph
from nanoflow_b200.utils import depcheck


def _host_graph(pipeline_type, tp, nano, gbs=48, fuse_rs=False, net_streams=1, fake_wire=0.0, attn_overlap=False,
                cross_layer=False, o_allgather=(), by_copy=False):
    cfg = builtin_config("tiny", gpu_num=tp, global_batch_size=gbs, pipeline_type=pipeline_type, nanobatch_sizes=nano)
    m, e = cfg.model, cfg.engine
    e.fuse_gemm_rs = fuse_rs
    e.net_streams = net_streams
    e.attn_overlap = attn_overlap
    e.cross_layer_pipeline = cross_layer
    e.o_allgather_nanos = list(o_allgather)
    e.max_batch_size = gbs
    fw = random_full_weights(m, seed=0)
    w = shard_weights(fw, m, 0, tp, dtype=torch.bfloat16, o1=bool(o_allgather))
    coll = TpCollectives.for_analysis(0, tp) if tp > 1 else None
    if coll is not None:
        coll.fake_wire_us_per_row = fake_wire
        coll.push_by_copy = by_copy
    bf = torch.bfloat16
    z = lambda *s, dtype=bf: torch.zeros(*s, dtype=dtype)
    sym = (lambda *s, dtype=bf: coll.alloc(s, dtype)) if coll else z
    T, B = gbs, gbs
    sizes = e.resolved_nanobatches()
    meta_dev = torch.zeros(8 * T + 8 * B + 4096, dtype=torch.int32)
    names = ["host_ids", "feedback_src", "positions", "token_req", "qo_indptr", "kv_indptr", "kv_last_page_len",
             "sample_rows", "kv_indices"]
    meta = {n: meta_dev[i * (T + 8):(i + 1) * (T + 8)] for i, n in enumerate(names)}
    x0 = z(T, m.hidden_size)
    pools = [z(16, 2, m.kv_heads_local, 16, m.head_dim) for _ in range(m.run_layers)]
    bufs = Buffers(x=[x0, sym(T + 8 * len(sizes), m.hidden_size) if tp > 1 else x0], h=sym(T, m.hidden_size),
                   qkv=z(T, m.qkv_size_local), q_rot=z(T, m.q_size_local), attn_out=z(T, m.q_size_local),
                   act=z(T, m.ffn_local), sample_h=z(B, m.hidden_size), sample_hn=z(B, m.hidden_size),
                   logits=z(B, w.lm_head.shape[0]), cand_val=sym(tp, B, dtype=torch.float32),
                   cand_idx=sym(tp, B, dtype=torch.int32), sampled=z(B, dtype=torch.int32), kv_pool=pools,
                   inv_freq=torch.zeros(m.head_dim // 2), status=torch.zeros(1, dtype=torch.int32),
                   decode_ws=torch.zeros(1024), meta=meta,
                   nano_items=[torch.zeros(s + 2, 3, dtype=torch.int32) for s in sizes],
                   gemm_ws=torch.zeros(1 << 16),
                   attn_full=sym(T, m.q_size_local * tp) if (o_allgather and tp > 1) else None)
    io = IoSpec(meta_dev, 4 * T, 8 * T)
    g = build_graph(m, e, w, bufs, coll, io)
    starts = [sum(sizes[:k]) for k in range(len(sizes))]
    pool_bytes = pools[0].numel() * 2
    acc = depcheck.graph_access(g, starts, sizes, heap_base=coll.heap.base if coll else 0, kv_pool_bytes=pool_bytes,
                                peer_bases=list(coll.heap.peer_base) if coll else ())
    return g, acc, (bufs, w, coll, meta_dev)


@pytest.mark.parametrize("pipeline_type,tp,nano", [
    ("NON_OVERLAP_LOCAL", 1, None), ("NANOBATCH_LOCAL", 1, [16, 32]), ("LOCAL", 1, [16, 32]),
    ("NON_OVERLAP", 2, None), ("NANOBATCH", 2, [16, 32]), ("PLLM", 2, [16, 32]), ("PLLM", 2, [16, 16, 16]),
    ("KQVBIAS", 2, [16, 32])])
def test_graph_has_no_unordered_conflicts(pipeline_type, tp, nano):
    g, acc, keep = _host_graph(pipeline_type, tp, nano)
    assert len(g.ops) > 10
    for i, op in enumerate(g.ops):
        assert all(d < i for d in op.deps + op.after_start)
    bad = depcheck.check(g, acc)
    assert not bad, "unordered conflicting ops: " + ", ".join(f"{g.ops[a].name} <-> {g.ops[b].name}" for a, b in bad[:6])


def test_fused_reduce_scatter_ops_are_in_the_tp_graph():
    g, acc, keep = _host_graph("PLLM", 2, [16, 32], fuse_rs=True)
    assert not depcheck.check(g, acc)
    fused = [op for op in g.ops if op.kernel == "nfk_gemm_bf16" and op.params.epilogue == 2]
    reducers = [op for op in g.ops if op.kernel == "nfk_allreduce" and op.params.src_mode == 1]
    assert fused and len(fused) == len(reducers)
    # every layer but the last uses the fused form for both K-split GEMMs
    assert len(fused) == 2 * (2 * 2 - 1)
    for ge, ar in zip(fused, reducers):
        assert ge.params.rs_flag_off == ar.params.flag_off and ge.params.rs_slab_off == ar.params.buf_off
    # flags carry only the iteration's epoch, so no two collectives of one iteration may share a block
    offs = [op.params.flag_off for op in g.ops if op.kernel in ("nfk_allreduce", "nfk_allgather")]
    assert len(offs) == len(set(offs))


@pytest.mark.parametrize("nanos", [(0,), (0, 1)])
def test_all_gather_form_of_the_o_projection(nanos):
    """o_allgather_nanos: for those nano-batches the attention output is gathered column-wise by strided
    copies + a barrier, the O projection runs on the N-split weight into this rank's column block of the
    symmetric buffer, and the row owners gather the blocks (src_mode 2) with residual + norm as usual."""
    g, acc, (bufs, w, coll, _) = _host_graph("PLLM", 2, [16, 32], o_allgather=nanos)
    assert not depcheck.check(g, acc)
    m_layers = 2
    for k in (0, 1):
        o1 = [op for op in g.ops if op.name.endswith(f"nb{k}.o1")]
        o2 = [op for op in g.ops if op.name.endswith(f"nb{k}.o")]
        gath = [op for op in g.ops if op.name.endswith(f"nb{k}.ag_o")]
        if k in nanos:
            assert len(o1) == m_layers and not o2 and len(gath) == m_layers
            for op in o1:
                assert op.params.N == bufs.x[1].shape[1] // 2 and op.params.K == bufs.attn_full.shape[1]
                assert op.params.ldd == bufs.x[1].stride(0)       # a column block of the symmetric buffer
                assert op.params.A == bufs.attn_full.data_ptr() + (0 if k == 0 else 16) * bufs.attn_full.stride(0) * 2
            assert all(op.params.src_mode == 2 and op.params.norm_w for op in gath)
            copies = [op for op in g.ops if f"nb{k}.ag_attn.copy" in op.name]
            assert len(copies) == 2 * m_layers and all(op.kernel == "nfk_memcpy2d_p" for op in copies)
            assert all(op.params.width == bufs.attn_out.shape[1] * 2 for op in copies)
        else:
            assert len(o2) == m_layers and not o1 and not gath
    # dropping the barrier's edge into the GEMM must be seen: the GEMM reads what the peers' copies write
    o1_idx = next(i for i, op in enumerate(g.ops) if op.name.endswith("nb0.o1"))
    g.ops[o1_idx].deps = [d for d in g.ops[o1_idx].deps if not g.ops[d].name.endswith("ag_attn.done")]
    assert depcheck.check(g, acc)


def test_copy_engine_push_is_ordered_before_its_consumers():
    g, acc, _ = _host_graph("PLLM", 2, [16, 32], by_copy=True)
    assert any(".push" in op.name for op in g.ops)
    assert not depcheck.check(g, acc)


def test_checker_sees_a_missing_dependency():
    g, acc, keep = _host_graph("LOCAL", 1, [16, 32])
    # drop the dependencies of one attention op that runs on its own stream: the checker must object
    victim = next(i for i, op in enumerate(g.ops) if op.name.endswith("attn_decode") and op.stream == "attn")
    g.ops[victim].deps = []
    assert depcheck.check(g, acc)


@pytest.mark.parametrize("pipeline_type,tp,nano,beside", [
    ("NON_OVERLAP_LOCAL", 1, None, True), ("LOCAL", 1, [16, 32], True), ("NON_OVERLAP", 2, None, True),
    ("PLLM", 2, [16, 32], True)])
def test_prefill_attention_gets_its_own_stream(pipeline_type, tp, nano, beside):
    g, acc, keep = _host_graph(pipeline_type, tp, nano)
    pre = [i for i, op in enumerate(g.ops) if op.name.endswith("attn_prefill")]
    dec = [i for i, op in enumerate(g.ops) if op.name.endswith("attn_decode")]
    assert pre and len(pre) == len(dec)
    assert all((g.ops[i].stream == "attn2") == beside for i in pre)
    if beside:
        hb = g.happens_before()
        # the two attention kernels of a nano-batch are unordered, everything that reads their rows waits for both
        assert all(d not in hb[p] and p not in hb[d] for p, d in zip(pre, dec))
        g.ops[pre[1]].deps = []
        assert depcheck.check(g, acc)


# ---- the C++ executor, built against a logging stand-in for the CUDA runtime ------------------------
LAUNCH, RECORD, WAIT, BEGIN_CAPTURE, END_CAPTURE, INSTANTIATE, UPDATE, GRAPH_LAUNCH, EVENT_SYNC = range(9)


def _ancestors(log):
    """Happens-before implied by a log of runtime calls: program order per stream, and a wait on an
    event orders what follows it after that event's latest record at the time of the call. Returns one
    bit set per log entry (its ancestors, itself included)."""
    anc = [0] * len(log)
    last_on_stream, last_record = {}, {}
    for i, (kind, stream, event, op, captured, params) in enumerate(log):
        a = 1 << i
        if stream >= 0 and stream in last_on_stream:
            a |= anc[last_on_stream[stream]]
        if kind == WAIT and event in last_record:
            a |= anc[last_record[event]]
        anc[i] = a
        if stream >= 0:
            last_on_stream[stream] = i
        if kind == RECORD:
            last_record[event] = i
    return anc


def _host_executor(pipeline_type, tp, nano, graph_mode=False):
    from nanoflow_b200.runtime.native import NativeExecutor

    g, acc, keep = _host_graph(pipeline_type, tp, nano)
    single = all(op.stream == "gemm" for op in g.ops)
    ex = NativeExecutor(g, None, single_stream=single, use_cuda_graph=graph_mode, host_only=True)
    ex.mod.host_log_clear()
    return g, ex, keep


def _symbols(g, it):
    return {name: 3 + it + 2 * idx for name, idx in g.symbols.items()}


@pytest.mark.parametrize("pipeline_type,tp,nano", [("NON_OVERLAP_LOCAL", 1, None), ("LOCAL", 1, [16, 32]),
                                                   ("PLLM", 2, [16, 32]), ("NON_OVERLAP", 2, None)])
def test_executor_event_wiring_enforces_the_graph(pipeline_type, tp, nano):
    g, ex, keep = _host_executor(pipeline_type, tp, nano)
    n = len(g.ops)
    for it in range(2):
        ex.wait(ex.submit(_symbols(g, it)))
    log = ex.mod.host_log()
    ex.close()
    launches = [i for i, r in enumerate(log) if r[0] == LAUNCH]
    assert [log[i][3] for i in launches] == list(range(n)) * 2          # issue order = graph order, twice
    assert not any(r[4] for r in log)                                    # nothing captured in plain mode
    anc = _ancestors(log)
    first, second = launches[:n], launches[n:]
    for it_launches in (first, second):
        for j, op in enumerate(g.ops):
            for d in op.deps:
                assert anc[it_launches[j]] >> it_launches[d] & 1, f"{g.ops[d].name} -> {op.name} is not enforced"
    # every launch of an iteration precedes the event the host waits on, and the next iteration's launches
    syncs = [r[2] for r in log if r[0] == EVENT_SYNC]
    done = [max(i for i, r in enumerate(log) if r[0] == RECORD and r[2] == ev and r[1] == 0 and i < (launches[n] if k == 0 else len(log)))
            for k, ev in enumerate(syncs)]
    assert all(anc[done[0]] >> i & 1 for i in first) and all(anc[done[1]] >> i & 1 for i in second)
    assert all(anc[second[0]] >> i & 1 for i in first)
    # streams: ops run where the graph put them (one stream per class, the main stream when there is only one)
    by_class = {}
    for i in first:
        by_class.setdefault(g.ops[log[i][3]].stream, set()).add(log[i][1])
    assert all(len(s) == 1 for s in by_class.values())
    assert len({next(iter(s)) for s in by_class.values()}) == len(by_class)


def test_executor_patches_symbols_into_parameter_blocks():
    g, ex, keep = _host_executor("LOCAL", 1, [16, 32])
    syms = _symbols(g, 0)
    ex.wait(ex.submit(syms))
    log = [r for r in ex.mod.host_log() if r[0] == LAUNCH]
    ex.close()
    checked = 0
    for r, op in zip(log, g.ops):
        blob = r[5]
        assert len(blob) == len(bytes(op.params))
        want = bytearray(bytes(op.params))
        for field, sym in op.dyn:
            desc = getattr(type(op.params), field)
            want[desc.offset:desc.offset + desc.size] = int(syms[sym]).to_bytes(desc.size, "little", signed=True)
            checked += 1
        assert blob == bytes(want), op.name
    assert checked > len(g.ops) // 2


@pytest.mark.parametrize("pipeline_type,tp,nano", [("NON_OVERLAP_LOCAL", 1, None), ("LOCAL", 1, [16, 32])])
def test_executor_graph_mode_captures_whole_iterations(pipeline_type, tp, nano):
    g, ex, keep = _host_executor(pipeline_type, tp, nano, graph_mode=True)
    n = len(g.ops)
    for it in range(5):
        if it == 4:
            ex.mod.fail_next_graph_update()          # the runtime refuses the in-place update once
        ex.wait(ex.submit(_symbols(g, it)))
    assert ex.graph_stats == (3, 2)                  # two plain iterations first; built, updated, rebuilt
    log = ex.mod.host_log()
    ex.close()
    anc = _ancestors(log)
    begins = [i for i, r in enumerate(log) if r[0] == BEGIN_CAPTURE]
    ends = [i for i, r in enumerate(log) if r[0] == END_CAPTURE]
    assert len(begins) == len(ends) == 3
    plain = [i for i, r in enumerate(log) if r[0] == LAUNCH and i < begins[0]]
    assert len(plain) == 2 * n and not any(log[i][4] for i in plain)
    for b, e in zip(begins, ends):
        inside = [i for i in range(b + 1, e) if log[i][0] == LAUNCH]
        assert [log[i][3] for i in inside] == list(range(n))
        assert all(log[i][4] for i in inside), "a launch escaped the capture and ran eagerly"
        # every stream that joined the capture is joined back into the origin before the capture ends
        touched = [i for i in range(b + 1, e) if log[i][4]]
        assert all(anc[e] >> i & 1 for i in touched), "unjoined work at cudaStreamEndCapture"
        for j, op in enumerate(g.ops):
            for d in op.deps:
                assert anc[inside[j]] >> inside[d] & 1
        # the captured iteration is launched on the main stream as one unit, before the host's event
        after = log[e + 1:e + 6]
        kinds = [r[0] for r in after]
        assert GRAPH_LAUNCH in kinds and RECORD in kinds[kinds.index(GRAPH_LAUNCH):]
        assert after[kinds.index(GRAPH_LAUNCH)][1] == 0
    assert [r[0] for r in log if r[0] in (INSTANTIATE, UPDATE)] == [INSTANTIATE, UPDATE, UPDATE, INSTANTIATE]


def test_executor_reports_a_rejected_op_and_bounds_iterations_in_flight():
    from nanoflow_b200.runtime.native import load_host_module

    mod = load_host_module()
    ex = mod.Executor(0, 0, False, 1)
    ex.add_op("a", mod.noop_fn(), bytes(8), 0, [], [], [(0, 0, 4)])
    ex.add_op("b", mod.failing_fn(), bytes(8), 1, [0], [], [])
    with pytest.raises(RuntimeError, match="earlier op"):
        ex.add_op("c", mod.noop_fn(), bytes(8), 0, [5], [], [])
    with pytest.raises(RuntimeError, match="bad patch"):
        ex.add_op("c", mod.noop_fn(), bytes(8), 0, [], [], [(6, 0, 4)])
    t = ex.submit([7])
    with pytest.raises(RuntimeError, match="op b rejected its arguments .code 3."):
        ex.wait(t)
    ex.close()
    ok = mod.Executor(0, 0, True, 0)
    ok.add_op("a", mod.noop_fn(), bytes(8), 0, [], [], [])
    tickets = [ok.submit([]) for _ in range(8)]
    with pytest.raises(RuntimeError, match="too many iterations in flight"):
        ok.submit([])
    for t in tickets:
        ok.wait(t)
    ok.wait(ok.submit([]))
    assert ok.launches() == 9
    ok.close()


def test_executor_threads_are_race_free_under_thread_sanitizer():
    """The worker thread, the submitting thread and the waiting thread share the job queue, the ticket
    counters and the error string: 200 iterations with six in flight under ThreadSanitizer."""
    import os
    import subprocess
    import sys

    from nanoflow_b200.ops import build

    res = subprocess.run(["gcc", "-print-file-name=libtsan.so"], capture_output=True, text=True)
    tsan = res.stdout.strip()
    if res.returncode != 0 or not os.path.isabs(tsan) or not os.path.exists(tsan):
        pytest.skip("no ThreadSanitizer runtime on this machine")
    mod = build.build_executor_host(sanitize="thread")
    env = dict(os.environ, LD_PRELOAD=tsan, TSAN_OPTIONS="report_signal_unsafe=0 exitcode=66")
    script = os.path.join(os.path.dirname(__file__), "executor_host_stress.py")
    run = subprocess.run([sys.executable, script, str(mod.parent)], capture_output=True, text=True, env=env,
                         timeout=600)
    assert "ThreadSanitizer" not in run.stderr, run.stderr[-3000:]
    assert run.returncode == 0, run.stderr[-3000:]
    assert "launches 8000 graph launches 194 rebuilds 1" in run.stdout


@pytest.mark.parametrize("nano,fuse_rs", [([16, 32], False), ([16, 16, 16], False), ([16, 32], True)])
def test_second_network_stream_keeps_the_graph_ordered(nano, fuse_rs):
    """net_streams = 2: the all-reduces of odd nano-batches run on their own stream, unordered with the
    even ones; every buffer hazard is still covered by an explicit dependency, and the executor's event
    wiring enforces all of them."""
    from nanoflow_b200.runtime.native import NativeExecutor

    g, acc, keep = _host_graph("PLLM", 2, nano, fuse_rs=fuse_rs, net_streams=2)
    ars = [(i, op) for i, op in enumerate(g.ops) if op.kernel == "nfk_allreduce"]
    assert {op.stream for _, op in ars} == {"net", "net2"}
    assert all((op.stream == "net2") == (op.nano % 2 == 1) for _, op in ars)
    assert not depcheck.check(g, acc)
    hb = g.happens_before()
    first_layer = [i for i, op in ars if op.layer == 0 and op.name.endswith("ar_o")]
    assert first_layer[0] not in hb[first_layer[1]] and first_layer[1] not in hb[first_layer[0]]
    ex = NativeExecutor(g, None, single_stream=False, host_only=True)
    ex.mod.host_log_clear()
    ex.wait(ex.submit(_symbols(g, 0)))
    log = ex.mod.host_log()
    ex.close()
    anc = _ancestors(log)
    launches = [i for i, r in enumerate(log) if r[0] == LAUNCH]
    for j, op in enumerate(g.ops):
        for d in op.deps:
            assert anc[launches[j]] >> launches[d] & 1


def test_sleep_ops_stand_in_for_the_wire_time_of_absent_ranks():
    """fake_wire_us_per_row: every all-reduce is followed on its stream by a sleep op whose length is a
    symbol (rows of the nano-batch x the factor, set per iteration), and whatever waited for the
    all-reduce now waits for the sleep."""
    import ctypes

    from nanoflow_b200.runtime.graph import SleepParams
    from nanoflow_b200.runtime.native import NativeExecutor

    g, acc, keep = _host_graph("PLLM", 2, [16, 32], fake_wire=0.11)
    plain, _, keep2 = _host_graph("PLLM", 2, [16, 32])
    ars = [i for i, op in enumerate(g.ops) if op.kernel == "nfk_allreduce"]
    wires = [i for i, op in enumerate(g.ops) if op.kernel == "nfk_sleep_p"]
    assert len(wires) == len(ars) == len([op for op in plain.ops if op.kernel == "nfk_allreduce"])
    assert len(g.ops) == len(plain.ops) + len(wires) and {"nb0_wire_us", "nb1_wire_us"} <= set(g.symbols)
    for a, w in zip(ars, wires):
        assert w == a + 1 and g.ops[w].deps == [a] and g.ops[w].stream == g.ops[a].stream
        assert g.ops[w].name == g.ops[a].name + ".wire" and isinstance(g.ops[w].params, SleepParams)
        users = [op for op in g.ops if a in op.deps]
        assert users == [g.ops[w]]                       # nothing else waits for the bare all-reduce
    assert not depcheck.check(g, acc)
    ex = NativeExecutor(g, None, single_stream=False, host_only=True)
    ex.mod.host_log_clear()
    syms = _symbols(g, 0)
    syms["nb0_wire_us"], syms["nb1_wire_us"] = 123, 456
    ex.wait(ex.submit(syms))
    launches = [r for r in ex.mod.host_log() if r[0] == LAUNCH]
    ex.close()
    for w in wires:
        micros = ctypes.c_int.from_buffer_copy(launches[w][5][:4]).value
        assert micros == (123 if g.ops[w].nano == 0 else 456)


@pytest.mark.parametrize("nano", [[16, 32], [16, 16, 16], [16, 16, 16, 16]])
def test_decode_attention_on_its_own_stream_under_tensor_parallelism(nano):
    """attn_overlap: decode attention leaves the compute stream, all front-ends of a layer are issued
    before the first O projection, GEMMs keep to the shared-memory budget that leaves room for an
    attention CTA, and every buffer hazard (KV pool slices per nano-batch included) stays ordered."""
    from nanoflow_b200.runtime.native import NativeExecutor
    from nanoflow_b200.runtime.pipeline import GEMM_SMEM_KB_BESIDE_ATTENTION

    g, acc, keep = _host_graph("PLLM", 2, nano, gbs=sum(nano), attn_overlap=True)
    assert not depcheck.check(g, acc)
    names = [op.name for op in g.ops]
    dec = [i for i, op in enumerate(g.ops) if op.kernel == "nfk_attn_decode"]
    assert dec and all(g.ops[i].stream == "attn" and g.ops[i].params.num_ctas == 148 for i in dec)
    assert all(g.ops[i].params.decode_stages == 2 for i in dec)     # 64 KB per CTA: a collective's CTA still fits
    gemms = [op for op in g.ops if op.kernel == "nfk_gemm_bf16" and op.layer >= 0]
    assert all(op.params.smem_budget_kb == GEMM_SMEM_KB_BESIDE_ATTENTION for op in gemms)
    last_front = max(names.index(f"L0.nb{k}.rope_append") for k in range(len(nano)))
    assert all(names.index(f"L0.nb{k}.o") > last_front for k in range(len(nano)))
    hb = g.happens_before()
    # the decode kernel of nano-batch 0 is unordered with the QKV GEMM and the KV append of nano-batch 1 ...
    d0, q1, r1 = names.index("L0.nb0.attn_decode"), names.index("L0.nb1.qkv"), names.index("L0.nb1.rope_append")
    assert d0 not in hb[q1] and q1 not in hb[d0] and d0 not in hb[r1] and r1 not in hb[d0]
    # ... but a KV append is ordered with every attention that may read the pages it writes
    p1 = names.index("L0.nb1.attn_prefill")
    assert names.index("L0.nb0.rope_append") in hb[p1] and r1 in hb[p1]
    plain, acc_plain, keep2 = _host_graph("PLLM", 2, nano, gbs=sum(nano))
    assert all(op.stream != "attn" for op in plain.ops) and not depcheck.check(plain, acc_plain)
    assert all(op.params.decode_stages == 0 for op in plain.ops if op.kernel == "nfk_attn_decode")
    ex = NativeExecutor(g, None, single_stream=False, host_only=True)
    ex.mod.host_log_clear()
    ex.wait(ex.submit(_symbols(g, 0)))
    log = ex.mod.host_log()
    ex.close()
    anc = _ancestors(log)
    launches = [i for i, r in enumerate(log) if r[0] == LAUNCH]
    for j, op in enumerate(g.ops):
        for d in op.deps:
            assert anc[launches[j]] >> launches[d] & 1


@pytest.mark.parametrize("pipeline_type,tp,nano,attn_overlap", [("LOCAL", 1, [16, 32], False), ("LOCAL", 1, [16, 16, 16], False),
                                                                 ("PLLM", 2, [16, 32], True), ("PLLM", 2, [16, 16, 16], True)])
def test_cross_layer_software_pipeline_order(pipeline_type, tp, nano, attn_overlap):
    """cross_layer_pipeline: a nano-batch's QKV / RoPE of layer l+1 follows its FFN of layer l on the compute
    stream, ahead of the next nano-batch's O projection of layer l, so its attention (own stream) is unordered
    with those GEMMs; all buffer hazards stay ordered and the executor wires every dependency."""
    from nanoflow_b200.runtime.native import NativeExecutor

    g, acc, keep = _host_graph(pipeline_type, tp, nano, gbs=sum(nano), attn_overlap=attn_overlap, cross_layer=True)
    assert not depcheck.check(g, acc)
    names = [op.name for op in g.ops]
    for i, op in enumerate(g.ops):
        assert all(d < i for d in op.deps + op.after_start)
    hb = g.happens_before()
    if tp == 1:
        assert names.index("L0.nb0.down") < names.index("L1.nb0.qkv") < names.index("L0.nb1.o")
        a1, o1, gu1 = names.index("L1.nb0.attn_decode"), names.index("L0.nb1.o"), names.index("L0.nb1.gate_up")
    else:
        ix = names.index
        if len(nano) == 2:
            # nano-batch 1 runs a phase behind nano-batch 0:
            #   o(1,p-1) F(0,p) gate_up(1,p-1) o(0,p) down(1,p-1) gate_up(0,p) F(1,p) down(0,p)
            assert ix("L0.nb0.gate_up") < ix("L0.nb1.qkv") < ix("L0.nb0.down") < ix("L0.nb1.o") < ix("L1.nb0.qkv") \
                < ix("L0.nb1.gate_up") < ix("L1.nb0.o") < ix("L0.nb1.down") < ix("L1.nb0.gate_up") < ix("L1.nb1.qkv")
            a1, o1, gu1 = ix("L1.nb0.attn_decode"), ix("L0.nb1.gate_up"), ix("L0.nb1.gate_up")
        else:
            # O of nano-batch k, front-end of the nano-batch whose O projection comes next, FFN of k
            assert ix("L0.nb0.o") < ix("L0.nb1.qkv") < ix("L0.nb0.gate_up") < ix("L0.nb1.o")
            last = len(nano) - 1
            assert ix(f"L0.nb{last}.o") < ix("L1.nb0.qkv") < ix(f"L0.nb{last}.gate_up")
            a1, o1, gu1 = ix("L0.nb1.attn_decode"), ix("L0.nb0.down"), ix("L0.nb0.gate_up")
        assert all(op.stream == "gemm" for op in g.ops if op.kernel.startswith("nfk_attn_prefill"))
    assert g.ops[a1].stream == "attn"
    assert a1 not in hb[o1] and o1 not in hb[a1] and a1 not in hb[gu1] and gu1 not in hb[a1]
    # same ops as the per-layer order, only issued differently
    plain, _, keep2 = _host_graph(pipeline_type, tp, nano, gbs=sum(nano), attn_overlap=attn_overlap)
    assert sorted(names) == sorted(op.name for op in plain.ops)
    ex = NativeExecutor(g, None, single_stream=False, host_only=True)
    ex.mod.host_log_clear()
    ex.wait(ex.submit(_symbols(g, 0)))
    log = ex.mod.host_log()
    ex.close()
    anc = _ancestors(log)
    launches = [i for i, r in enumerate(log) if r[0] == LAUNCH]
    for j, op in enumerate(g.ops):
        for d in op.deps:
            assert anc[launches[j]] >> launches[d] & 1


def test_checker_still_sees_a_missing_append_dependency():
    g, acc, keep = _host_graph("PLLM", 2, [16, 32], attn_overlap=True)
    victim = next(i for i, op in enumerate(g.ops) if op.name == "L1.nb0.attn_decode")
    g.ops[victim].deps = []          # the decode kernel no longer waits for its own nano-batch's KV append
    assert depcheck.check(g, acc)


def test_collectives_beside_other_kernels_get_a_cta_budget_by_form_and_rank_count():
    from nanoflow_b200.runtime.pipeline import default_comm_ctas

    assert default_comm_ctas(8, True) == 32 and default_comm_ctas(4, True) == 64     # ~16 owned rows per CTA
    assert default_comm_ctas(2, True) == 96 and default_comm_ctas(8, False) == 96
    g, acc, keep = _host_graph("PLLM", 2, [16, 32])            # peer-load form (the analysis heap has no multicast mapping)
    ars = [op for op in g.ops if op.kernel == "nfk_allreduce" and op.layer >= 0]
    assert ars and all(op.params.num_ctas == 96 for op in ars)
    g1, _, keep1 = _host_graph("NON_OVERLAP", 2, None)         # nothing runs beside: the collective's own default (all SMs)
    coll = keep1[2]
    assert all(op.params.num_ctas == coll.num_ctas for op in g1.ops if op.kernel == "nfk_allreduce" and op.layer >= 0)
