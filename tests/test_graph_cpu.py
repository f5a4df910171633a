"""Static checks of the op graph on CPU: every pipeline variant builds, dependencies only point
backwards, and no two ops that touch the same bytes (one of them writing) are left unordered."""
import pytest
import torch

from nanoflow_b200.config import builtin_config
from nanoflow_b200.models import random_full_weights, shard_weights
from nanoflow_b200.parallel.collectives import TpCollectives
from nanoflow_b200.runtime.pipeline import Buffers, IoSpec, build_graph
from nanoflow_b200.utils import depcheck


def _host_graph(pipeline_type, tp, nano, gbs=48, fuse_rs=False):
    cfg = builtin_config("tiny", gpu_num=tp, global_batch_size=gbs, pipeline_type=pipeline_type, nanobatch_sizes=nano)
    m, e = cfg.model, cfg.engine
    e.fuse_gemm_rs = fuse_rs
    e.max_batch_size = gbs
    fw = random_full_weights(m, seed=0)
    w = shard_weights(fw, m, 0, tp, dtype=torch.bfloat16)
    coll = TpCollectives.for_analysis(0, tp) if tp > 1 else None
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
                   gemm_ws=torch.zeros(1 << 16))
    io = IoSpec(meta_dev, 4 * T, 8 * T)
    g = build_graph(m, e, w, bufs, coll, io)
    starts = [sum(sizes[:k]) for k in range(len(sizes))]
    pool_bytes = pools[0].numel() * 2
    acc = depcheck.graph_access(g, starts, sizes, heap_base=coll.heap.base if coll else 0, kv_pool_bytes=pool_bytes)
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
