"""End-to-end GPU engine against the fp32 oracle on the tiny Llama config (2 layers, hidden 256,
4 q / 2 kv heads of 64, SwiGLU 688, vocab 1024): 4 prompts x 32 tokens, 16 greedy tokens each."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from nanoflow_b200.config import builtin_config
from nanoflow_b200.models import ReferenceLlama, random_full_weights, shard_weights
from nanoflow_b200.serving import DistKVPool, RequestManager, Scheduler
from nanoflow_b200.serving.loop import ServingLoop


def _run(pipeline_type, nano, executor, gbs=48, guards=False, tail=0.0, cross_layer=False):
    from nanoflow_b200.runtime.engine import Engine

    cfg = builtin_config("tiny", gpu_num=1, global_batch_size=gbs, pipeline_type=pipeline_type,
                         nanobatch_sizes=nano)
    cfg.engine.max_batch_size = gbs
    cfg.engine.debug_guards = guards
    cfg.engine.cross_layer_pipeline = cross_layer
    fw = random_full_weights(cfg.model, seed=0, std=0.05)
    # the oracle sees the same bf16-rounded weights; only activation rounding differs
    for lay in fw.layers:
        for k, v in vars(lay).items():
            if v is not None:
                setattr(lay, k, v.bfloat16().float())
    fw.embed, fw.norm, fw.lm_head = fw.embed.bfloat16().float(), fw.norm.bfloat16().float(), fw.lm_head.bfloat16().float()
    oracle = ReferenceLlama(cfg.model, fw)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 1024, size=32, dtype=np.int32) for _ in range(4)]
    rm = RequestManager(vocab_size=1024)
    for p in prompts:
        rm.add_request(32, 16, 0.0, prompt=p)
    rm.finalize_stats()
    pool = DistKVPool(2, 2, 64, 64, 16, 1)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                    nanobatch_sizes=cfg.engine.resolved_nanobatches(), average_prefill_length=32,
                    average_decode_length=16, group_size=2, decode_tail_fraction=tail)
    eng = Engine(cfg, shard_weights(fw, cfg.model, 0, 1, device="cuda"), num_pages=64, executor=executor)
    loop = ServingLoop(eng, sch, rm, est_cycle_time=1.0)
    st = loop.run()
    eng.check_status()
    if guards:
        # every activation buffer is fenced and no kernel wrote outside its rows and columns; a byte
        # changed from the host behind one of them is reported with the buffer's name
        assert len(eng.guards) >= 9 and not eng.guards.check()
        raw = eng.bufs.attn_out.view(torch.uint8).view(-1)
        torch.as_strided(raw, (1,), (1,), raw.storage_offset() + raw.numel() + 3).fill_(0)
        with pytest.raises(RuntimeError, match="attn_out .rear guard, byte 3"):
            eng.check_status()
        eng.check_status()       # guards were restored
    eng.finalize()
    assert len(st.retired) == 4
    exact = 0
    for r in st.retired:
        assert len(r.output) == 16
        prompt = prompts[r.req_idx].tolist()
        want = oracle.generate(prompt, 16)
        exact += int(want == r.output)
        # greedy consistency under teacher forcing: the engine's token is (near-)arg-max for the oracle
        seq = torch.tensor(prompt + r.output[:-1])
        logits, _ = oracle.forward(seq)
        steps = logits[len(prompt) - 1:]
        chosen = steps[torch.arange(16), torch.tensor(r.output)]
        gap = steps.max(dim=-1).values - chosen
        assert gap.max().item() < 0.05 * steps.abs().max().item(), f"engine token far from oracle arg-max: {gap}"
    return exact


@pytest.mark.parametrize("pipeline_type,nano", [("NON_OVERLAP_LOCAL", None), ("NANOBATCH_LOCAL", [16, 32]),
                                                ("LOCAL", [16, 32])])
def test_engine_matches_oracle_py_executor(pipeline_type, nano):
    _run(pipeline_type, nano, "python")   # asserts greedy consistency with the oracle


def test_engine_keeps_inside_guarded_buffers():
    _run("LOCAL", [16, 32], "native", guards=True)


def test_engine_with_decode_requests_at_both_ends_of_the_batch():
    """Part of the decode requests scheduled behind the prompt chunks, into the last nano-batch: the
    decode kernel of that nano-batch starts at a request index past the prompts."""
    _run("LOCAL", [16, 32], "native", tail=0.5)


@pytest.mark.parametrize("nano,tail,executor", [([16, 32], 0.0, "native"), ([16, 16, 16], 0.5, "native"), ([24, 24], 0.5, "graph")])
def test_engine_cross_layer_software_pipeline(nano, tail, executor):
    """QKV / RoPE of layer l+1 issued behind the same nano-batch's FFN of layer l (attention under the other
    nano-batches' GEMMs): same tokens as the oracle."""
    _run("LOCAL", nano, executor, cross_layer=True, tail=tail)


def test_engine_matches_oracle_native_executor():
    _run("LOCAL", [16, 32], "native")


@pytest.mark.parametrize("pipeline_type,nano", [("NON_OVERLAP_LOCAL", None), ("LOCAL", [16, 32])])
def test_engine_cuda_graph_executor(pipeline_type, nano):
    """Iterations captured and launched as CUDA graphs (single stream and forked streams): the token
    counts change from iteration to iteration, so every launch goes through the in-place update."""
    _run(pipeline_type, nano, "graph")


@pytest.mark.parametrize("o1", [False, True])
def test_virtual_tensor_parallel_rank_runs_alone(o1):
    """One GPU runs rank 0's share of a two-way tensor-parallel job with the collectives reduced to
    their local part (the reference's vnranks aid): shapes, nano-batch overlap and the fused
    all-reduce + norm path are exercised without a second GPU; tokens are not meaningful.
    ``o1``: the first nano-batch's O projection in its all-gather form (strided copies, N-split weight,
    column-block gather)."""
    from nanoflow_b200.parallel.collectives import TpCollectives
    from nanoflow_b200.runtime.engine import Engine

    gbs = 48
    cfg = builtin_config("tiny", gpu_num=2, global_batch_size=gbs, pipeline_type="PLLM", nanobatch_sizes=[16, 32])
    cfg.engine.max_batch_size = gbs
    cfg.engine.o_allgather_nanos = [0] if o1 else []
    fw = random_full_weights(cfg.model, seed=0, std=0.05)
    coll = TpCollectives(0, 1, torch.device("cuda", 0), heap_bytes=64 << 20)
    eng = Engine(cfg, shard_weights(fw, cfg.model, 0, 2, device="cuda", o1=o1), collectives=coll, num_pages=64)
    assert any(op.name.endswith(".o1") for op in eng.graph.ops) == o1
    rm = RequestManager(vocab_size=1024, random_ids=True)
    for _ in range(4):
        rm.add_request(32, 8, 0.0)
    rm.finalize_stats()
    pool = DistKVPool(2, 2, 64, 64, 16, 2)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                    nanobatch_sizes=cfg.engine.resolved_nanobatches(), average_prefill_length=32,
                    average_decode_length=8, group_size=2)
    st = ServingLoop(eng, sch, rm, est_cycle_time=1.0).run()
    eng.check_status()
    eng.finalize()
    assert len(st.retired) == 4 and all(len(r.output) == 8 for r in st.retired)
    assert all(0 <= t < 1024 for r in st.retired for t in r.output)


def test_gated_gemms_behind_the_all_reduce_give_the_same_tokens():
    """gate_gemm: QKV and gate/up start together with the all-reduce + norm that delivers their input rows
    and wait per 128-row block. One GPU runs rank 0's share of a two-way job (collectives reduced to their
    local part, as above): the flag protocol between the collective and the GEMM runs for real, and the
    sampled tokens equal those of the ungated pipeline."""
    from nanoflow_b200.parallel.collectives import TpCollectives
    from nanoflow_b200.runtime.engine import Engine

    def serve(gate, ptype, nano):
        gbs = 384
        cfg = builtin_config("tiny", gpu_num=2, global_batch_size=gbs, pipeline_type=ptype, nanobatch_sizes=nano)
        cfg.engine.max_batch_size = gbs
        cfg.engine.gate_gemm = gate
        fw = random_full_weights(cfg.model, seed=0, std=0.05)
        coll = TpCollectives(0, 1, torch.device("cuda", 0), heap_bytes=64 << 20)
        eng = Engine(cfg, shard_weights(fw, cfg.model, 0, 2, device="cuda"), collectives=coll, num_pages=256)
        gated = [op for op in eng.graph.ops if op.gated]
        assert bool(gated) == gate
        rm = RequestManager(vocab_size=1024, random_ids=True, seed=3)
        for _ in range(6):
            rm.add_request(150, 6, 0.0)
        rm.finalize_stats()
        pool = DistKVPool(2, 2, 64, 256, 16, 2)
        sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                        nanobatch_sizes=cfg.engine.resolved_nanobatches(), average_prefill_length=150,
                        average_decode_length=6, group_size=2)
        st = ServingLoop(eng, sch, rm, est_cycle_time=1.0).run()
        eng.check_status()
        coll.check_status()
        eng.finalize()
        assert len(st.retired) == 6
        return {r.req_idx: list(r.output) for r in st.retired}

    for ptype, nano in (("NON_OVERLAP", None), ("PLLM", [128, 256])):
        assert serve(True, ptype, nano) == serve(False, ptype, nano)


def test_kv_offload_and_restore():
    """PLLM_OFFLOAD: pages of retired requests reach pinned host memory layer by layer, match the
    oracle's rotated K / V, and can be scattered back into fresh pages."""
    from nanoflow_b200.runtime.engine import Engine
    from nanoflow_b200.serving.kv_cache import DistKVCache
    from nanoflow_b200.serving.offload import KVOffloadManager

    gbs = 48
    cfg = builtin_config("tiny", gpu_num=1, global_batch_size=gbs, pipeline_type="PLLM_OFFLOAD",
                         nanobatch_sizes=[16, 32])
    cfg.engine.max_batch_size = gbs
    assert cfg.engine.offload
    fw = random_full_weights(cfg.model, seed=0, std=0.05)
    for lay in fw.layers:
        for k, v in vars(lay).items():
            if v is not None:
                setattr(lay, k, v.bfloat16().float())
    fw.embed, fw.norm, fw.lm_head = fw.embed.bfloat16().float(), fw.norm.bfloat16().float(), fw.lm_head.bfloat16().float()
    oracle = ReferenceLlama(cfg.model, fw)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 1024, size=n, dtype=np.int32) for n in (20, 33, 7)]
    rm = RequestManager(vocab_size=1024)
    for p in prompts:
        rm.add_request(len(p), 6, 0.0, prompt=p)
    rm.finalize_stats()
    pool = DistKVPool(2, 2, 64, 64, 16, 1)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs, nanobatch_sizes=[16, 32],
                    average_prefill_length=20, average_decode_length=6, group_size=2, hold_retired_pages=True)
    eng = Engine(cfg, shard_weights(fw, cfg.model, 0, 1, device="cuda"), num_pages=64, executor="native")
    off = KVOffloadManager(eng)
    loop = ServingLoop(eng, sch, rm, est_cycle_time=1.0, offload=off)
    st = loop.run()
    # a few idle cycles so the last retired requests ride on an iteration... they retire only when
    # another iteration runs; with an empty queue nothing runs, so only earlier retirees are stored
    eng.check_status()
    assert len(st.retired) == 3
    assert pool.num_free_pages + sum(r.kv_cache.num_pages for _, r in sch._held_pages) == 64
    stored = [r for r in st.retired if r.req_idx in off.store]
    assert stored, "no request was offloaded"
    for r in stored:
        kvs = off.store[r.req_idx]
        seq = prompts[r.req_idx].tolist() + r.output
        n_kv = kvs.seqlen
        _, caches = oracle.forward(torch.tensor(seq[:n_kv]))
        for l in range(2):
            pages = kvs.data[l].view(-1, 2, 2, 16, 64).float()          # [n_pages, K/V, kv_heads, 16, hd]
            k = pages[:, 0].permute(0, 2, 1, 3).reshape(-1, 2, 64)[:n_kv]
            v = pages[:, 1].permute(0, 2, 1, 3).reshape(-1, 2, 64)[:n_kv]
            assert torch.allclose(k, caches[l]["k"], atol=6e-2, rtol=5e-2)
            assert torch.allclose(v, caches[l]["v"], atol=6e-2, rtol=5e-2)
        # restore into fresh pages and compare with the host copy
        kv = DistKVCache(pool)
        kv.allocate_tokens(n_kv)
        off.restore(r.req_idx, kv)
        torch.cuda.synchronize()
        ids = torch.from_numpy(np.ascontiguousarray(kv.indicies)).long().cuda()
        for l in range(2):
            assert torch.equal(eng.bufs.kv_pool[l][ids].reshape(len(ids), -1).cpu(), kvs.data[l])
        kv.release()
    eng.finalize()
