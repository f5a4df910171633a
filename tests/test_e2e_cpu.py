"""End-to-end on CPU: trace -> scheduler (async control flow, chunked prefill, nano-batches) ->
CPU backend with tensor-parallel shards, compared token by token with the fp32 oracle.

Config under test: the tiny Llama decoder (2 layers, hidden 256, 4 q / 2 kv heads of 64, SwiGLU 688,
vocab 1024, eps 1e-5, theta 10000), weights N(0, 0.02) seed 0, 4 prompts x 32 uniform token ids
(seed 0), greedy, 16 new tokens."""
import numpy as np
import pytest
import torch

from nanoflow_b200.config import builtin_config
from nanoflow_b200.models import ReferenceLlama, random_full_weights, shard_weights
from nanoflow_b200.runtime.cpu_backend import CpuEngine
from nanoflow_b200.serving import DistKVPool, RequestManager, Scheduler
from nanoflow_b200.serving.loop import ServingLoop


def _serve(tp, gbs, nano, prompts, out_len, pages=64, model="tiny", **sched_kw):
    cfg = builtin_config(model, gpu_num=tp, global_batch_size=gbs, pipeline_type="PLLM" if nano else "NON_OVERLAP",
                         **({"nanobatch_sizes": nano} if nano else {}))
    cfg.engine.max_batch_size = gbs
    fw = random_full_weights(cfg.model, seed=0)
    oracle = ReferenceLlama(builtin_config(model).model, fw)
    rm = RequestManager(vocab_size=cfg.model.vocab_size)
    for p in prompts:
        rm.add_request(len(p), out_len, 0.0, prompt=p)
    rm.finalize_stats()
    pool = DistKVPool(cfg.model.run_layers, cfg.model.num_kv_heads, cfg.model.head_dim, pages, 16, tp)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=gbs,
                    nanobatch_sizes=cfg.engine.resolved_nanobatches(), average_prefill_length=rm.average_prefill_length,
                    average_decode_length=out_len, group_size=cfg.model.group_size, **sched_kw)
    eng = CpuEngine(cfg, [shard_weights(fw, cfg.model, r, tp, dtype=torch.float32) for r in range(tp)], num_pages=pages)
    st = ServingLoop(eng, sch, rm, est_cycle_time=1.0).run()
    return st, oracle, pool


def test_greedy_decode_matches_oracle_with_decode_requests_at_both_ends_of_the_batch():
    """``decode_tail_fraction``: part of the decode requests sit after the prompt chunks (in the last
    nano-batch); outputs are the oracle's, token for token."""
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 1024, size=int(n), dtype=np.int32) for n in (32, 9, 21, 40, 17, 33)]
    st, oracle, pool = _serve(2, 48, [16, 32], prompts, 12, decode_tail_fraction=0.5)
    assert len(st.retired) == 6 and pool.num_free_pages == 64
    for r in st.retired:
        assert r.output == oracle.generate(prompts[r.req_idx].tolist(), 12)


@pytest.mark.parametrize("tp,gbs,nano", [(1, 48, None), (1, 48, [16, 32]), (2, 48, [16, 32]), (2, 160, [64, 96])])
def test_greedy_decode_matches_oracle(tp, gbs, nano):
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 1024, size=32, dtype=np.int32) for _ in range(4)]
    st, oracle, pool = _serve(tp, gbs, nano, prompts, 16)
    assert len(st.retired) == 4 and pool.num_free_pages == 64
    for r in st.retired:
        assert r.output == oracle.generate(prompts[r.req_idx].tolist(), 16)


def test_ragged_prompts_tiny_batch_and_single_token_requests():
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 1024, size=n, dtype=np.int32) for n in (1, 2, 17, 16, 40, 3)]
    st, oracle, pool = _serve(1, 24, [8, 16], prompts, 5)
    assert len(st.retired) == 6
    for r in st.retired:
        assert r.output == oracle.generate(prompts[r.req_idx].tolist(), 5)


def test_eos_stops_generation_like_the_oracle():
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 1024, size=12, dtype=np.int32) for _ in range(3)]
    # pick as "EOS" the token the oracle emits third for request 0
    cfg = builtin_config("tiny")
    oracle = ReferenceLlama(cfg.model, random_full_weights(cfg.model, seed=0))
    eos = oracle.generate(prompts[0].tolist(), 8)[2]
    st, oracle, pool = _serve(1, 48, None, prompts, 8, eos_token_id=eos, stop_on_eos=True)
    for r in st.retired:
        assert r.output == oracle.generate(prompts[r.req_idx].tolist(), 8, eos_token_id=eos)


def test_qwen_style_bias_and_llama31_rope_scaling_paths():
    """QKV bias (Qwen2) and Llama-3.1 frequency scaling go through the same serving path."""
    import copy
    from nanoflow_b200 import config as C

    for name, patch in (("tiny-bias", {"model_type": "qwen2", "architectures": ["Qwen2ForCausalLM"]}),
                        ("tiny-l31", {"rope_scaling": dict(C._LLAMA31_SCALING, original_max_position_embeddings=16)})):
        C.MODEL_ARCHS[name] = dict(copy.deepcopy(C.MODEL_ARCHS["tiny"]), **patch)
        try:
            rng = np.random.default_rng(3)
            prompts = [rng.integers(0, 1024, size=n, dtype=np.int32) for n in (20, 33)]
            st, oracle, pool = _serve(2, 48, [16, 32], prompts, 6, model=name)
            assert oracle.cfg.qkv_bias == (name == "tiny-bias")
            for r in st.retired:
                assert r.output == oracle.generate(prompts[r.req_idx].tolist(), 6)
        finally:
            del C.MODEL_ARCHS[name]


def test_module_level_api_with_the_reference_bindings_names():
    """setModelConfig -> createModelWeight -> init -> config -> update / run_async / run_async_wait ->
    getPipelineOutput -> finalize, as a user of the reference's ``pllm_python`` module would call them."""
    import nanoflow_b200.pllm_python as pllm
    from nanoflow_b200.config import make_config
    from nanoflow_b200.models import random_full_weights

    raw = make_config("tiny", gpu_num=2, global_batch_size=48, pipeline_type="PLLM", nanobatch_sizes=[16, 32])
    cfg = pllm.setModelConfig(raw, backend="cpu")
    with pytest.raises(RuntimeError, match="init first"):
        pllm.config()
    weights = pllm.createModelWeight(seed=0)
    assert len(weights) == 2
    pllm.init(weights, pllm.createInitData(num_pages=64))
    pllm.config()
    assert pllm.num_pages() == 64
    oracle = ReferenceLlama(cfg.model, random_full_weights(cfg.model, seed=0))
    prompt = np.arange(5, 25, dtype=np.int32)
    rm = RequestManager(vocab_size=cfg.model.vocab_size)
    rm.add_request(len(prompt), 6, 0.0, prompt=prompt)
    rm.finalize_stats()
    rm.simulate_issue(1.0)
    pool = DistKVPool(cfg.model.run_layers, cfg.model.num_kv_heads, cfg.model.head_dim, 64, 16, 2)
    sch = Scheduler(pool, rm.avaliable_request_queue, global_batch_size=48, nanobatch_sizes=[16, 32],
                    average_prefill_length=20, average_decode_length=6, group_size=cfg.model.group_size)
    out = []
    while True:
        plan = sch.schedule()
        if plan is None:
            break
        pllm.update(plan)
        pllm.run_async()
        toks = pllm.run_async_wait()
        assert (pllm.getPipelineOutput() == toks).all()
        sch.process_outputs(plan, toks)
        out.extend(int(t) for t in toks)
    pllm.finalize()
    assert pllm.engine() is None
    assert out[:6] == oracle.generate(prompt.tolist(), 6)


def test_oracle_agrees_with_the_hugging_face_llama_implementation():
    """The fp32 oracle every engine test is compared with, against an independent implementation: the
    tiny model's weights loaded into ``transformers.LlamaForCausalLM`` (the reference's ground truth is HF
    greedy decoding, groundtruth/test.py:12-38). Logits of a 32-token prompt and 16 greedy tokens; also
    with Llama-3.1 rotary scaling and with QKV bias (Qwen2)."""
    transformers = pytest.importorskip("transformers")
    from nanoflow_b200.models import random_full_weights

    def hf_model(cfg, fw, cls, conf_cls, **extra):
        conf = conf_cls(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_layers,
                        num_attention_heads=cfg.num_q_heads, num_key_value_heads=cfg.num_kv_heads,
                        vocab_size=cfg.vocab_size, rms_norm_eps=cfg.rms_norm_eps, max_position_embeddings=4096,
                        tie_word_embeddings=False, attn_implementation="eager", **extra)
        model = cls(conf).float().eval()
        sd = {"model.embed_tokens.weight": fw.embed, "model.norm.weight": fw.norm, "lm_head.weight": fw.lm_head}
        for l, lay in enumerate(fw.layers):
            p = f"model.layers.{l}."
            sd.update({p + "self_attn.q_proj.weight": lay.wq, p + "self_attn.k_proj.weight": lay.wk,
                       p + "self_attn.v_proj.weight": lay.wv, p + "self_attn.o_proj.weight": lay.wo,
                       p + "mlp.gate_proj.weight": lay.wg, p + "mlp.up_proj.weight": lay.wu,
                       p + "mlp.down_proj.weight": lay.wd, p + "input_layernorm.weight": lay.ln_attn,
                       p + "post_attention_layernorm.weight": lay.ln_ffn})
            if lay.bq is not None:
                sd.update({p + "self_attn.q_proj.bias": lay.bq, p + "self_attn.k_proj.bias": lay.bk,
                           p + "self_attn.v_proj.bias": lay.bv})
        missing, unexpected = model.load_state_dict({k: v.float() for k, v in sd.items()}, strict=False)
        assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
        return model

    import dataclasses

    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 1024, size=32, dtype=np.int64)
    base = builtin_config("tiny").model
    llama31 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    cases = [("llama", base, transformers.LlamaForCausalLM, transformers.LlamaConfig, {}),
             ("llama-3.1 rope", dataclasses.replace(base, rope_scaling=dict(llama31)), transformers.LlamaForCausalLM,
              transformers.LlamaConfig, {"rope_scaling": dict(llama31)}),
             ("qwen2 bias", dataclasses.replace(base, qkv_bias=True), transformers.Qwen2ForCausalLM,
              transformers.Qwen2Config, {})]
    for name, cfg, cls, conf_cls, extra in cases:
        fw = random_full_weights(cfg, seed=0, std=0.05)
        assert (fw.layers[0].bq is not None) == cfg.qkv_bias
        oracle = ReferenceLlama(cfg, fw)
        rope = dict(extra.pop("rope_scaling", None) or {"rope_type": "default"}, rope_theta=cfg.rope_theta)
        try:
            hf = hf_model(cfg, fw, cls, conf_cls, rope_parameters=rope, **extra)
        except TypeError:      # older transformers: separate rope_theta / rope_scaling arguments
            sc = {k: v for k, v in rope.items() if k != "rope_theta"}
            hf = hf_model(cfg, fw, cls, conf_cls, rope_theta=cfg.rope_theta,
                          rope_scaling=None if sc == {"rope_type": "default"} else sc, **extra)
        with torch.no_grad():
            want = hf(torch.from_numpy(prompt)[None]).logits[0]
            got, _ = oracle.forward(torch.from_numpy(prompt))
            assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (name, (got - want).abs().max())
            ids = torch.from_numpy(prompt)[None]
            gen = hf.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=16, do_sample=False,
                              pad_token_id=0)[0, 32:].tolist()
        assert oracle.generate(prompt.tolist(), 16) == gen, name
