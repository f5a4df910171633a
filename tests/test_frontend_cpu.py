"""Config schema, trace frontend, KV page accounting, weight files, stats files, trace generators."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from nanoflow_b200 import config as C
from nanoflow_b200.datasets import traces
from nanoflow_b200.models import random_full_weights, shard_weights
from nanoflow_b200.models.weights import load_rank_weights, rank_state_dicts, save_weights
from nanoflow_b200.serving import (BatchedDistKVCache, DistKVCache, DistKVPool, KVPoolExhausted, RequestManager)


def test_shipped_configs_parse_and_derive_per_gpu_sizes():
    files = glob.glob(str(C.CONFIG_DIR / "*" / "*.json"))
    assert len(files) >= 50
    for f in files:
        cfg = C.load_config(f)
        assert cfg.engine.pipeline_type in C.PIPELINE_TYPES
        assert sum(cfg.engine.resolved_nanobatches()) == cfg.engine.global_batch_size
    cfg = C.load_config(C.shipped_config_path("llama2-70B", "2048"))
    m = cfg.model
    # per-GPU shapes of Llama-2-70B at TP 8 (the reference derives the same: pipeline/include/config.h:90-100)
    assert (m.hidden_size, m.q_heads_local, m.kv_heads_local, m.ffn_local, m.qkv_size_local) == (8192, 8, 1, 3584, 1280)
    q = C.load_config(C.shipped_config_path("qwen2-72B", "2048"))
    assert q.model.qkv_bias and q.engine.pipeline_type == "KQVBIAS" and q.model.vocab_local * 8 >= 152064
    l31 = C.load_config(C.shipped_config_path("llama3.1-8B", "2048"))
    assert l31.model.rope_scaling["rope_type"] == "llama3" and l31.engine.pipeline_type == "LOCAL"
    # the scaled-down sets: few layers' weights run as the full depth; a fixed small KV pool
    nested = glob.glob(str(C.CONFIG_DIR / "*" / "*" / "*.json"))
    assert len(nested) >= 8 * len(glob.glob(str(C.CONFIG_DIR / "*")))
    for f in nested:
        C.load_config(f)
    few = C.load_config(C.shipped_config_path("llama2-70B", "fewer_layers/2048"))
    assert (few.model.num_layers, few.model.run_layers) == (4, 80) and few.model.param_count() < 5e9
    small = C.load_config(C.shipped_config_path("llama2-70B", "small_kv/2048"))
    assert small.engine.num_pages == 400 * 64 and small.model.num_layers == 80
    # the files on disk are what the generator writes
    import json
    for name, raw in C.shipped_variants("llama3-8B").items():
        assert json.load(open(C.shipped_config_path("llama3-8B", name))) == raw, name


def test_reference_config_file_loads_unchanged():
    """A config in the reference's own schema (gemm_op_tag, nanobatch_1_size, kqv sizes) is accepted."""
    raw = C.make_config("llama2-70B", gpu_num=8, global_batch_size=2048, pipeline_type="PLLM")
    raw["pipeline_configs"] = {"gemm_op_tag": ["128_128_32_64_64_32_3_5_RowMajor_RowMajor_RowMajor"] * 9,
                               "global_batch_size": 2048, "nanobatch_1_size": 640, "kqv1_size": 256, "kqv3_size": 768}
    raw["model_configs"].update({"allocate_kv_data_batch": 1480, "gpu_mem": 68719476736, "page_mem_size": 32768})
    cfg = C.parse_config(raw)
    assert cfg.engine.resolved_nanobatches() == [640, 1408]
    assert cfg.engine.num_pages == 1480 * 64 and len(cfg.engine.gemm_op_tag) == 9


@pytest.mark.parametrize("mutate,msg", [
    (lambda r: r.pop("pipeline_configs"), "missing section"),
    (lambda r: r["serve_configs"].update(pipeline_type="WARP"), "unknown pipeline_type"),
    (lambda r: r["pipeline_configs"].update(nanobatch_sizes=[100, 100]), "must sum"),
    (lambda r: r["model_configs"].update(gpu_num=3), "not divisible"),
])
def test_malformed_configs_are_rejected(mutate, msg):
    raw = C.make_config("llama3-8B", gpu_num=1, global_batch_size=2048)
    mutate(raw)
    with pytest.raises(ValueError, match=msg):
        C.parse_config(raw)


def test_trace_reader_and_release_clock(tmp_path):
    p = tmp_path / "t.csv"
    p.write_text("idx,input_len,output_len,arrival\n0,10,3,0.0\n1,20,4,0.5\n2,5,2,1.5\n")
    rm = RequestManager(str(p), vocab_size=100, random_ids=True)
    rm.read_request()
    assert rm.full_request_queue.size == 3 and rm.average_prefill_length == 11 and rm.average_decode_length == 3
    rm.simulate_issue(0.6)
    assert rm.avaliable_request_queue.size == 2
    rm.simulate_issue(1.0)
    assert rm.avaliable_request_queue.size == 3
    r = rm.avaliable_request_queue.get()
    assert r.prompt.dtype == np.int32 and r.prompt.size == 10 and r.prompt.max() < 100


@pytest.mark.parametrize("body,err", [
    ("0,10\n", "expected idx"), ("0,abc,3,0.0\n", "invalid literal"), ("0,0,3,0.0\n", "input_len"),
    ("0,10,0,0.0\n", "output_len"), ("0,-1,3,0.0,hello\n", "no tokenizer"), ("", "no requests")])
def test_malformed_traces_are_rejected(tmp_path, body, err):
    p = tmp_path / "bad.csv"
    p.write_text("idx,input_len,output_len,arrival\n" + body)
    with pytest.raises(ValueError, match=err):
        RequestManager(str(p)).read_request()


def test_kv_pool_and_cache_accounting():
    pool = DistKVPool(2, 8, 128, 10, 16, 8)
    a, b = DistKVCache(pool), DistKVCache(pool)
    a.allocate_tokens(17)
    assert a.num_pages == 2 and a.last_page_offset == 1 and pool.num_free_pages == 8
    a.allocate_tokens(15)
    assert a.num_pages == 2 and a.seqlen == 32 and a.last_page_offset == 16
    b.allocate_tokens(100)
    assert b.num_pages == 7 and pool.num_free_pages == 1
    with pytest.raises(KVPoolExhausted):
        a.allocate_tokens(33)
    assert a.seqlen == 32 and a.num_pages == 2                      # failed allocation changed nothing
    batched = BatchedDistKVCache([a], [b])
    assert batched.kv_indptr.tolist() == [0, 2, 9] and batched.kv_last_page_len.tolist() == [16, 4]
    assert sorted(batched.kv_indices.tolist()) == sorted(a.indicies.tolist() + b.indicies.tolist())
    b.release()
    a.release()
    assert pool.num_free_pages == 10
    with pytest.raises(ValueError):
        pool.free_page(3)                                            # double free
    with pytest.raises(ValueError):
        DistKVPool(2, 6, 128, 10, 16, 4)                             # heads not divisible by devices


def test_weight_files_have_reference_keys_and_layout(tmp_path):
    cfg = C.builtin_config("tiny", gpu_num=2).model
    fw = random_full_weights(cfg, seed=3)
    sds = rank_state_dicts(fw, 2, dtype=torch.float32)
    keys = set(sds[0])
    assert {"ModelNorm", "Embed", "LmHead", "O1_0", "O2_0", "U_0", "G_0", "D_0", "KQV_0", "BKQV_0", "LNATT_0", "LNFFN_0"} <= keys
    h, hd = cfg.hidden_size, cfg.head_dim
    assert sds[0]["KQV_0"].shape == (h, cfg.qkv_size_local)             # [K, N], K | V | Q packed
    assert sds[0]["O2_0"].shape == (cfg.q_size_local, h) and sds[0]["D_0"].shape == (cfg.ffn_local, h)
    assert sds[0]["LmHead"].shape == (h, cfg.vocab_size)
    kv = cfg.kv_size_local
    assert torch.equal(sds[1]["KQV_0"][:, :kv].t(), fw.layers[0].wk[kv:2 * kv])
    assert torch.equal(sds[1]["KQV_0"][:, 2 * kv:].t(), fw.layers[0].wq[cfg.q_size_local:])
    save_weights(fw, 2, str(tmp_path), dtype=torch.float32)
    for r in range(2):
        got = load_rank_weights(str(tmp_path), cfg, r, 2, dtype=torch.float32)
        want = shard_weights(fw, cfg, r, 2, dtype=torch.float32)
        assert torch.equal(got.lm_head, want.lm_head)
        for a, b in zip(got.layers, want.layers):
            for k in ("wqkv", "wo", "wg", "wu", "wd", "ln_attn", "ln_ffn"):
                assert torch.equal(getattr(a, k), getattr(b, k)), k
    with pytest.raises(FileNotFoundError):
        load_rank_weights(str(tmp_path), cfg, 5, 8)


def test_trace_generators():
    rows = traces.fixed_trace(1024, 512, 10)
    assert all(r == (1024, 512, 0.0) for r in rows)
    t1, t2 = traces.poisson_arrivals(1000, 20.0), traces.poisson_arrivals(1000, 20.0)
    assert np.array_equal(t1, t2) and np.all(np.diff(t1) > 0) and abs(t1[-1] / 1000 - 0.05) < 0.01
    pairs = traces.lognormal_lengths(5000)
    ins, outs = np.array(pairs).T
    assert ins.min() >= 16 and ins.max() <= 4096 and outs.min() >= 1 and outs.max() <= 2048
    assert 450 < np.median(ins) < 750 and 180 < np.median(outs) < 330
    kept = traces.filter_lengths([(100, 10), (4000, 10), (3000, 1024), (3072, 1025), (10, 0)])
    assert kept == [(100, 10), (3000, 1024)]
    assert len(traces.real_trace([(100, 10), (200, 20)], 7, rate=5.0)) == 7


def test_serve_command_line_on_the_cpu_backend(tmp_path):
    """``python -m nanoflow_b200.serve`` end to end on the CPU backend: a config file, a trace with identical
    prompts, the reference's flags, and every output file it promises."""
    import csv
    import gzip
    import json

    from nanoflow_b200 import serve
    from nanoflow_b200.config import make_config

    cfg = make_config("tiny", gpu_num=2, global_batch_size=48, pipeline_type="PLLM", nanobatch_sizes=[16, 32])
    cfg_path = tmp_path / "tiny.json"
    cfg_path.write_text(json.dumps(cfg))
    trace = tmp_path / "trace.csv"
    with open(trace, "w") as f:
        f.write("idx,input_len,output_len,arrival\n")
        for i in range(6):
            f.write(f"{i},20,5,0.0\n")
    prefix = str(tmp_path / "out" / "run")
    rc = serve.main(["-t", str(trace), "-c", str(cfg_path), "--backend", "cpu", "--until_empty", "true",
                     "--random_ids", "false", "-o", prefix, "--allocate_page_num", "64", "--output_idx", "true"])
    assert rc == 0
    for ext in (".stat", ".stat.csv", ".req_time", ".req_tokens", ".req_tokens.uniq", ".schedule"):
        assert (tmp_path / "out" / ("run" + ext)).exists(), ext
    rows = list(csv.DictReader(open(prefix + ".stat.csv")))
    assert len(rows) == 1 and float(rows[0]["token_per_second"]) > 0
    # synthetic prompts are range(len): six identical prompts must give one distinct output
    uniq = open(prefix + ".req_tokens.uniq").read().strip().splitlines()
    assert len(uniq) == 1 and uniq[0].split()[0] == "6"
    assert len(open(prefix + ".req_tokens").read().strip().splitlines()) == 6
    # profile mode: ten cycles under torch.profiler, Chrome trace written compressed
    prefix2 = str(tmp_path / "prof" / "run")
    rc = serve.main(["-t", str(trace), "-c", str(cfg_path), "--backend", "cpu", "--random_ids", "false", "-o", prefix2,
                     "--allocate_page_num", "64", "--profile_mode", "true"])
    assert rc == 0
    with gzip.open(prefix2 + ".trace.json.gz", "rt") as f:
        tr = json.load(f)
    names = {ev.get("name") for ev in tr["traceEvents"]}
    assert {"model_inference", "schedule", "update", "launch", "wait_previous", "process_outputs"} <= names
    # one log file per rank beside the outputs
    text = open(tmp_path / "out" / "log_0.txt").read()
    assert "serving" in text and "done:" in text and "requests retired" in text


def test_eval_harness_runs_resumes_merges_and_plots_on_the_cpu_backend(tmp_path):
    """One fixed-length point, a two-rate online sweep and the summary / merge / plot steps of the
    experiment runner on the tiny model (CPU backend, one process per point)."""
    import json
    import os

    from nanoflow_b200.eval import harness

    out = str(tmp_path / "res")
    common = ["--model", "tiny", "--gpus", "1", "--batch", "48", "--out", out, "--backend", "cpu",
              "--run_cycles", "40", "--skip_cycles", "0"]
    assert harness.main(["fixed-offline", "--workloads", "512-2", *common]) == 0
    stat = os.path.join(out, "fixed-tiny-512-2.stat.csv")
    assert os.path.exists(stat)
    before = os.path.getmtime(stat)
    assert harness.main(["fixed-offline", "--workloads", "512-2", *common]) == 0     # finished point: skipped
    assert os.path.getmtime(stat) == before
    assert harness.main(["online", "--rates", "40", "80", "--requests", "6", *common]) == 0
    assert harness.main(["summarize", "--out", out]) == 0
    assert harness.main(["merge", "--model", "tiny", "--out", out]) == 0
    merged = json.load(open(os.path.join(out, "pllm.json")))
    assert merged["offline_throughput_const"]["512-2"] > 0
    sweep = merged["online_throughput"]["b48"]
    assert sweep["request_rate"] == [40.0, 80.0] and all(v > 0 for v in sweep["normalized_latency"])
    assert harness.main(["plot", "--out", out]) == 0
    assert os.path.exists(os.path.join(out, "figures.txt")) or os.path.exists(os.path.join(out, "figure_0.png"))


def test_bench_reference_arm_reports_why_it_cannot_run():
    """``bench.py --impl reference`` must print one JSON line with ``impl`` and ``unavailable`` and exit 0
    wherever the reference cannot be installed (it is a CMake project with empty submodules here)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and isinstance(out["unavailable"], str) and "\n" not in out["unavailable"]


def test_hugging_face_snapshot_is_converted_and_served(tmp_path):
    """A Hugging Face snapshot directory (config.json + safetensors) named by ``hf_path``: serve writes the
    per-rank weight files on first use, loads them, and the generated tokens are those of
    ``transformers`` greedy decoding on the same prompt; the converter's command line gives the same files."""
    import json

    transformers = pytest.importorskip("transformers")
    pytest.importorskip("safetensors")
    from nanoflow_b200 import serve
    from nanoflow_b200.config import make_config
    from nanoflow_b200.models import weights as W

    torch.manual_seed(0)
    conf = transformers.LlamaConfig(hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                                    num_key_value_heads=2, vocab_size=1024, rms_norm_eps=1e-5,
                                    max_position_embeddings=4096, tie_word_embeddings=False,
                                    attn_implementation="eager")
    hf = transformers.LlamaForCausalLM(conf).float().eval()
    for prm in hf.parameters():                      # larger weights: well-separated logits
        prm.data.mul_(3.0)
    hf_dir = tmp_path / "hf"
    hf.save_pretrained(str(hf_dir), safe_serialization=True)
    wdir = tmp_path / "converted"
    cfg = make_config("tiny", gpu_num=2, global_batch_size=48, pipeline_type="PLLM", nanobatch_sizes=[16, 32])
    cfg["serve_configs"]["weight_path"], cfg["serve_configs"]["hf_path"] = str(wdir), str(hf_dir)
    cfg_path = tmp_path / "tiny.json"
    cfg_path.write_text(json.dumps(cfg))
    trace = tmp_path / "trace.csv"
    trace.write_text("idx,input_len,output_len,arrival\n0,20,8,0.0\n1,33,8,0.0\n")
    prefix = str(tmp_path / "run")
    assert serve.main(["-t", str(trace), "-c", str(cfg_path), "--backend", "cpu", "--until_empty", "true",
                       "--random_ids", "false", "-o", prefix, "--allocate_page_num", "64"]) == 0
    assert sorted(p.name for p in wdir.iterdir()) == ["weight_rank_0.pt", "weight_rank_1.pt"]
    got = {}
    for line in open(prefix + ".req_tokens").read().strip().splitlines():
        idx, toks = line.split(":")
        got[int(idx)] = [int(t) for t in toks.split()]
    for idx, n in ((0, 20), (1, 33)):
        prompt = torch.arange(n)[None]               # synthetic prompts are 0, 1, 2, ... (not random here)
        with torch.no_grad():
            want = hf.generate(prompt, attention_mask=torch.ones_like(prompt), max_new_tokens=8, do_sample=False,
                               pad_token_id=0)[0, n:].tolist()
        assert got[idx] == want, idx
    # the command-line converter writes the same tensors
    out2 = tmp_path / "cli"
    assert W.main(["--hf", str(hf_dir), "--out", str(out2), "--nranks", "2", "--dtype", "fp32"]) == 0
    a, b = torch.load(out2 / "weight_rank_1.pt"), torch.load(wdir / "weight_rank_1.pt")
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)


def test_demo_entry_points(tmp_path, capsys):
    """``demo serve`` (trace of identical prompts -> serve -> first output) on the tiny model and CPU backend;
    ``demo perf --dry_run`` lists one serve command per experiment point without running any."""
    from nanoflow_b200 import demo

    out = tmp_path / "d"
    assert demo.main(["serve", "--model", "tiny", "--backend", "cpu", "--decode-length", "5", "--requests", "4",
                      "--out", str(out), "--prompt", "one two three four five six"]) == 0
    txt = capsys.readouterr().out
    assert "first request (demo.req_tokens): 0:" in txt
    lines = open(out / "demo.req_tokens").read().strip().splitlines()
    assert len(lines) == 4 and len({ln.split(":")[1] for ln in lines}) == 1      # identical prompts, identical outputs
    assert open(out / "trace.csv").read().splitlines()[1].startswith("0,6,5,")   # six words -> six synthetic ids
    assert demo.main(["perf", "--model", "tiny", "--gpus", "1", "--backend", "cpu", "--out", str(tmp_path / "p"),
                      "--dry_run", "--batch", "48"]) == 0
    cmds = [ln for ln in capsys.readouterr().out.splitlines() if "nanoflow_b200.serve" in ln]
    assert len(cmds) >= 5 + 1 + 7      # fixed workloads, one length distribution, the request-rate sweep
