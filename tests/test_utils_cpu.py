"""Command-line helpers and the GEMM autotuner's candidate list (no GPU needed)."""
import csv

import pytest

from nanoflow_b200.ops import autotune
from nanoflow_b200.utils import schedule_tools as st


def test_gen_req_format(tmp_path):
    p = tmp_path / "req.csv"
    assert st.gen_req("hello world", 7, 4, str(p), n=5) == 5
    lines = p.read_text().splitlines()
    assert lines[0] == "0,-1,7,0.0, hello world"
    assert lines[4].startswith("4,-1,7,1.0,")


def test_cycle_log_to_csv(tmp_path):
    log = tmp_path / "log.txt"
    log.write_text(
        "------------------ Cycle 0 ------------------\n"
        "memory usage %: 12.5\ndecode effective bsz: 3\n"
        "------------------ Skip Cycle 1 ------------------\n"
        "memory usage %: 13.0\nprefill effective bsz: 256\n")
    out = tmp_path / "log.csv"
    assert st.cycle_log_to_csv(str(log), str(out)) == 2
    rows = list(csv.DictReader(out.open()))
    assert rows[0]["Cycle"] == "0" and rows[0]["is_skip_cycle"] == "False" and rows[0]["memory usage %"] == "12.5"
    assert rows[1]["is_skip_cycle"] == "True" and rows[1]["prefill effective bsz"] == "256"
    assert rows[1]["decode effective bsz"] == ""


def test_plot_schedule_writes_something(tmp_path):
    p = tmp_path / "run.schedule"
    with p.open("w") as f:
        f.write("iteration,decode_tokens,prefill_tokens,batch_size,idle_tokens,page_usage,queue,retired\n")
        for i in range(50):
            f.write(f"{i},{100 + i},{156 - i},256,0,{i / 50},10,0\n")
    files = st.plot_schedule(str(p))
    assert files and all((tmp_path / f.split("/")[-1]).exists() for f in files)
    assert "max" in st.text_plot([1.0, 2.0, 3.0])


def test_plot_trend(tmp_path):
    p = tmp_path / "trend.csv"
    p.write_text("\n".join(f"{i},{2 * i}" for i in range(20)))
    out = st.plot_trend(str(p))
    assert out.startswith(str(p))


def test_autotune_candidates():
    for (M, N, K, sw) in [(256, 8192, 8192, False), (4096, 1280, 8192, False), (100, 3584, 8192, True),
                          (2048, 28672, 8192, True), (1, 128, 64, False)]:
        c = autotune.candidates(M, N, K, sw)
        assert c[0] == autotune.AUTO                       # the cost model's own choice is always timed
        assert len(c) == len({tuple(sorted(x.items())) for x in c})
        for x in c[1:]:
            assert x["tile_m"] * x["tile_n"] <= 512 and x["tile_n"] % 32 == 0
            assert not (x["cta_group"] == 2 and (x["tile_m"] != 1 or M <= 128))
            assert not (sw and x["split_k"] != 1)
            assert not (x["split_k"] > 1 and x["stream_k"] == 1)
            # tiles wider than one MMA instruction: CTA pairs only, never for the SwiGLU form, and what the
            # launcher's planner accepts
            if x["tile_n"] > 256:
                assert x["cta_group"] == 2 and x["tile_m"] == 1 and not sw and x["tile_n"] <= N
                from nanoflow_b200 import ops
                plan = ops.gemm_plan(M, N, K, tile_m=1, tile_n=x["tile_n"], cta_group=2, split_k=1, stream_k=2)
                assert plan["tile_n"] == x["tile_n"] and plan["stages"] >= 2
    wide = [x["tile_n"] for x in autotune.candidates(4096, 1280, 8192, False) if x["tile_n"] > 256]
    assert 320 in wide


def _walk(w, W, tiles, num_kb, split_k, tail_first, q):
    """The kernel's work distribution (csrc/kernels/gemm.cu, struct Walk) restated: worker w's units."""
    out = []
    dp_tiles = tail_first if q > 0 else tiles
    units, kb_per = dp_tiles * split_k, -(-num_kb // split_k)
    cur = w
    while cur < units:
        ks = cur // dp_tiles
        kb0 = min(num_kb, ks * kb_per)
        out.append((cur % dp_tiles, kb0, min(num_kb, kb0 + kb_per), 1))
        cur += W
    if q > 0:
        total = (tiles - tail_first) * num_kb
        g = min(w * q, total)
        g_end = min(g + q, total)
        while g < g_end:
            t, kb0 = divmod(g, num_kb)
            n = min(num_kb - kb0, g_end - g)
            first, last = (t * num_kb) // q, (min((t + 1) * num_kb, total) - 1) // q
            out.append((tail_first + t, kb0, kb0 + n, last - first + 1))
            g += n
    return out


def test_gemm_plan_covers_every_tile_once():
    """The launcher's plan (shape choice + stream-K tail), asked for without a GPU, tiles the whole
    problem: every (tile, k-block) belongs to exactly one worker and no tile is cut into more pieces
    than the partial-sum slots the plan reserves."""
    from nanoflow_b200 import ops

    cases = [dict(M=256, N=8192, K=8192), dict(M=4096, N=1280, K=8192), dict(M=3712, N=8192, K=3584),
             dict(M=2048, N=28672, K=8192, swiglu=True), dict(M=3712, N=1280, K=1024, cta_group=2, tile_n=256,
                                                                tile_m=1, stream_k=1),
             dict(M=300, N=4096, K=1536, tile_m=4, tile_n=128, stream_k=1), dict(M=1000, N=3000, K=1024, num_ctas=37),
             dict(M=256, N=8192, K=2048, split_k=4, tile_m=2, tile_n=256), dict(M=130, N=40, K=64)]
    for c in cases:
        pl = ops.gemm_plan(workspace_bytes=256 << 20, **c)
        assert pl["stages"] >= 2 and pl["smem_bytes"] <= 227 * 1024
        assert 1 <= pl["workers"] <= 148 // pl["cta_group"]
        seen = {}
        for w in range(pl["workers"]):
            for tile, kb0, kb1, pieces in _walk(w, pl["workers"], pl["tiles"], pl["num_kb"], pl["split_k"],
                                                pl["tail_first_tile"], pl["tail_range_kb"]):
                assert kb1 > kb0 or pl["split_k"] > 1
                assert pieces <= max(1, pl["tail_max_pieces"])
                seen.setdefault(tile, []).append((kb0, kb1))
        assert sorted(seen) == list(range(pl["tiles"])), c
        for tile, segs in seen.items():
            segs = sorted(s for s in segs if s[1] > s[0])
            assert segs[0][0] == 0 and segs[-1][1] == pl["num_kb"]
            assert all(a[1] == b[0] for a, b in zip(segs, segs[1:])), (c, tile, segs)


def test_guarded_arena_reports_writes_outside_a_buffer():
    import torch

    from nanoflow_b200.utils.guards import GUARD_BYTES, GuardedArena

    arena = GuardedArena("cpu")
    a = arena.zeros("a", (5, 7), torch.bfloat16)        # 70 bytes: the rear guard starts inside the 16-byte padding
    b = arena.zeros("b", (4,), torch.int32)
    c = arena.zeros("a", (3,), torch.float32)           # a second buffer of the same name gets a suffix
    assert a.shape == (5, 7) and a.dtype == torch.bfloat16 and a.is_contiguous() and a.data_ptr() % 16 == 0
    assert not a.any() and not b.any() and len(arena) == 3
    a.fill_(1.0); b.fill_(-1); c.fill_(2.0)             # full use of the payloads leaves the guards alone
    assert arena.check() == []
    flat = a.view(torch.uint8).view(-1)
    past = torch.as_strided(flat, (2,), (1,), flat.storage_offset() + flat.numel())   # the two bytes after a's last element
    past.fill_(0)
    before = torch.as_strided(b.view(torch.uint8).view(-1), (1,), (1,), GUARD_BYTES - 4)   # 4 bytes before b's first
    before.fill_(7)
    assert arena.check() == [("a", "rear", 0), ("b", "front", GUARD_BYTES - 4)]
    arena.restore()
    assert arena.check() == []
    assert (a == 1.0).all() and (b == -1).all() and (c == 2.0).all()
    try:
        GuardedArena("cpu", guard_bytes=24)
    except ValueError:
        pass
    else:
        raise AssertionError("guard size must be a multiple of 16")


def test_parameter_search_finds_the_best_point_and_writes_a_loadable_config(tmp_path):
    from nanoflow_b200.config import load_config
    from nanoflow_b200.eval import search as S

    assert S.split_sizes(8192, 0.5) == [4096, 4096] and S.split_sizes(8192, 0.44) == [3584, 4608]
    assert S.split_sizes(1408, 0.01) == [128, 1280] and S.split_sizes(1408, 0.99) == [1280, 128]
    with pytest.raises(ValueError):
        S.split_sizes(200, 0.5)
    calls = []

    def runner(pt):       # a separable surface with its top at share 0.45 (3712 of 8192), 96 CTAs, tail 0.25
        calls.append(pt)
        return 50000 - 4e-3 * (pt["nano"][0] - 3712) ** 2 - 2.0 * abs(pt["comm_ctas"] - 96) - 4000 * abs(pt["decode_tail"] - 0.25)

    best, v, log = S.search(8192, [0.40, 0.45, 0.50, 0.55, 0.60], [64, 96, 128], [0.0, 0.25, 0.5], runner, rounds=3)
    assert best["nano"] == [3712, 4480] and best["comm_ctas"] == 96 and best["decode_tail"] == 0.25
    assert v == max(r["value"] for r in log) and len(log) == len(calls)
    keys = [(tuple(c["nano"]), c["comm_ctas"], c["decode_tail"]) for c in calls]
    assert len(set(keys)) == len(keys)                      # no point measured twice
    assert len(calls) < 5 * 3 * 3                           # and far fewer than the full grid
    files = S.write_results(str(tmp_path), "llama2-70B", 8, 8192, "PLLM", best, v, log)
    cfg = load_config(files[0], tp=8)
    assert cfg.engine.resolved_nanobatches() == [3712, 4480] and cfg.engine.sm_budget["comm"] == 96
    assert cfg.engine.decode_tail_fraction == 0.25 and cfg.engine.pipeline_type == "PLLM"
    rows = open(files[1]).read().strip().splitlines()
    assert rows[0] == "nanobatches,comm_ctas,decode_tail,switches,tokens_per_s" and len(rows) == len(log) + 1
    # more nano-batches and bench switches as further axes
    assert S.split_sizes(8192, 0.25, count=4) == [2048, 2048, 2048, 2048] and sum(S.split_sizes(8192, 0.3, count=3)) == 8192

    def runner2(pt):      # best: four nano-batches with the attention overlap on, two network streams
        v = 40000.0 + (3000 if (len(pt["nano"]) == 4 and pt["switches"]["attn-overlap"]) else 0)
        return v + (500 if pt["switches"]["net-streams"] == 2 else 0) - 1e-3 * abs(pt["nano"][0] - 8192 // len(pt["nano"]))

    best2, v2, log2 = S.search(8192, [0.45, 0.5, 0.55], [96], [0.0], runner2, rounds=3, nano_counts=[2, 4],
                               switches={"attn-overlap": [False, True], "net-streams": [1, 2]})
    assert best2["nano"] == [2048] * 4 and best2["switches"] == {"attn-overlap": True, "net-streams": 2}
    files2 = S.write_results(str(tmp_path / "b"), "llama2-70B", 8, 8192, "PLLM", best2, v2, log2)
    cfg2 = load_config(files2[0], tp=8)
    assert cfg2.engine.attn_overlap and cfg2.engine.net_streams == 2 and cfg2.engine.resolved_nanobatches() == [2048] * 4


def test_whatif_replay_of_an_op_graph():
    from nanoflow_b200.utils import whatif

    g = whatif.structural_graph(8, [4096, 4096], layers=3)
    names = [op.name for op in g.ops]
    assert "L2.nb1.ar_d" in names and "L0.nb0.attn_prefill" in names
    kind = lambda op: op.name.split(".")[-1]
    base = {"qkv": 90, "rope_append": 14, "attn_decode": 300, "attn_prefill": 60, "o": 70, "gate_up": 390, "down": 176,
            "ar_o": 420, "ar_d": 480}
    dur = [float(base.get(kind(op), 5)) for op in g.ops]
    sim = whatif.simulate(g, dur)
    # dependencies and stream order hold in the replay
    last = {}
    for i, op in enumerate(g.ops):
        assert all(sim["start"][i] >= sim["end"][d] - 1e-9 for d in op.deps)
        if op.stream in last:
            assert sim["start"][i] >= sim["end"][last[op.stream]] - 1e-9
        last[op.stream] = i
        assert abs(sim["end"][i] - sim["start"][i] - dur[i]) < 1e-9
    path = sim["critical_path"]
    assert sim["end"][path[-1]] == sim["makespan"] and sim["start"][path[0]] == 0.0
    assert all(abs(sim["start"][b] - sim["end"][a]) < 1e-9 for a, b in zip(path, path[1:]))
    # a single stream adds everything up; overlap can only be shorter; a faster collective never hurts
    assert abs(whatif.simulate(g, dur, single_stream=True)["makespan"] - sum(dur)) < 1e-6
    assert sim["makespan"] < sum(dur)
    faster = whatif.scale_durations(g, dur, {"ar_o": "0.5", "ar_d.nb1": "-100"})
    assert faster[names.index("L1.nb0.ar_o")] == 210 and faster[names.index("L1.nb1.ar_d")] == 380
    assert faster[names.index("L1.nb0.ar_d")] == 480
    assert whatif.simulate(g, faster)["makespan"] <= sim["makespan"]
    assert whatif.stream_gaps(g, sim, "gemm") > 0
    # durations come from a timeline by op name
    ev = [{"ph": "X", "name": "L1.nb0.qkv", "dur": 77.0}, {"ph": "M", "name": "x"}]
    d2 = whatif.durations_from_timeline(g, ev, default_us=4.0, launch_gap_us=1.0)
    assert d2[names.index("L1.nb0.qkv")] == 78.0 and d2[names.index("L0.nb0.qkv")] == 5.0


def test_timeline_of_several_ranks_in_one_trace(tmp_path):
    import json

    from nanoflow_b200.utils import timeline as tl

    r0 = [("L0.nb0.qkv", "gemm", 0.0, 90.0), ("L0.nb0.ar_o", "net", 90.0, 500.0), ("L0.nb0.gate_up", "gemm", 500.0, 900.0)]
    r1 = [("L0.nb0.qkv", "gemm", 0.0, 300.0), ("L0.nb0.ar_o", "net", 300.0, 500.0), ("L0.nb0.gate_up", "gemm", 500.0, 900.0)]
    path = tmp_path / "t.json"
    s = tl.dump_ranks([r0, r1], str(path))
    assert s["rank0"]["collectives_us"] == 410.0 and s["rank1"]["collectives_us"] == 200.0
    assert s["rank1"]["compute_stream_busy_us"] == 700.0 > s["rank0"]["compute_stream_busy_us"]     # rank 1 is the late one
    d = json.load(open(path))
    assert {e["pid"] for e in d["traceEvents"]} == {0, 1} and d["ranks"] == s
    assert d["aggregate"]["_iteration"]["total_us"] == 900.0
