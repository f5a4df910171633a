"""Command-line helpers and the GEMM autotuner's candidate list (no GPU needed)."""
import csv

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
