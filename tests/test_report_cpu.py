"""The report module on a measured ``bench.py`` line kept as a fixture."""

import json
import os

from moe_bench_b200 import report as R

HERE = os.path.dirname(os.path.abspath(__file__))
SAMPLE = os.path.join(HERE, "golden", "bench_line_sample.json")


def test_reference_row_keys_and_extensions():
    line = json.load(open(SAMPLE))
    row = R.rows_from_bench(line)
    # the reference's columns (report.py:13-23)
    for key in ("num_tokens", "latency_us", "tflops", "local_assignments", "timing", "rel_err", "verify"):
        assert key in row
    assert row["num_tokens"] == 8192 and row["local_assignments"] == 8192 * 8
    assert abs(row["latency_us"] - line["ms_per_step"] * 1e3) < 1e-9
    # 6*N*K flop per assignment (reference bench.py:40-49)
    assert abs(row["tflops"] - 6 * 2048 * 7168 * 65536 / (row["latency_us"] * 1e-6) / 1e12) < 1e-6 * row["tflops"]
    assert 0 < row["roofline_frac"] <= 1.2 and row["vllm_us"] > row["latency_us"]
    assert set(row["stage_achieved"]) == {"align", "gate_up_gemm", "down_gemm", "combine"}
    pay = R.payload([row], line["config"])
    assert set(pay) == {"config", "implementation", "results"}      # report.py:68-81


def test_table_renders(tmp_path, capsys):
    out = tmp_path / "rows.json"
    R.main([SAMPLE, "--json", str(out)])
    text = capsys.readouterr().out
    assert "TFLOP/s" in text and "gate_up_gemm" in text and "8192" in text
    assert json.load(open(out))["results"][0]["verify"] == "ok"


def test_measured_line_carries_its_sweep_points():
    """The fixture is a whole default line: its secondary list is the bf16 and fp8 token sweep."""
    line = json.load(open(SAMPLE))
    rows = R.rows_from_secondary(line)
    assert sorted({(r["precision"], r["num_tokens"]) for r in rows}) == sorted(
        (p, t) for p in ("bf16", "fp8") for t in (1, 8, 128, 2048, 8192))
    assert all(r["verify"] == "ok" and r["latency_us"] > 0 for r in rows)
    fp8 = {r["num_tokens"]: r["latency_us"] for r in rows if r["precision"] == "fp8"}
    bf16 = {r["num_tokens"]: r["latency_us"] for r in rows if r["precision"] == "bf16"}
    assert all(fp8[t] < bf16[t] for t in fp8)          # fp8 is the faster precision at every point


def test_secondary_legs_become_rows():
    line = json.load(open(SAMPLE))
    line["secondary"] = [
        {"precision": "fp8", "tokens_per_gpu": 128, "mode": "single", "ms": 1.8, "tflops": 50.0,
         "layer_roofline_frac": 0.94, "verify": "ok", "rel_err": 2.3e-3, "stage_ms": {"gate_up_gemm": 1.1}},
        {"precision": "fp8", "tokens_per_gpu": 1, "skipped": "time budget"},
    ]
    rows = R.rows_from_secondary(line)
    assert len(rows) == 1                               # a skipped leg has no timing and makes no row
    r = rows[0]
    assert r["num_tokens"] == 128 and r["local_assignments"] == 128 * 8 and r["precision"] == "fp8"
    assert abs(r["latency_us"] - 1800.0) < 1e-9 and r["verify"] == "ok" and r["stage_us"]["gate_up_gemm"] == 1100.0
    assert "fp8" in R.format_table([R.rows_from_bench(line)] + rows)
