"""Turn ``bench.py`` JSON lines into the reference's result rows and a table.

    python -m moe_bench_b200.report run1.json [run2.json ...] [--json out.json]

The reference reports one row per token count with the keys ``num_tokens,
latency_us, tflops, local_assignments, timing, rel_err, verify`` and writes
``{"config", "implementation", "results"}`` (reference ``report.py:13-23,68-81``).
``rows_from_bench`` produces those keys from a line of this repository's
``bench.py`` and adds the columns the reference lacks: fraction of the layer
roofline, the dominant kernel's roofline entry, per-stage achieved GB/s or
TFLOP/s, the end-to-end number, and the vLLM and CPU baselines of the same run.
"""

from __future__ import annotations

import argparse
import json
from typing import Any, Dict, Iterable, List

_COLUMNS = [
    ("num_tokens", "tokens", "{:>7d}"),
    ("precision", "prec", "{:>5s}"),
    ("n_gpus", "gpus", "{:>4d}"),
    ("mode", "mode", "{:>6s}"),
    ("latency_us", "latency(us)", "{:>12.1f}"),
    ("tflops", "TFLOP/s", "{:>9.1f}"),
    ("roofline_frac", "of roofline", "{:>11.2f}"),
    ("e2e_tflops", "e2e TFLOP/s", "{:>11.1f}"),
    ("gemm1_frac", "gate/up frac", "{:>12.2f}"),
    ("sm_mhz_in_kernel", "MHz in kernel", "{:>13.0f}"),
    ("vllm_us", "vLLM(us)", "{:>10.1f}"),
    ("cpu_tflops", "CPU TFLOP/s", "{:>11.3f}"),
    ("rel_err", "rel_err", "{:>9.2e}"),
    ("verify", "verify", "{:>6s}"),
]


def rows_from_bench(line: Dict[str, Any]) -> Dict[str, Any]:
    """One reference-style result row (plus extension columns) from one bench line."""
    cfg = line.get("config", {})
    tokens = int(cfg.get("tokens_per_gpu", 0))
    row: Dict[str, Any] = {
        # the reference's keys
        "num_tokens": tokens,
        "latency_us": float(line["ms_per_step"]) * 1e3,
        "tflops": float(line["value"]),
        "local_assignments": tokens * int(cfg.get("topk", 0)),
        "timing": "events",
        "rel_err": line.get("rel_err"),
        "verify": line.get("verify", "n/a"),
        # extensions
        "precision": line.get("dtype", "?"),
        "n_gpus": int(line.get("n_gpus", 1)),
        "roofline_frac": line.get("layer_roofline_frac"),
        "e2e_tflops": (line.get("e2e") or {}).get("value"),
        "gemm1_frac": (line.get("roofline") or {}).get("frac"),
        "gemm1_bound": (line.get("roofline") or {}).get("bound"),
        "sm_mhz_in_kernel": ((line.get("clocks") or {}).get("in_kernel_sm_mhz") or {}).get("gate_up_gemm"),
        "vllm_us": None,
        "cpu_tflops": (line.get("cpu_baseline") or {}).get("value"),
        "cpu_cores": (line.get("cpu_baseline") or {}).get("cores"),
        "stage_us": {k: v * 1e3 for k, v in (line.get("stage_ms") or {}).items()},
        "stage_achieved": {},
    }
    base = line.get("gpu_baseline") or {}
    if "ms_per_step" in base:
        row["vllm_us"] = float(base["ms_per_step"]) * 1e3
    for name, st in (line.get("stage_roofline") or {}).items():
        unit = "TFLOP/s" if st.get("bound") == "tensor" else "GB/s"
        val = st.get("achieved_tflops") if unit == "TFLOP/s" else st.get("achieved_gbs")
        row["stage_achieved"][name] = {"value": val, "unit": unit, "frac": st.get("frac")}
    return row


def rows_from_secondary(line: Dict[str, Any]) -> List[Dict[str, Any]]:
    """Rows for the other sweep points a bench line carries under ``secondary``.

    The reference's sweep prints one row per token count (``bench.py:52-118``); a
    ``bench.py`` line of this repository holds the headline point at the top level
    and the remaining points (other token counts, fp8, tensor parallel) as a list.
    """
    cfg = line.get("config", {})
    topk = int(cfg.get("topk", 0))
    rows = []
    for leg in line.get("secondary") or []:
        if "ms" not in leg:
            continue
        tokens = int(leg.get("tokens_per_gpu", 0))
        rows.append({
            "num_tokens": tokens,
            "latency_us": float(leg["ms"]) * 1e3,
            "tflops": float(leg.get("tflops", 0.0)),
            "local_assignments": tokens * topk,
            "timing": "events",
            "rel_err": leg.get("rel_err"),
            "verify": leg.get("verify", "n/a"),
            "precision": leg.get("precision", "?"),
            "mode": leg.get("mode"),
            "n_gpus": int(line.get("n_gpus", 1)),
            "roofline_frac": leg.get("layer_roofline_frac"),
            "stage_us": {k: v * 1e3 for k, v in (leg.get("stage_ms") or {}).items()},
            "stage_achieved": {},
        })
    return rows


def format_table(rows: Iterable[Dict[str, Any]]) -> str:
    rows = list(rows)
    cols = [c for c in _COLUMNS if any(r.get(c[0]) is not None for r in rows)]
    widths = [max(len(t), len(fmt.format(0 if "d" in fmt or "f" in fmt or "e" in fmt else ""))) for _, t, fmt in cols]
    out = [" ".join(t.rjust(w) for (_, t, _), w in zip(cols, widths)), "-" * (sum(widths) + len(widths) - 1)]
    for r in rows:
        cells = []
        for (key, _, fmt), w in zip(cols, widths):
            v = r.get(key)
            cells.append(("-" if v is None else fmt.format(v)).rjust(w))
        out.append(" ".join(cells))
    return "\n".join(out)


def stage_table(row: Dict[str, Any]) -> str:
    out = [f"stages at {row['num_tokens']} tokens ({row['precision']}):"]
    for name, us in row["stage_us"].items():
        ach = row["stage_achieved"].get(name)
        tail = "" if not ach or ach["value"] is None else f"  {ach['value']:9.1f} {ach['unit']:7s} ({ach['frac']:.2f} of its roofline)"
        out.append(f"  {name:22s} {us:9.1f} us{tail}")
    return "\n".join(out)


def payload(rows: List[Dict[str, Any]], config: Dict[str, Any], implementation: str = "b200") -> Dict[str, Any]:
    """The reference's JSON shape (``report.py:68-81``)."""
    return {"config": config, "implementation": implementation, "results": rows}


def _load(path: str) -> Dict[str, Any]:
    with open(path, encoding="utf-8") as f:
        text = f.read().strip()
    return json.loads(text.splitlines()[-1] if text.count("\n") and not text.startswith("{\n") else text)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m moe_bench_b200.report")
    ap.add_argument("files", nargs="+", help="files holding one bench.py JSON line each")
    ap.add_argument("--json", help="also write the reference-shaped payload here")
    args = ap.parse_args(argv)
    lines = [_load(p) for p in args.files]
    rows = [rows_from_bench(l) for l in lines]
    headline = {id(r) for r in rows}
    for l, head in zip(lines, list(rows)):
        head["mode"] = (l.get("config") or {}).get("mode") or ("single" if head["n_gpus"] == 1 else None)
        same = lambda r: (r["num_tokens"], r["precision"], r.get("mode")) == (head["num_tokens"], head["precision"], head["mode"])
        rows.extend(r for r in rows_from_secondary(l) if not same(r))
    rows.sort(key=lambda r: (r["precision"], r["n_gpus"], r.get("mode") or "", r["num_tokens"]))
    print(format_table(rows))
    for r in rows:
        if r["stage_us"] and id(r) in headline:
            print()
            print(stage_table(r))
    if args.json:
        with open(args.json, "w", encoding="utf-8") as f:
            json.dump(payload(rows, lines[0].get("config", {})), f, indent=2)
        print(f"\nWrote {args.json}")


if __name__ == "__main__":
    main()
