"""The plugin under the reference's OWN harness, on the GPU: its input generator, its
CUDA-graph timing loop (10 calls per graph, bench.py:52-101), its ground truth and its
verify columns (bench.py:104-153, reference.py:207-250), with this library registered
as ``--impl b200``.  Needs the reference package staged by ``oracle/stage_reference.py``
(``python __graft_entry__.py`` does it where the checkout is present); skipped otherwise.
Runs in a child process: the reference switches torch's default device and imports vLLM."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r"""
import dataclasses, json, os, sys
root, staged, precision = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path.insert(0, root); sys.path.insert(0, staged)
import torch
import moe_bench_b200.register as R
regs = R.register("moe_bench")
from moe_bench.baseline import get_implementation
from moe_bench.bench import run_sweep
from moe_bench.config import MoEBenchConfig, ParallelMode, Precision
cfg = MoEBenchConfig.from_file(os.path.join(staged, "moe_bench", "configs", "deepseek_v32.yaml"))
cfg = dataclasses.replace(cfg, world_size=1, parallel_mode=ParallelMode.TP, precision=Precision(precision),
                          num_tokens=[128, 2048], warmup_iters=3, bench_iters=5, device="cuda:0")
torch.set_default_device(cfg.device)
impl = get_implementation("b200")
rows = run_sweep(cfg, impl)
print("ROWS " + json.dumps(rows))
"""


def _staged_parent():
    sys.path.insert(0, ROOT)
    from oracle.stage_reference import staged_parent

    return staged_parent()


@pytest.mark.parametrize("precision", ["bf16", "fp8"])
def test_reference_run_sweep_times_and_verifies_the_plugin(precision):
    staged = _staged_parent()
    if staged is None:
        pytest.skip("reference package not staged (oracle/stage_reference.py)")
    env = dict(os.environ, TORCHDYNAMO_DISABLE="1")
    res = subprocess.run([sys.executable, "-c", _CHILD, ROOT, staged, precision], capture_output=True, text=True,
                         timeout=1500, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("ROWS ")][-1]
    rows = json.loads(line[5:])
    assert [r["num_tokens"] for r in rows] == [128, 2048]
    for r in rows:
        # the reference captured ten forwards of this library in one CUDA graph and replayed it
        assert r["timing"] == "graph", r
        assert r["verify"] == "ok", r
        assert r["latency_us"] > 0 and r["tflops"] > 0 and r["local_assignments"] == r["num_tokens"] * 8


@pytest.mark.parametrize("precision,mode", [("fp8", "ep"), ("bf16", "ep"), ("bf16", "tp")])
def test_reference_run_distributed_times_and_verifies_the_scheme(precision, mode, tmp_path):
    """Two GPUs: the reference spawns its own workers, builds each rank's problem with
    its own generator, times ``scheme.run`` with its own loop and checks every rank's
    output against its full-model ground truth (distributed.py:36-84)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    staged = _staged_parent()
    if staged is None:
        pytest.skip("reference package not staged (oracle/stage_reference.py)")
    out = tmp_path / "rows.json"
    env = dict(os.environ, TORCHDYNAMO_DISABLE="1", LOCALHOST="127.0.0.1", NCCL_NVLS_ENABLE="0")
    child = os.path.join(ROOT, "tests", "reference_distributed_child.py")
    res = subprocess.run([sys.executable, child, ROOT, staged, precision, mode, "2", str(out)],
                         capture_output=True, text=True, timeout=1500, env=env)
    assert res.returncode == 0, (res.stdout[-1500:], res.stderr[-3000:])
    payload = json.load(open(out))
    rows = payload["results"]
    assert [r["num_tokens"] for r in rows] == [128, 1024]
    for r in rows:
        assert r["verify"] == "ok" and r["latency_us"] > 0, r
