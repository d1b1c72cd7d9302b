"""Child program of ``test_gpu_reference_harness.py``: the reference's OWN distributed
harness (``run_distributed`` → ``mp.spawn`` → ``_worker`` → ``_time_scheme`` /
``_verify_rank``, distributed.py:36-222) driving ``--scheme b200``.

    python tests/reference_distributed_child.py <repo root> <staged parent> <precision> <mode> <world> <out.json>

The registration sits at module level on purpose: ``mp.spawn`` re-imports this file in
every worker (as ``__mp_main__``), and ``get_scheme`` must find the scheme there
(distributed.py:99)."""

import dataclasses
import os
import sys

root, staged = sys.argv[1], sys.argv[2]
sys.path.insert(0, root)
sys.path.insert(0, staged)

import moe_bench_b200.register as R  # noqa: E402

R.register("moe_bench")

if __name__ == "__main__":
    from moe_bench.config import MoEBenchConfig, ParallelMode, Precision
    from moe_bench.distributed import run_distributed

    precision, mode, world, out = sys.argv[3], sys.argv[4], int(sys.argv[5]), sys.argv[6]
    cfg = MoEBenchConfig.from_file(os.path.join(staged, "moe_bench", "configs", "deepseek_v32.yaml"))
    cfg = dataclasses.replace(cfg, world_size=world, parallel_mode=ParallelMode(mode), precision=Precision(precision),
                              distributed=True, num_tokens=[128, 1024], warmup_iters=3, bench_iters=5,
                              output_json=out)
    run_distributed(cfg, "b200")
