"""World-size-2 CPU (gloo) check of the distributed dataflow model against the
reference's distributed ground truth: the ring order, the partial-row
addressing and the owner masks, and the slot arithmetic of the push combine, that
the CUDA scheme uses, for EP and TP, bf16, fp16 and fp8."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, precision, out_q, combine=None):
    sys.path.insert(0, ROOT)
    from moe_bench_b200 import problem as P
    from oracle import dist_model as D
    from oracle import moe_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = P.MoEBenchConfig(
            hidden_size=256, intermediate_size=256, num_experts=8, topk=2, parallel_mode=P.ParallelMode(mode),
            world_size=world, precision=P.Precision(precision), distributed=True,
            routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM), seed=0, device="cpu",
        )
        prob = P.make_problem(cfg, 48, rank)
        got = D.forward_rank(prob, rank, world, combine=combine)
        ref = O.reference_moe(P.make_golden_problem(cfg, 48, rank))
        res = O.verify_output(precision, got, ref)
        out_q.put((rank, res.passed, res.rel_err, res.message))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,precision,combine", [
    ("ep", "bf16", "push"), ("ep", "bf16", "partial"), ("tp", "bf16", None), ("ep", "fp8", "push"),
    ("ep", "fp8", "partial"), ("tp", "fp8", None), ("ep", "fp16", "push"), ("tp", "fp16", None)])
def test_distributed_dataflow_model_world2(mode, precision, combine):
    world = 2
    port = 29500 + (os.getpid() + hash((mode, precision, combine))) % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, precision, q, combine)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, passed, rel, msg in sorted(results):
        assert passed, f"rank {rank}: {msg}"
        assert rel < 2e-2, (rank, rel)
