"""Generate the golden fixtures in this directory from the moe_bench reference.

Run where the reference package is importable as ``reference`` from its parent
directory (it needs torch and vLLM; CPU only is enough):

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py --ref-parent <dir holding reference/>

It writes ``golden.pt`` next to this file: for each case the SHA-256 of every
input tensor the reference generated (so this package's own generator can be
checked byte for byte without shipping the weights), the routing tensors, and
the reference's outputs (``reference_moe``; the slot tables of the reference's
host schedule builder for the sort-and-pad stage).

The fp8 case needs one substitution: the reference's activation quantiser is a
vLLM CUDA/Triton op that does not run on a CPU, so it is replaced, for this
script only, by ``oracle.moe_oracle.group_quant_fp8``.  The fixture therefore
pins everything around the quantiser (block matmul order, SiLU-mul, bf16
round, combine, weight quantisation) but not the quantiser itself.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def sha(t: torch.Tensor) -> str:
    raw = t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-parent", required=True, help="directory that contains the reference/ package")
    args = ap.parse_args()
    sys.path.insert(0, args.ref_parent)
    sys.path.insert(0, ROOT)

    from reference.config import Distribution, MoEBenchConfig, ParallelMode, Precision, RoutingConfig
    from reference.data import make_golden_problem, make_problem
    from reference import data as rdata
    from reference import reference as rref

    from oracle.moe_oracle import group_quant_fp8

    torch.set_num_threads(1)  # one thread: fp32 sums do not depend on the pool size
    out: dict = {"cases": {}}

    def record(name, problem, extra=None):
        ref = rref.reference_moe(problem)
        case = {
            "config": problem.config.to_dict(),
            "num_tokens": problem.num_tokens,
            "sha_hidden": sha(problem.hidden_states),
            "sha_w1": sha(problem.w1),
            "sha_w2": sha(problem.w2),
            "topk_ids": problem.topk_ids.clone(),
            "topk_weights": problem.topk_weights.clone(),
            "expert_map": None if problem.expert_map is None else problem.expert_map.clone(),
            "num_local_assignments": problem.num_local_assignments,
            "reference": ref.clone(),
            "hidden_sum": float(problem.hidden_states.float().sum()),
            "w1_sum": float(problem.w1.float().sum()),
        }
        if problem.quant_config is not None:
            case["sha_w1_scale"] = sha(problem.quant_config.w1_scale)
            case["sha_w2_scale"] = sha(problem.quant_config.w2_scale)
        if extra:
            case.update(extra)
        out["cases"][name] = case
        print(name, "||ref||=%.6f sum=%.6f" % (float(ref.norm()), float(ref.sum())))

    def cfg(dist, mode=ParallelMode.TP, world=1, prec=Precision.BF16, **kw):
        base = dict(
            hidden_size=256, intermediate_size=128, num_experts=8, topk=2,
            parallel_mode=mode, world_size=world, precision=prec, num_tokens=[64],
            routing=RoutingConfig(distribution=dist), seed=0, device="cpu",
        )
        base.update(kw)
        return MoEBenchConfig(**base)

    # config 1 (CPU plumbing case) under the three id-generating branches
    for dist in (Distribution.UNIFORM, Distribution.BALANCED, Distribution.SINGLE):
        record(f"config1_{dist.value}_bf16", make_problem(cfg(dist), 64))
    record("config1_skewed_bf16", make_problem(cfg(Distribution.SKEWED), 64))
    record("config1_uniform_fp16", make_problem(cfg(Distribution.UNIFORM, prec=Precision.FP16), 64))
    # EP: rank 1 of 2 (expert_map masks half of the experts)
    record("config1_ep2_rank1_bf16", make_problem(cfg(Distribution.UNIFORM, ParallelMode.EP, 2), 64, rank=1))
    # ragged token counts, including a single token
    for t in (1, 7):
        record(f"config1_uniform_bf16_T{t}", make_problem(cfg(Distribution.UNIFORM), t))
    # distributed golden problems: TP shards concatenated, EP all experts
    c = cfg(Distribution.UNIFORM, ParallelMode.TP, 2, distributed=True)
    record("golden_tp2_rank1_bf16", make_golden_problem(c, 64, 1))
    c = cfg(Distribution.UNIFORM, ParallelMode.EP, 2, distributed=True)
    record("golden_ep2_rank1_bf16", make_golden_problem(c, 64, 1))

    # fp8 (activation quantiser substituted, see module docstring)
    import vllm.model_executor.layers.fused_moe.utils as fmu

    def _quant(a, a_scale, quant_dtype, per_act_token_quant, block_shape):
        assert a_scale is None and not per_act_token_quant
        return group_quant_fp8(a, block_shape[1])

    fmu.moe_kernel_quantize_input = _quant
    record("config1_uniform_fp8", make_problem(cfg(Distribution.UNIFORM, prec=Precision.FP8), 64))
    record(
        "config1_ep2_rank0_fp8",
        make_problem(cfg(Distribution.UNIFORM, ParallelMode.EP, 2, prec=Precision.FP8), 64, rank=0),
    )

    # sort-and-pad: slot tables of the reference's host schedule builder, W = 1
    # The builder gathers every rank's ids with a collective; for one rank that
    # gather is a copy, so it is stubbed instead of starting a process group.
    import torch.distributed as dist

    from reference import tk_scheme

    dist.all_gather_into_tensor = lambda dst, src, **kw: dst.copy_(src.view_as(dst))

    out["align"] = {}
    for name, dcfg, t in (
        ("uniform_E8_T64", cfg(Distribution.UNIFORM), 64),
        ("single_E8_T64", cfg(Distribution.SINGLE), 64),
        ("skewed_E64_T300", cfg(Distribution.SKEWED, num_experts=64, topk=8), 300),
        ("uniform_E256_T5", cfg(Distribution.UNIFORM, num_experts=256, topk=8), 5),
    ):
        p = make_problem(dcfg, t)
        res = tk_scheme._build_schedules(
            p.topk_ids, t, 1, dcfg.num_experts, dcfg.num_experts, 0, "cpu"
        )
        disp_idx, comb_idx, padded = res[0], res[1], res[2]
        out["align"][name] = {
            "config": dcfg.to_dict(),
            "num_tokens": t,
            "row_block": tk_scheme.ROW_BLOCK,
            "topk_ids": p.topk_ids.clone(),
            "slot_src_tok": disp_idx[:, 1].clone(),      # token in each padded row, -1 = pad
            "assignment_slot": comb_idx[:, 1].clone(),   # row of flat assignment t*k+kpos
            "padded_per_expert": padded.clone(),
        }
        print("align", name, "rows", disp_idx.shape[0])

    torch.save(out, os.path.join(HERE, "golden.pt"))
    print("wrote", os.path.join(HERE, "golden.pt"))


if __name__ == "__main__":
    main()
