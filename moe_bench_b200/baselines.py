"""Reported GPU baselines (not part of the product path): the reference's own
implementations run through vLLM, when vLLM is installed on the box.

``vllm_compute_only`` is the reference's ``NaiveFusedExperts.run``
(baseline.py:62-76); ``vllm_serial_scheme`` is its ``SerialNaive`` scheme
(schemes.py:84-143): all-gather of tokens and routing, ``fused_experts`` with
the expert map, reduce-scatter.  Both return a zero-argument callable that runs
one step, or raise ``BaselineUnavailable`` with the reason.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class BaselineUnavailable(RuntimeError):
    pass


def _fused_experts():
    try:
        from vllm.model_executor.layers.fused_moe.fused_moe import fused_experts
    except Exception as exc:  # noqa: BLE001
        raise BaselineUnavailable(f"vLLM fused_experts not importable: {type(exc).__name__}: {exc}") from exc
    return fused_experts


def _quant_config(problem):
    qc = problem.quant_config
    if qc is None:
        return None
    try:
        from vllm.model_executor.layers.fused_moe.config import FusedMoEQuantConfig
    except Exception as exc:  # noqa: BLE001
        raise BaselineUnavailable(f"vLLM FusedMoEQuantConfig not importable: {exc}") from exc
    return FusedMoEQuantConfig.make(
        quant_dtype=torch.float8_e4m3fn, w1_scale=qc.w1_scale, w2_scale=qc.w2_scale,
        block_shape=list(qc.block_shape),
    )


def vllm_compute_only(problem):
    fused_experts = _fused_experts()
    qc = _quant_config(problem)
    ep = problem.config.parallel_mode.value == "ep"

    def run():
        return fused_experts(
            hidden_states=problem.hidden_states, w1=problem.w1, w2=problem.w2,
            topk_weights=problem.topk_weights, topk_ids=problem.topk_ids,
            global_num_experts=problem.config.num_experts,
            expert_map=problem.expert_map if ep else None, quant_config=qc,
        )

    return run


def vllm_serial_scheme(problem, world: int):
    fused_experts = _fused_experts()
    qc = _quant_config(problem)
    ep = problem.config.parallel_mode.value == "ep"
    t, k = problem.hidden_states.shape
    topk = problem.topk_ids.shape[1]
    dev = problem.hidden_states.device
    hidden_full = torch.empty(t * world, k, device=dev, dtype=problem.hidden_states.dtype)
    ids_full = torch.empty(t * world, topk, device=dev, dtype=problem.topk_ids.dtype)
    w_full = torch.empty(t * world, topk, device=dev, dtype=problem.topk_weights.dtype)
    out = torch.empty(t, k, device=dev, dtype=problem.hidden_states.dtype)

    def run():
        dist.all_gather_into_tensor(hidden_full, problem.hidden_states)
        dist.all_gather_into_tensor(ids_full, problem.topk_ids)
        dist.all_gather_into_tensor(w_full, problem.topk_weights)
        res = fused_experts(
            hidden_states=hidden_full, w1=problem.w1, w2=problem.w2, topk_weights=w_full, topk_ids=ids_full,
            global_num_experts=problem.config.num_experts,
            expert_map=problem.expert_map if ep else None, quant_config=qc,
        )
        dist.reduce_scatter_tensor(out, res)
        return out

    return run
