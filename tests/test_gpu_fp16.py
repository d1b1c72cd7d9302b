"""fp16 precision (reference config.py:54, 212-213) through the plugin: the
bf16 data flow with IEEE-half tensors.  Tolerance: the reference's fp16 check,
atol 1e-2, rtol 0 (reference.py:41), plus a bound on the relative L2 error.
"""

import dataclasses

import pytest
import torch

from moe_bench_b200 import capi
from moe_bench_b200 import problem as P
from moe_bench_b200.plugin import get_implementation
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _to_dev(prob):
    def mv(t):
        return None if t is None else t.to(DEV)

    return dataclasses.replace(
        prob, hidden_states=mv(prob.hidden_states), w1=mv(prob.w1), w2=mv(prob.w2),
        topk_ids=mv(prob.topk_ids), topk_weights=mv(prob.topk_weights), expert_map=mv(prob.expert_map),
    )


def _run(prob):
    impl = get_implementation("b200")
    impl.setup(prob)
    out = impl.run(prob)
    assert impl.device_status() == 0
    assert out.shape == prob.hidden_states.shape and out.dtype == torch.float16
    return impl, out


def _check(out, ref):
    res = O.verify_output("fp16", out, ref)  # atol 1e-2, rtol 0
    assert res.passed, res.message
    # half keeps 11 significand bits against bf16's 8: the relative error is ~8x smaller
    assert res.rel_err < 2e-3, res.rel_err


def test_fp16_layer_matches_reference_output(golden):
    case = golden["cases"]["config1_uniform_fp16"]
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    prob = P.make_problem(cfg, case["num_tokens"], 0)
    assert prob.w1.dtype == torch.float16
    _, out = _run(_to_dev(prob))
    _check(out, case["reference"])


@pytest.mark.parametrize(
    "tokens,hidden,inter,experts,topk,dist,world",
    [
        (1, 512, 256, 16, 4, "uniform", 1),
        (129, 512, 256, 16, 4, "uniform", 1),
        (1000, 1024, 512, 32, 8, "skewed", 1),
        (513, 768, 384, 8, 2, "single", 1),
        (300, 512, 256, 16, 4, "uniform", 2),   # expert parallel: rank 1 of 2, non-local experts skipped
    ],
)
def test_fp16_layer_matches_oracle(tokens, hidden, inter, experts, topk, dist, world):
    cfg = P.MoEBenchConfig(
        hidden_size=hidden, intermediate_size=inter, num_experts=experts, topk=topk, world_size=world,
        parallel_mode=P.ParallelMode.EP, precision=P.Precision.FP16,
        routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=9, device="cpu",
    )
    prob = P.make_problem(cfg, tokens, world - 1)
    _, out = _run(_to_dev(prob))
    _check(out, O.reference_moe(prob))


def test_fp16_and_bf16_runs_differ_only_by_rounding():
    """The same values run at both 16-bit precisions (inputs representable in
    both: bf16 values with small exponents convert to half exactly) agree to
    bf16 rounding; the fp16 run is the closer one to the fp32 oracle."""
    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=16, topk=4, world_size=1,
                           routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM), seed=2, device="cpu")
    prob = P.make_problem(cfg, 256)
    # bf16 values below 2^-16 need more bits than half's subnormals have: flush them in both runs
    flush = lambda t: torch.where(t.float().abs() < 2.0 ** -16, torch.zeros_like(t), t)  # noqa: E731
    prob = dataclasses.replace(prob, hidden_states=flush(prob.hidden_states), w1=flush(prob.w1), w2=flush(prob.w2))
    as_half = dataclasses.replace(
        prob, config=dataclasses.replace(cfg, precision=P.Precision.FP16),
        hidden_states=prob.hidden_states.half(), w1=prob.w1.half(), w2=prob.w2.half(),
    )
    # the conversion lost nothing
    assert torch.equal(as_half.w1.float(), prob.w1.float()) and torch.equal(as_half.hidden_states.float(), prob.hidden_states.float())
    ref = O.reference_moe(prob)
    _, out16 = _run(_to_dev(as_half))
    impl = get_implementation("b200")
    impl.setup(_to_dev(prob))
    outbf = impl.run(_to_dev(prob))
    e16 = (out16.cpu().float() - ref).norm() / ref.norm()
    ebf = (outbf.cpu().float() - ref).norm() / ref.norm()
    assert e16 < ebf and e16 < 1e-3, (float(e16), float(ebf))


def test_mixed_dtypes_are_rejected():
    x = torch.zeros(4, 256, dtype=torch.float16, device=DEV)
    w1 = torch.zeros(2, 256, 256, dtype=torch.bfloat16, device=DEV)
    w2 = torch.zeros(2, 256, 128, dtype=torch.bfloat16, device=DEV)
    ids = torch.zeros(4, 1, dtype=torch.int32, device=DEV)
    wts = torch.ones(4, 1, device=DEV)
    out = torch.empty_like(x)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    with pytest.raises(capi.MB200Error, match="all be bf16 or all fp16"):
        capi.moe_forward_bf16(x, w1, w2, ids, wts, None, out, ws)
