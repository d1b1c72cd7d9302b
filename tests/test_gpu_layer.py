"""Layer-level GPU parity through the plugin (``MoEImplementation.setup/run``):
against the reference's own outputs (golden fixtures), against the CPU oracle on
seeded inputs, and through size-independent properties at the full
DeepSeek-V3.2 sizes.  Tolerance: the reference's bf16 check, atol 2e-2, rtol 0
(reference.py:39-43), plus a bound on the relative L2 error.
"""

import dataclasses

import pytest
import torch

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
    assert out.shape == prob.hidden_states.shape and out.dtype == torch.bfloat16
    return impl, out


def _check(out, ref, max_rel=1e-2):
    res = O.verify_output("bf16", out, ref)
    assert res.passed, res.message
    assert res.rel_err < max_rel, res.rel_err
    return res


GOLDEN_BF16 = [
    ("config1_uniform_bf16", "problem", 0),
    ("config1_balanced_bf16", "problem", 0),
    ("config1_single_bf16", "problem", 0),
    ("config1_skewed_bf16", "problem", 0),
    ("config1_ep2_rank1_bf16", "problem", 1),
    ("config1_uniform_bf16_T1", "problem", 0),
    ("config1_uniform_bf16_T7", "problem", 0),
    ("golden_tp2_rank1_bf16", "golden", 1),
    ("golden_ep2_rank1_bf16", "golden", 1),
]


@pytest.mark.parametrize("name,kind,rank", GOLDEN_BF16)
def test_layer_matches_reference_outputs(golden, name, kind, rank):
    """Inputs regenerated on the CPU (byte-identical to the reference's, see
    the CPU tests), run on the GPU, compared with the reference's own output."""
    case = golden["cases"][name]
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    make = P.make_problem if kind == "problem" else P.make_golden_problem
    prob = make(cfg, case["num_tokens"], rank)
    _, out = _run(_to_dev(prob))
    _check(out, case["reference"])


def test_tokens_without_local_expert_are_zero(golden):
    case = golden["cases"]["config1_ep2_rank1_bf16"]
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    prob = P.make_problem(cfg, case["num_tokens"], 1)
    _, out = _run(_to_dev(prob))
    local = (prob.expert_map[prob.topk_ids.long()] >= 0).any(dim=1)
    assert (~local).any()
    assert bool((out.cpu()[~local] == 0).all())


@pytest.mark.parametrize(
    "tokens,hidden,inter,experts,topk,dist",
    [
        (1, 512, 256, 16, 4, "uniform"),
        (129, 512, 256, 16, 4, "uniform"),
        (1000, 1024, 512, 32, 8, "skewed"),
        (513, 768, 384, 8, 2, "single"),
        (4096, 256, 128, 64, 8, "balanced"),
    ],
)
def test_layer_matches_oracle_on_seeded_inputs(tokens, hidden, inter, experts, topk, dist):
    cfg = P.MoEBenchConfig(
        hidden_size=hidden, intermediate_size=inter, num_experts=experts, topk=topk, world_size=1,
        routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=5, device="cpu",
    )
    prob = P.make_problem(cfg, tokens)
    _, out = _run(_to_dev(prob))
    _check(out, O.reference_moe(prob))


def test_run_is_repeatable_and_side_effect_free():
    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=16, topk=4, world_size=1,
                           routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM), device="cpu")
    prob = _to_dev(P.make_problem(cfg, 300))
    snap = [t.clone() for t in (prob.hidden_states, prob.w1, prob.w2, prob.topk_ids, prob.topk_weights)]
    impl, out = _run(prob)
    first = out.clone()
    for _ in range(5):
        again = impl.run(prob)
    torch.cuda.synchronize()
    assert torch.equal(first, again)  # deterministic: no atomics on the data path
    for a, b in zip(snap, (prob.hidden_states, prob.w1, prob.w2, prob.topk_ids, prob.topk_weights)):
        assert torch.equal(a, b)


def test_run_under_cuda_graph():
    """The harness captures 10 calls in one graph (reference bench.py:69-75)."""
    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=16, topk=4, world_size=1,
                           routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM), device="cpu")
    prob = _to_dev(P.make_problem(cfg, 200))
    impl, out = _run(prob)
    eager = out.clone()
    out.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(10):
            captured = impl.run(prob)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    assert impl.device_status() == 0


# ---------------------------------------------------------------------------
# DeepSeek-V3.2 shape (hidden 7168, intermediate 2048, 256 experts, top-8)
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dsv32():
    cfg = P.deepseek_v32_config(device=DEV)
    return cfg, P.make_weights(cfg)


def _subset(prob, idx):
    return dataclasses.replace(
        prob, num_tokens=len(idx), hidden_states=prob.hidden_states[idx].contiguous(),
        topk_ids=prob.topk_ids[idx].contiguous(), topk_weights=prob.topk_weights[idx].contiguous(),
    )


@pytest.mark.parametrize("tokens", [1, 8, 128])
def test_dsv32_small_token_counts_against_oracle(dsv32, tokens):
    cfg, weights = dsv32
    prob = P.make_problem(cfg, tokens, weights=weights)
    _, out = _run(prob)
    idx = torch.arange(tokens) if tokens <= 8 else torch.randperm(tokens, generator=torch.Generator().manual_seed(0))[:16]
    ref = O.reference_moe(_subset(prob, idx.to(DEV)))
    _check(out[idx.to(DEV)], ref)


@pytest.mark.parametrize("tokens", [2048, 8192])
def test_dsv32_full_size_properties(dsv32, tokens):
    """At the full sweep sizes the oracle is too slow for every token, so:
    (a) 16 sampled tokens are checked against the oracle, (b) the same tokens
    run alone through the plugin must reproduce their rows of the big run (a
    token's output depends on no other token), (c) outputs are finite."""
    cfg, weights = dsv32
    prob = P.make_problem(cfg, tokens, weights=weights)
    impl, out = _run(prob)
    big = out.clone()
    assert bool(torch.isfinite(big.float()).all())
    idx = torch.randperm(tokens, generator=torch.Generator().manual_seed(1))[:16].to(DEV)
    sub = _subset(prob, idx)
    _check(big[idx], O.reference_moe(sub))
    _, small = _run(sub)
    res = O.verify_output("bf16", small, big[idx].float(), atol=4e-3)
    assert res.passed and res.rel_err < 1e-3, (res.message, res.rel_err)
