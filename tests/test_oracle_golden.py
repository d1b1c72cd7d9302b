"""The CPU oracle and this package's input generator against fixtures produced
by the moe_bench reference itself (tests/golden/make_golden.py)."""

import hashlib

import numpy as np
import pytest
import torch

from moe_bench_b200 import problem as P
from oracle import moe_oracle as O


def _sha(t):
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _build(case):
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    name_rank = case.get("_rank", 0)
    return cfg, name_rank


CASES = {
    # name -> (builder, rank)
    "config1_uniform_bf16": ("problem", 0),
    "config1_balanced_bf16": ("problem", 0),
    "config1_single_bf16": ("problem", 0),
    "config1_skewed_bf16": ("problem", 0),
    "config1_uniform_fp16": ("problem", 0),
    "config1_ep2_rank1_bf16": ("problem", 1),
    "config1_uniform_bf16_T1": ("problem", 0),
    "config1_uniform_bf16_T7": ("problem", 0),
    "golden_tp2_rank1_bf16": ("golden", 1),
    "golden_ep2_rank1_bf16": ("golden", 1),
    "config1_uniform_fp8": ("problem", 0),
    "config1_ep2_rank0_fp8": ("problem", 0),
}


def _make(golden, name):
    case = golden["cases"][name]
    kind, rank = CASES[name]
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    fn = P.make_problem if kind == "problem" else P.make_golden_problem
    return case, fn(cfg, case["num_tokens"], rank)


@pytest.mark.parametrize("name", sorted(CASES))
def test_generator_is_byte_identical_to_reference(golden, name):
    case, prob = _make(golden, name)
    assert _sha(prob.hidden_states) == case["sha_hidden"]
    assert _sha(prob.w1) == case["sha_w1"]
    assert _sha(prob.w2) == case["sha_w2"]
    assert torch.equal(prob.topk_ids, case["topk_ids"])
    assert torch.equal(prob.topk_weights, case["topk_weights"])
    if case["expert_map"] is None:
        assert prob.expert_map is None
    else:
        assert torch.equal(prob.expert_map, case["expert_map"])
    assert prob.num_local_assignments == case["num_local_assignments"]
    if "sha_w1_scale" in case:
        assert _sha(prob.quant_config.w1_scale) == case["sha_w1_scale"]
        assert _sha(prob.quant_config.w2_scale) == case["sha_w2_scale"]


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_layer_matches_reference_output(golden, name):
    case, prob = _make(golden, name)
    torch.set_num_threads(1)
    out = O.reference_moe(prob)
    ref = case["reference"]
    # Same operations in a different grouping (per-expert gathers instead of
    # boolean masks): agreement to fp32 rounding, far inside any layer tolerance.
    torch.testing.assert_close(out, ref, atol=2e-5, rtol=1e-5)
    assert abs(float(out.norm()) - float(ref.norm())) < 1e-3


def test_known_answers_config1(golden):
    """Scalars recorded from the reference for the CPU plumbing case."""
    assert P._mix_seed(0, 0, 64, 0) == 64000192
    assert P._mix_seed(0, 1, 0, 0) == 1426103689
    case = golden["cases"]["config1_uniform_bf16"]
    assert case["topk_ids"][:3].tolist() == [[3, 0], [6, 4], [0, 2]]
    assert abs(float(case["reference"].norm()) - 53.66294860839844) < 1e-4
    assert abs(case["hidden_sum"] - (-8.89138412475586)) < 1e-4


@pytest.mark.parametrize("name", ["uniform_E8_T64", "single_E8_T64", "skewed_E64_T300", "uniform_E256_T5"])
def test_align_matches_reference_schedule(golden, name):
    g = golden["align"][name]
    ids = g["topk_ids"].numpy()
    e = g["config"]["num_experts"]
    k = ids.shape[1]
    counts, offsets, sorted_ids, inverse = O.align(ids, None, e, g["row_block"])
    assert np.array_equal(inverse, g["assignment_slot"].numpy())
    assert np.array_equal((offsets[1:] - offsets[:-1]), g["padded_per_expert"].numpy())
    tok = np.where(sorted_ids >= 0, sorted_ids // k, -1)
    assert np.array_equal(tok, g["slot_src_tok"].numpy())


def test_align_with_expert_map_and_empty_experts():
    ids = np.array([[0, 5], [5, 6], [7, 1]], dtype=np.int32)
    emap = np.array([-1, -1, -1, -1, 0, 1, 2, 3], dtype=np.int32)
    counts, offsets, sorted_ids, inverse = O.align(ids, emap, 4, 4)
    assert counts.tolist() == [0, 2, 1, 1]
    assert offsets.tolist() == [0, 0, 4, 8, 12]
    assert sorted_ids.tolist() == [1, 2, -1, -1, 3, -1, -1, -1, 4, -1, -1, -1]
    assert inverse.tolist() == [-1, 0, 1, 4, 8, -1]


def test_group_quant_properties():
    torch.manual_seed(1)
    x = torch.randn(5, 256, dtype=torch.bfloat16)
    x[0, :128] = 0  # all-zero group: scale floors at eps/448, q = 0
    q, s = O.group_quant_fp8(x, 128)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (5, 2)
    assert torch.all(q[0, :128].float() == 0)
    deq = q.float().view(5, 2, 128) * s.unsqueeze(-1)
    err = (deq.view(5, 256) - x.float()).abs()
    assert float(err.max()) <= float(x.float().abs().max()) / 16 + 1e-6
    # the element holding the group's amax maps to +-448 exactly
    assert float(q.float().abs().view(5, 2, 128).amax(-1)[1:].min()) == 448.0


def test_route_topk_oracle():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(17, 32, generator=g)
    ids, w = O.route_topk(logits, 4)
    ref = torch.topk(torch.softmax(logits, -1), 4)
    assert torch.equal(ids.long(), ref.indices)
    torch.testing.assert_close(w.sum(-1), torch.ones(17))
    # ties: lowest expert index first
    ids, _ = O.route_topk(torch.zeros(2, 8), 3)
    assert ids.tolist() == [[0, 1, 2], [0, 1, 2]]
