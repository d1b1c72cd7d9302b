"""Gating front end on the GPU: logits -> mb200_route_topk -> MoEProblem -> layer."""

import dataclasses

import pytest
import torch

from moe_bench_b200 import gating as G
from moe_bench_b200 import problem as P
from moe_bench_b200.plugin import get_implementation
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dist", ["uniform", "skewed", "single", "balanced"])
def test_routed_problem_matches_oracle_selection_and_layer(dist):
    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=64, topk=8, world_size=1,
                           routing=P.RoutingConfig(distribution=P.Distribution(dist), num_active_experts=40),
                           seed=4, device=DEV)
    prob, logits = G.make_routed_problem(cfg, 300)
    o_ids, o_w = O.route_topk(logits.cpu(), cfg.topk)
    assert torch.equal(prob.topk_ids.cpu(), o_ids)          # bit-exact selection and order
    torch.testing.assert_close(prob.topk_weights.cpu(), o_w, atol=1e-6, rtol=2e-5)
    assert int(prob.topk_ids.max()) < 40
    if dist in ("single", "balanced"):
        ref_ids, _ = P._make_routing(dataclasses.replace(cfg, device="cpu"), 300, None)
        assert torch.equal(prob.topk_ids.cpu(), ref_ids)
    impl = get_implementation("b200")
    impl.setup(prob)
    out = impl.run(prob)
    assert impl.device_status() == 0
    res = O.verify_output("bf16", out, O.reference_moe(prob))
    assert res.passed and res.rel_err < 1e-2, (res.message, res.rel_err)


def test_front_end_at_full_size():
    cfg = P.deepseek_v32_config(device=DEV)
    logits = G.router_logits(cfg, 8192)
    assert logits.shape == (8192, 256)
    from moe_bench_b200 import capi

    ids, w = capi.route_topk(logits, 8)
    o_ids, _ = O.route_topk(logits.cpu(), 8)
    assert torch.equal(ids.cpu(), o_ids)
    torch.testing.assert_close(w.sum(dim=1).cpu(), torch.ones(8192), atol=1e-5, rtol=0)
