"""Host side of the gating front end: the logits generator (CPU tensors) against
the oracle's selection.  The kernel itself is covered by the GPU tests."""

import hashlib

import pytest
import torch

from moe_bench_b200 import capi
from moe_bench_b200 import gating as G
from moe_bench_b200 import problem as P
from oracle import moe_oracle as O


def _cfg(dist, **kw):
    base = dict(hidden_size=256, intermediate_size=128, num_experts=64, topk=4, world_size=1,
                routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=3, device="cpu")
    base.update(kw)
    return P.MoEBenchConfig(**base)


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("dist", ["single", "balanced"])
def test_deterministic_distributions_reproduce_the_reference_ids(dist):
    """single / balanced: the top-k of the logits is exactly data.py's id table,
    in its order (data.py:198-215)."""
    cfg = _cfg(dist, routing=P.RoutingConfig(distribution=P.Distribution(dist), num_active_experts=48))
    ids, w = O.route_topk(G.router_logits(cfg, 777), cfg.topk)
    ref_ids, _ = P._make_routing(cfg, 777, None)
    assert torch.equal(ids, ref_ids)
    torch.testing.assert_close(w.sum(dim=1), torch.ones(777))


def test_uniform_and_skewed_have_the_reference_law():
    """uniform: all active experts about equally loaded, inactive ones never;
    skewed: Zipf popularity like multinomial(p, k, replacement=False)."""
    cfg = _cfg("uniform", routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM, num_active_experts=48))
    ids, _ = O.route_topk(G.router_logits(cfg, 6000), cfg.topk)
    cnt = torch.bincount(ids.flatten().long(), minlength=64).float()
    assert int(cnt[48:].sum()) == 0
    assert float(cnt[:48].std() / cnt[:48].mean()) < 0.1
    assert all(len(set(r.tolist())) == cfg.topk for r in ids[:200])  # distinct per row

    cfg = _cfg("skewed")
    ids, _ = O.route_topk(G.router_logits(cfg, 6000), cfg.topk)
    got = torch.bincount(ids.flatten().long(), minlength=64).float()
    ref_ids, _ = P._make_routing(cfg, 6000, torch.Generator().manual_seed(0))
    ref = torch.bincount(ref_ids.flatten().long(), minlength=64).float()
    # same popularity curve as the reference's own draw, within sampling noise
    assert float((got - ref).abs().sum() / ref.sum()) < 0.06
    assert got[0] > got[7] > got[40]


def test_router_stream_is_separate_and_seeded():
    cfg = _cfg("uniform")
    a = G.router_logits(cfg, 100)
    assert _sha(a) == _sha(G.router_logits(cfg, 100))
    assert _sha(a) != _sha(G.router_logits(cfg, 100, input_rank=1))
    # drawing logits does not touch the input / weight streams of the reference generator
    before = P.make_problem(cfg, 100)
    G.router_logits(cfg, 100)
    after = P.make_problem(cfg, 100)
    assert _sha(before.hidden_states) == _sha(after.hidden_states) and _sha(before.w1) == _sha(after.w1)


def test_routed_problem_needs_a_gpu():
    with pytest.raises(capi.MB200Error, match="no CPU path"):
        G.make_routed_problem(_cfg("uniform"), 16)
