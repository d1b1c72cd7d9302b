"""Gating front end: router logits -> softmax -> top-k -> renormalised weights,
wired into problem creation.

The reference has no router: ``data.py:178-235`` draws ``topk_ids`` directly
(constant for ``single``, round-robin for ``balanced``, ``multinomial`` without
replacement for ``uniform`` / ``skewed``) and ``topk_weights = softmax(rand)``.
This module supplies the stage in front of it: logits over all experts whose
top-k reproduces each of those distributions, drawn from a generator stream of
their own (tag 2; ``data.py`` uses 0 for inputs and 1 for weights), so the
hidden states and weights of a problem stay byte-identical to the reference's,
and ``mb200_route_topk`` turns them into the routing tensors of a
``MoEProblem``.  There is no CPU path for the selection itself; the CPU oracle
(``oracle.moe_oracle.route_topk``) is the checker in the tests.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import torch

from . import capi
from .problem import Distribution, MoEBenchConfig, MoEProblem, MoEWeights, _input_rank, _make_routing, _mix_seed, make_problem

_STREAM_ROUTER = 2
_LOSER = -30000.0  # exp() of it is 0 in fp32: an expert that must never be selected


def router_logits(config: MoEBenchConfig, num_tokens: int, input_rank: int = 0) -> torch.Tensor:
    """fp32 ``[T, E]`` logits on ``config.device`` for the configured distribution.

    uniform   N(0,1) over the active experts: every k-subset equally likely.
    skewed    log p_e + Gumbel(0,1), p_e ~ (e+1)^-alpha: top-k of that is a draw
              without replacement with probabilities p (the Gumbel-top-k identity),
              the law of ``torch.multinomial(p, k, replacement=False)``
              (``data.py:216-228``).
    single    experts 0..k-1 win for every token, in that order (``data.py:198-206``).
    balanced  the reference's round-robin ids win, in its order (``data.py:207-215``).
    Experts beyond ``routing.num_active_experts`` never win.
    """
    dev, e, k = config.device, config.num_experts, config.topk
    active = config.routing.num_active_experts
    active = e if active is None else min(active, e)
    gen = torch.Generator(device=dev)
    gen.manual_seed(_mix_seed(config.seed, _STREAM_ROUTER, num_tokens, input_rank))
    dist = config.routing.distribution
    noise = torch.randn(num_tokens, e, device=dev, dtype=torch.float32, generator=gen)
    if dist in (Distribution.SINGLE, Distribution.BALANCED):
        ids, _ = _make_routing(config, num_tokens, None)  # both are deterministic: no generator draw
        logits = noise * 0.01 + _LOSER
        win = torch.arange(k, 0, -1, device=dev, dtype=torch.float32).expand(num_tokens, k)
        logits.scatter_(1, ids.long(), win.contiguous())
        return logits
    if dist == Distribution.SKEWED:
        u = torch.rand(num_tokens, e, device=dev, dtype=torch.float32, generator=gen).clamp_(1e-20, 1.0 - 1e-7)
        gumbel = -torch.log(-torch.log(u))
        logp = -config.routing.skew_alpha * torch.log(torch.arange(1, e + 1, device=dev, dtype=torch.float32))
        logits = gumbel + logp
    else:
        logits = noise
    if active < e:
        logits[:, active:] = _LOSER
    return logits


def make_routed_problem(
    config: MoEBenchConfig, num_tokens: int, rank: int = 0, weights: Optional[MoEWeights] = None
) -> Tuple[MoEProblem, torch.Tensor]:
    """``make_problem`` whose routing comes from the gating kernel instead of
    ``data.py``'s direct draw.  Returns the problem and the logits it was routed
    from.  Hidden states and weights are the reference's for the same seed."""
    prob = make_problem(config, num_tokens, rank, weights)
    logits = router_logits(config, num_tokens, _input_rank(config, rank))
    if not logits.is_cuda:
        raise capi.MB200Error("the gating kernel needs config.device to be a CUDA device; there is no CPU path")
    ids, wts = capi.route_topk(logits, config.topk)
    return dataclasses.replace(prob, topk_ids=ids, topk_weights=wts), logits
