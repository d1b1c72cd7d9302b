"""CPU model of the distributed dataflow (expert parallel and tensor parallel).
TEST INFRASTRUCTURE ONLY.

It restates, with torch CPU ops and ``torch.distributed`` (gloo) exchanges in
place of peer-memory loads, what each rank of the CUDA scheme does: stage its
tokens and routing, read every rank's routing in ring order (own rank first),
compute its experts' share for the tokens routed to it, pre-reduce the
contributions of each token into one row, and let each token's own rank sum the
rows of the ranks that hold one.  It is checked against the reference's own
distributed ground truth, ``reference_moe(make_golden_problem(...))``
(reference distributed.py:64-84), so the index arithmetic of the scheme (ring
order, partial-row addressing, owner masks) is pinned without a GPU.
"""

from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from . import moe_oracle as O


def forward_rank(problem, rank: int, world: int, group=None) -> torch.Tensor:
    """This rank's ``(T, K)`` output of the distributed layer, fp32."""
    cfg = problem.config
    ep = cfg.parallel_mode.value == "ep"
    t, hidden = problem.hidden_states.shape
    topk = problem.topk_ids.shape[1]

    # "symmetric buffers": every rank can read every rank's staged data
    staged = [None] * world
    dist.all_gather_object(staged, (problem.hidden_states, problem.topk_ids, problem.topk_weights), group=group)

    # ring order: own rank first, then rank+1, ...
    order = [(rank + i) % world for i in range(world)]
    x_all = torch.cat([staged[s][0] for s in order])
    ids_all = torch.cat([staged[s][1] for s in order])
    w_all = torch.cat([staged[s][2] for s in order])

    local = dataclasses.replace(
        problem, num_tokens=world * t, hidden_states=x_all, topk_ids=ids_all, topk_weights=w_all,
        expert_map=problem.expert_map if ep else None,
    )
    # per-token row holding this rank's weighted contributions, rounded to bf16 like the wire format
    partial = O.reference_moe(local).to(torch.bfloat16)

    partials = [None] * world
    dist.all_gather_object(partials, partial, group=group)

    out = torch.zeros(t, hidden, dtype=torch.float32)
    e_local = cfg.num_experts // world if ep else 0
    for p in range(world):
        ring = (rank - p + world) % world           # where this rank's tokens sit on rank p
        rows = partials[p][ring * t : (ring + 1) * t].float()
        if ep:
            owns = ((problem.topk_ids // e_local) == p).any(dim=1)
            rows = rows * owns.unsqueeze(-1)
        out += rows
    return out
