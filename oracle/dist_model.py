"""CPU model of the distributed dataflow (expert parallel and tensor parallel).
TEST INFRASTRUCTURE ONLY.

It restates, with torch CPU ops and ``torch.distributed`` (gloo) exchanges in
place of peer-memory loads, what each rank of the CUDA scheme does: stage its
tokens and routing, read every rank's routing in ring order (own rank first),
compute its experts' share for the tokens routed to it, and then either
(``combine="partial"``: tensor parallel, and expert parallel with few rows per
expert in fp8) pre-reduce the contributions of each token into one row and let
each token's own rank sum the rows of the ranks that hold one, or
(``combine="push"``: expert parallel otherwise) send every weighted assignment
row ``n = (ring*T + t)*k + j`` to rank ``(rank + ring) mod W`` at slot
``n - ring*T*k`` and let that rank sum the k rows of each of its tokens.  It is
checked against the reference's own
distributed ground truth, ``reference_moe(make_golden_problem(...))``
(reference distributed.py:64-84), so the index arithmetic of the scheme (ring
order, partial-row addressing, owner masks) is pinned without a GPU.
"""

from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from . import moe_oracle as O


def _per_assignment(problem) -> torch.Tensor:
    """Weighted rows ``(T*k, K)`` of the assignments whose expert is local (zero elsewhere)."""
    cfg = problem.config
    if cfg.precision.value == "fp8":
        qc = problem.quant_config
        per = O.moe_fp8(problem.hidden_states, problem.w1, problem.w2, qc.w1_scale, qc.w2_scale, problem.topk_ids,
                        problem.expert_map, list(cfg.block_shape), cfg.torch_dtype)
    else:
        per = O.moe_dense(problem.hidden_states, problem.w1, problem.w2, problem.topk_ids, problem.expert_map)
    per = per * problem.topk_weights.float().unsqueeze(-1)
    return per.reshape(-1, per.shape[-1])


def forward_rank(problem, rank: int, world: int, group=None, combine: str | None = None) -> torch.Tensor:
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
    if combine is None:
        combine = "push" if ep else "partial"
    if combine == "push":
        assert ep, "the push combine is the expert-parallel form"
        wire = cfg.torch_dtype
        rows = _per_assignment(local).to(wire)                      # y[n], n = (ring*T + t)*k + j
        local_slot = torch.from_numpy(O.local_slots(ids_all.numpy(), problem.expert_map.numpy())) >= 0
        own = t * topk
        outbox = [None] * world                                     # what this rank sends to each home rank
        for ring in range(world):
            n = torch.arange(ring * own, (ring + 1) * own)
            keep = local_slot[n]
            outbox[(rank + ring) % world] = (n[keep] - ring * own, rows[n[keep]])
        inbox = [None] * world
        dist.all_gather_object(inbox, outbox, group=group)
        recv = torch.zeros(own, hidden, dtype=wire)
        seen = torch.zeros(own, dtype=torch.int32)
        for src in range(world):
            slots, data = inbox[src][rank]
            recv[slots] = data
            seen[slots] += 1
        assert bool((seen == 1).all()), "every assignment slot is written by exactly one rank"
        return recv.float().view(t, topk, hidden).sum(dim=1)
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
