"""GPU parity of the individual stages against the CPU oracle, through the C ABI.

Integer stages (routing ids, sort-and-pad, e4m3 bytes) must be bit-exact;
floating-point stages state their tolerance next to the check.
"""

import numpy as np
import pytest
import torch

from moe_bench_b200 import capi
from moe_bench_b200 import problem as P
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _routing(dist, tokens, experts, topk, seed=0, **kw):
    cfg = P.MoEBenchConfig(
        hidden_size=256, intermediate_size=128, num_experts=experts, topk=topk, world_size=1,
        routing=P.RoutingConfig(distribution=P.Distribution(dist), **kw), seed=seed, device="cpu",
    )
    gen = torch.Generator().manual_seed(seed + 17)
    return P._make_routing(cfg, tokens, gen)[0]


ALIGN_CASES = [
    # (distribution, tokens, experts, topk, ep_world)   ep_world 0 = no expert_map
    ("uniform", 64, 8, 2, 0),
    ("uniform", 1, 256, 8, 0),      # one token: 8 experts hit, 248 empty
    ("uniform", 8, 256, 8, 0),
    ("uniform", 128, 256, 8, 0),
    ("single", 300, 256, 8, 0),     # every token on experts 0..7
    ("skewed", 1024, 256, 8, 0),    # 8192 assignments: last size of the one-block path
    ("uniform", 1025, 256, 8, 0),   # first size of the three-kernel path, ragged tail
    ("skewed", 2048, 256, 8, 0),
    ("uniform", 8192, 256, 8, 0),   # full-size sweep point
    ("balanced", 777, 64, 8, 0),
    ("uniform", 1024, 256, 8, 8),   # EP: rank 3 of 8 owns 32 experts
    ("single", 512, 256, 8, 8),     # EP with no local assignment at all on rank 3
    ("uniform", 5000, 1024, 4, 0),  # maximum supported expert count
    ("uniform", 65536, 256, 8, 8),  # EP=8 at 8192 tokens per rank: 524 288 assignments, 1024 units, 32 local experts
    ("uniform", 40000, 320, 8, 0),  # 320 experts: three groups of threads scan the units side by side, 64 threads idle
    ("uniform", 40000, 384, 8, 0),  # 384 experts: two groups
]


@pytest.mark.parametrize("pad", [16, 128])
@pytest.mark.parametrize("dist,tokens,experts,topk,ep", ALIGN_CASES)
def test_align_bit_exact(dist, tokens, experts, topk, ep, pad):
    ids = _routing(dist, tokens, experts, topk)
    emap, local = None, experts
    if ep:
        local = experts // ep
        emap = torch.full((experts,), -1, dtype=torch.int32)
        emap[3 * local : 4 * local] = torch.arange(local, dtype=torch.int32)
    counts, prefix, sorted_ids, inverse = capi.align(
        ids.to(DEV), None if emap is None else emap.to(DEV), local, pad
    )
    torch.cuda.synchronize()
    o_counts, o_off, o_sorted, o_inv = O.align(ids.numpy(), None if emap is None else emap.numpy(), local, pad)
    assert np.array_equal(counts.cpu().numpy(), o_counts)
    assert np.array_equal(prefix.cpu().numpy() * pad, o_off)
    rows = int(o_off[-1])
    assert np.array_equal(sorted_ids.cpu().numpy()[:rows], o_sorted)
    assert np.array_equal(inverse.cpu().numpy(), o_inv)
    # rows past the last expert are never written
    assert bool((sorted_ids[rows:] == -2).all())


def test_align_is_a_permutation_at_full_size():
    """Size-independent property at the largest sweep point: every local
    assignment appears exactly once, inverse inverts sorted_ids, and rows are
    grouped by expert in ascending assignment order."""
    ids = _routing("uniform", 8192, 256, 8, seed=3)
    counts, prefix, sorted_ids, inverse = capi.align(ids.to(DEV), None, 256, 16)
    s = sorted_ids.cpu().numpy()
    inv = inverse.cpu().numpy()
    real = s[s >= 0]
    assert np.array_equal(np.sort(real), np.arange(8192 * 8))
    assert np.array_equal(s[inv], np.arange(8192 * 8))
    flat = ids.numpy().reshape(-1)
    pre = prefix.cpu().numpy()
    for e in (0, 17, 255):
        seg = s[pre[e] * 16 : pre[e + 1] * 16]
        seg = seg[seg >= 0]
        assert np.all(flat[seg] == e) and np.all(np.diff(seg) > 0)


@pytest.mark.parametrize("tokens,experts,topk", [(1, 8, 2), (64, 8, 2), (333, 256, 8), (8192, 256, 8), (50, 1000, 40)])
def test_route_topk(tokens, experts, topk):
    gen = torch.Generator().manual_seed(tokens * 7 + experts)
    logits = torch.randn(tokens, experts, generator=gen)
    if tokens > 1:
        logits[1] = 0.0          # all equal: ties broken by lowest index
        logits[0, 3] = logits[0, 5]
    ids, w = capi.route_topk(logits.to(DEV), topk)
    o_ids, o_w = O.route_topk(logits, topk)
    assert torch.equal(ids.cpu(), o_ids)  # bit-exact selection and order
    # weights: exp/sum evaluated in a different order than torch.softmax; fp32 rounding only
    torch.testing.assert_close(w.cpu(), o_w, atol=1e-6, rtol=2e-5)


def test_route_topk_single_distribution():
    """Logits that make experts 0..7 win for every token reproduce the
    'single' routing of the reference (data.py:198-206)."""
    logits = torch.randn(100, 256, generator=torch.Generator().manual_seed(1))
    logits[:, :8] = 10.0 - torch.arange(8).float() * 0.5
    ids, _ = capi.route_topk(logits.to(DEV), 8)
    assert torch.equal(ids.cpu(), torch.arange(8, dtype=torch.int32).repeat(100, 1))


@pytest.mark.parametrize("rows,hidden", [(1, 128), (7, 256), (512, 7168), (4096, 2048)])
def test_group_quant_fp8_bit_exact(rows, hidden):
    gen = torch.Generator().manual_seed(rows + hidden)
    x = (torch.randn(rows, hidden, generator=gen) * 3).to(torch.bfloat16)
    x[0, :128] = 0                      # all-zero group
    if rows > 2:
        x[2, 5] = 3.0e4                 # one huge element sets the group's scale
    q, s = capi.group_quant_fp8(x.to(DEV))
    oq, os_ = O.group_quant_fp8(x)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


def _stage_problem(tokens, hidden, inter, experts, topk, dist="uniform", seed=0):
    cfg = P.MoEBenchConfig(
        hidden_size=hidden, intermediate_size=inter, num_experts=experts, topk=topk, world_size=1,
        routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=seed, device="cpu",
    )
    return P.make_problem(cfg, tokens)


@pytest.mark.parametrize(
    "tokens,hidden,inter,experts,topk,dist",
    [
        (64, 256, 128, 8, 2, "uniform"),     # config 1: one tile per expert
        (300, 512, 256, 4, 2, "uniform"),    # several M tiles per expert, ragged last tile
        (40, 1024, 384, 16, 4, "single"),    # empty experts
        (200, 192, 320, 8, 2, "uniform"),    # hidden/intermediate not multiples of the tile width
        (2000, 256, 128, 4, 2, "uniform"),   # ~1000 rows per expert: several 256-token blocks, balanced split
        (37, 512, 256, 32, 1, "uniform"),    # one or two rows per expert: 16-token boxes
    ],
)
def test_grouped_gemm_stages(tokens, hidden, inter, experts, topk, dist):
    """Gate/up + SiLU-mul and down + weight stages against fp32 matmuls on the CPU."""
    prob = _stage_problem(tokens, hidden, inter, experts, topk, dist)
    ids = prob.topk_ids
    counts, prefix, sorted_ids, inverse = capi.align(ids.to(DEV), None, experts, capi.PAD_ROWS_BF16)
    cap = sorted_ids.shape[0]
    s_cpu = sorted_ids.cpu()
    x = prob.hidden_states
    rows = (s_cpu >= 0).nonzero().flatten()
    row_tok = (s_cpu[rows] // topk).long()
    flat = ids.reshape(-1).long()
    row_exp = flat[s_cpu[rows].long()]

    xg = torch.zeros(cap, hidden, dtype=torch.bfloat16)
    xg[rows] = x[row_tok]
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    act = torch.full((cap, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    capi.grouped_gemm_bf16(0, xg.to(DEV), prob.w1.to(DEV), hidden, inter, counts, prefix, sorted_ids, None, act, status)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    h = torch.zeros(len(rows), 2 * inter)
    for e in range(experts):
        m = row_exp == e
        if m.any():
            h[m] = x[row_tok[m]].float() @ prob.w1[e].float().t()
    ref_act = O.silu_and_mul(h)
    got_act = act.cpu()[rows].float()
    # fp32 accumulation of exact bf16 products, then one bf16 rounding: 2^-8 relative
    torch.testing.assert_close(got_act, ref_act, atol=2e-3, rtol=8e-3)
    # padding rows are never written
    pad = (s_cpu < 0).nonzero().flatten()
    assert bool(torch.isnan(act.cpu()[pad].float()).all())

    # second stage consumes the rounded activations the first one produced
    a2 = act.clone()
    a2[pad.to(DEV)] = 0
    w = prob.topk_weights.reshape(-1)
    y = torch.full((tokens * topk, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
    capi.grouped_gemm_bf16(1, a2, prob.w2.to(DEV), hidden, inter, counts, prefix, sorted_ids, w.to(DEV), y, status)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    ref_y = torch.zeros(len(rows), hidden)
    a_in = act.cpu()[rows].float()
    for e in range(experts):
        m = row_exp == e
        if m.any():
            ref_y[m] = a_in[m] @ prob.w2[e].float().t()
    ref_y *= w[s_cpu[rows].long()].unsqueeze(-1)
    got_y = y.cpu()[s_cpu[rows].long()].float()
    torch.testing.assert_close(got_y, ref_y, atol=2e-3, rtol=8e-3)


def _gated_inputs(tokens=300, hidden=512, inter=256, experts=4, topk=2):
    prob = _stage_problem(tokens, hidden, inter, experts, topk, "uniform")
    counts, prefix, sorted_ids, _ = capi.align(prob.topk_ids.to(DEV), None, experts, capi.PAD_ROWS_BF16)
    cap = sorted_ids.shape[0]
    s_cpu = sorted_ids.cpu()
    rows = (s_cpu >= 0).nonzero().flatten()
    xg = torch.zeros(cap, hidden, dtype=torch.bfloat16)
    xg[rows] = prob.hidden_states[(s_cpu[rows] // topk).long()]
    return prob, counts, prefix, sorted_ids, xg.to(DEV), cap


def test_gated_gate_up_matches_the_plain_stage_when_rows_have_arrived():
    """Rows delivered by someone else: with every granule counter at its target the
    gated stage loads the same rows and must give the plain stage's bits."""
    prob, counts, prefix, sorted_ids, xg, cap = _gated_inputs()
    hidden, inter = prob.hidden_states.shape[1], prob.w1.shape[1] // 2
    w1 = prob.w1.to(DEV)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    plain = torch.zeros(cap, inter, dtype=torch.bfloat16, device=DEV)
    capi.grouped_gemm_bf16(0, xg, w1, hidden, inter, counts, prefix, sorted_ids, None, plain, status)
    done = torch.full((cap // 16 + 1,), 3, dtype=torch.int32, device=DEV)
    gated = torch.zeros(cap, inter, dtype=torch.bfloat16, device=DEV)
    capi.grouped_gemm_bf16_gated(xg, w1, hidden, inter, counts, prefix, sorted_ids, done, 3, gated, status)
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    assert torch.equal(plain, gated) and bool(plain.float().abs().sum() > 0)


def test_wait_for_rows_that_never_arrive_gives_up_with_a_status_and_the_context_stays_usable():
    """The in-kernel waits are bounded: with granule counters that nothing raises and a
    50 ms wait limit in the status block, the tile loader gives up (site 6 -> status
    106), the other warps leave through the abort flag, the launch returns and the
    next forward on the same context is clean.  Nothing traps or hangs: the wait
    simply runs out."""
    import time

    prob, counts, prefix, sorted_ids, xg, cap = _gated_inputs()
    hidden, inter = prob.hidden_states.shape[1], prob.w1.shape[1] // 2
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    status[1] = 50  # milliseconds one wait may last
    never = torch.zeros(cap // 16 + 1, dtype=torch.int32, device=DEV)
    out = torch.zeros(cap, inter, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    t0 = time.time()
    capi.grouped_gemm_bf16_gated(xg, prob.w1.to(DEV), hidden, inter, counts, prefix, sorted_ids, never, 1, out, status)
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    assert int(status[0].item()) == 106

    # the same context runs a clean forward afterwards
    from moe_bench_b200.plugin import get_implementation

    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=4, topk=2, world_size=1,
                           seed=0, device=DEV)
    p2 = P.make_problem(cfg, 100)
    impl = get_implementation("b200")
    impl.setup(p2)
    res = O.verify_output("bf16", impl.run(p2), O.reference_moe(p2))
    assert impl.device_status() == 0 and res.passed, res.message
