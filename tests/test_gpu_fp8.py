"""fp8 block-quantised path on the GPU: stage-level against the CPU oracle's
block matmul, layer-level against the reference-pinned golden outputs and the
oracle, at the reference's fp8 tolerance (atol 3.5e-2, rtol 3.5e-2;
reference.py:39-43)."""

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

    qc = prob.quant_config
    qc = None if qc is None else P.BlockQuantConfig(mv(qc.w1_scale), mv(qc.w2_scale), list(qc.block_shape))
    return dataclasses.replace(
        prob, hidden_states=mv(prob.hidden_states), w1=mv(prob.w1), w2=mv(prob.w2), topk_ids=mv(prob.topk_ids),
        topk_weights=mv(prob.topk_weights), expert_map=mv(prob.expert_map), quant_config=qc,
    )


def _fp8_problem(tokens, hidden, inter, experts, topk, dist="uniform", seed=0, mode="tp", world=1, rank=0):
    cfg = P.MoEBenchConfig(
        hidden_size=hidden, intermediate_size=inter, num_experts=experts, topk=topk, world_size=world,
        parallel_mode=P.ParallelMode(mode), precision=P.Precision.FP8,
        routing=P.RoutingConfig(distribution=P.Distribution(dist)), seed=seed, device="cpu",
    )
    return P.make_problem(cfg, tokens, rank)


@pytest.mark.parametrize("cols", [False, True])
@pytest.mark.parametrize(
    "tokens,hidden,inter,experts,topk,dist",
    [(64, 256, 128, 8, 2, "uniform"), (300, 512, 256, 4, 2, "uniform"), (40, 1024, 384, 16, 4, "single")],
)
def test_fp8_gemm_stages(tokens, hidden, inter, experts, topk, dist, cols):
    """Both fp8 kernel families: 128-row token tiles, and tokens on the MMA N dimension
    (schedule padded to 16 rows; 150 rows per expert here means two token blocks)."""
    prob = _fp8_problem(tokens, hidden, inter, experts, topk, dist)
    qc = prob.quant_config
    ids = prob.topk_ids
    counts, prefix, sorted_ids, inverse = capi.align(
        ids.to(DEV), None, experts, capi.PAD_ROWS_BF16 if cols else capi.PAD_ROWS_FP8
    )
    cap = sorted_ids.shape[0]
    s_cpu = sorted_ids.cpu()
    rows = (s_cpu >= 0).nonzero().flatten()
    row_tok = (s_cpu[rows] // topk).long()
    row_exp = ids.reshape(-1).long()[s_cpu[rows].long()]

    xq, xs = O.group_quant_fp8(prob.hidden_states)
    a = torch.zeros(cap, hidden, dtype=torch.uint8)
    a[rows] = xq.view(torch.uint8)[row_tok]
    a_s_t = torch.ones(hidden // 128, cap)
    a_s_t[:, rows] = xs[row_tok].t()
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    actq = torch.zeros(cap, inter, dtype=torch.uint8, device=DEV)
    acts_t = torch.zeros(inter // 128, cap, dtype=torch.float32, device=DEV)
    capi.grouped_gemm_fp8(
        0, a.to(DEV), a_s_t.contiguous().to(DEV), prob.w1.to(DEV), qc.w1_scale.contiguous().to(DEV), hidden, inter,
        counts, prefix, sorted_ids, None, actq, acts_t, status, cols=cols,
    )
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    # oracle: block matmul -> SiLU-mul -> bf16 -> group quant
    ref_act = torch.zeros(len(rows), inter)
    for e in range(experts):
        m = row_exp == e
        if m.any():
            h = O.block_matmul(xq[row_tok[m]], prob.w1[e], xs[row_tok[m]], qc.w1_scale[e], [128, 128])
            ref_act[m] = O.silu_and_mul(h).to(torch.bfloat16).float()
    got_q = actq.cpu()[rows].view(torch.float8_e4m3fn).float()
    got_s = acts_t.cpu()[:, rows].t()
    got_act = (got_q.view(len(rows), inter // 128, 128) * got_s.unsqueeze(-1)).view(len(rows), inter)
    # dequantised activations: e4m3 has 3 mantissa bits -> 2^-4 relative per element
    torch.testing.assert_close(got_act, ref_act, atol=2e-2, rtol=7e-2)
    rq, rs = O.group_quant_fp8(ref_act.to(torch.bfloat16))
    # scales agree unless a rounding flip moved the group's amax (one bf16 ulp)
    torch.testing.assert_close(got_s, rs, atol=0, rtol=1e-2)
    assert float((got_q != rq.float()).float().mean()) < 0.02

    # second stage on the activations the first one produced
    w = prob.topk_weights.reshape(-1)
    y = torch.full((tokens * topk, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
    capi.grouped_gemm_fp8(
        1, actq, acts_t, prob.w2.to(DEV), qc.w2_scale.contiguous().to(DEV), hidden, inter, counts, prefix,
        sorted_ids, w.to(DEV), y, None, status, cols=cols,
    )
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0
    ref_y = torch.zeros(len(rows), hidden)
    aq_rows = actq.cpu()[rows].view(torch.float8_e4m3fn)
    for e in range(experts):
        m = row_exp == e
        if m.any():
            ref_y[m] = O.block_matmul(aq_rows[m], prob.w2[e], got_s[m], qc.w2_scale[e], [128, 128])
    ref_y *= w[s_cpu[rows].long()].unsqueeze(-1)
    got_y = y.cpu()[s_cpu[rows].long()].float()
    # same e4m3 inputs on both sides: only fp32 summation order and the bf16 store differ
    torch.testing.assert_close(got_y, ref_y, atol=2e-3, rtol=8e-3)


def _check(out, ref):
    res = O.verify_output("fp8", out, ref)
    assert res.passed, res.message
    assert res.rel_err < 3e-2, res.rel_err


@pytest.mark.parametrize("name,rank", [("config1_uniform_fp8", 0), ("config1_ep2_rank0_fp8", 0)])
def test_fp8_layer_matches_reference_outputs(golden, name, rank):
    case = golden["cases"][name]
    cfg = P.MoEBenchConfig.from_dict(case["config"])
    prob = P.make_problem(cfg, case["num_tokens"], rank)
    impl = get_implementation("b200")
    impl.fp8_scale_format = "fp32"   # the fixtures were made with the plain fp32 activation scales
    dprob = _to_dev(prob)
    impl.setup(dprob)
    out = impl.run(dprob)
    assert impl.device_status() == 0
    capi.use_reference_fp8_scale_format()
    _check(out, case["reference"])


@pytest.mark.parametrize(
    "tokens,hidden,inter,experts,topk,dist",
    [(1, 512, 256, 16, 4, "uniform"), (129, 512, 256, 16, 4, "uniform"), (1000, 1024, 512, 32, 8, "skewed"),
     (513, 768, 384, 8, 2, "single")],
)
def test_fp8_layer_matches_oracle(tokens, hidden, inter, experts, topk, dist):
    prob = _fp8_problem(tokens, hidden, inter, experts, topk, dist, seed=7)
    impl = get_implementation("b200")
    dprob = _to_dev(prob)
    impl.setup(dprob)
    out = impl.run(dprob)
    assert impl.device_status() == 0
    _check(out, O.reference_moe(prob))
    again = impl.run(dprob).clone()
    assert torch.equal(again, impl.run(dprob))


def test_fp8_dsv32_shape_sampled_tokens():
    """DeepSeek-V3.2 dims, fp8, 32 of the 256 experts (one expert-parallel
    rank's share) at 1024 tokens: sampled tokens against the oracle and
    batch-independence of a token's output."""
    cfg = P.deepseek_v32_config(device=DEV, precision=P.Precision.FP8, parallel_mode=P.ParallelMode.EP, world_size=8)
    weights = P.make_weights(cfg, rank=2)
    prob = P.make_problem(cfg, 1024, rank=2, weights=weights)
    impl = get_implementation("b200")
    impl.setup(prob)
    big = impl.run(prob).clone()
    assert impl.device_status() == 0 and bool(torch.isfinite(big.float()).all())
    idx = torch.randperm(1024, generator=torch.Generator().manual_seed(2))[:24].to(DEV)
    sub = dataclasses.replace(prob, num_tokens=24, hidden_states=prob.hidden_states[idx].contiguous(),
                              topk_ids=prob.topk_ids[idx].contiguous(), topk_weights=prob.topk_weights[idx].contiguous())
    _check(big[idx], O.reference_moe(sub))
    impl2 = get_implementation("b200")
    impl2.setup(sub)
    small = impl2.run(sub)
    res = O.verify_output("fp8", small, big[idx].float(), atol=4e-3, rtol=0)
    assert res.passed and res.rel_err < 1e-3, (res.message, res.rel_err)


@pytest.mark.parametrize("fmt", ["fp32", "ue8m0"])
def test_group_quant_matches_vllm_op_if_present(fmt):
    """The activation quantiser the reference calls on a GPU is vLLM's
    per_token_group_quant_fp8; where vLLM is installed, compare byte for byte, in both
    scale formats (which one the reference gets depends on the box: vLLM picks
    power-of-two scales where its DeepGEMM path is enabled)."""
    try:
        from vllm.model_executor.layers.quantization.utils.fp8_utils import per_token_group_quant_fp8
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"vLLM not importable: {exc}")
    x = (torch.randn(257, 7168, generator=torch.Generator().manual_seed(4)) * 2).to(torch.bfloat16).to(DEV)
    try:
        vq, vs = per_token_group_quant_fp8(x, 128, use_ue8m0=(fmt == "ue8m0"))
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"vLLM quantiser not runnable here: {exc}")
    capi.set_fp8_scale_format(fmt)
    try:
        q, s = capi.group_quant_fp8(x)
    finally:
        capi.use_reference_fp8_scale_format()
    same_scale = float((s == vs.reshape(s.shape)).float().mean())
    same_bytes = float((q.view(torch.uint8) == vq.view(torch.uint8)).float().mean())
    print(f"vLLM quantiser agreement ({fmt}): scales {same_scale:.6f}, bytes {same_bytes:.6f}")
    assert same_scale == 1.0 and same_bytes == 1.0
    # and the CPU oracle's quantiser in the same format
    oq, os_ = O.group_quant_fp8(x.cpu(), scale_format=fmt)
    assert torch.equal(oq.view(torch.uint8), q.cpu().view(torch.uint8)) and torch.equal(os_, s.cpu())


@pytest.mark.parametrize("fmt", ["fp32", "ue8m0"])
def test_layer_in_both_activation_scale_formats(fmt):
    """The whole fp8 layer in each scale format (whichever the box's vLLM picks, both are
    exercised), against the oracle computing in the same format."""
    from moe_bench_b200.plugin import get_implementation

    cfg = P.MoEBenchConfig(hidden_size=512, intermediate_size=256, num_experts=8, topk=2, world_size=1,
                           precision=P.Precision.FP8, seed=0, device=DEV)
    for tokens in (5, 700):   # tokens-on-columns kernels, 128-row-tile kernels
        prob = P.make_problem(cfg, tokens)
        impl = get_implementation("b200")
        impl.fp8_scale_format = fmt
        impl.setup(prob)
        out = impl.run(prob)
        assert impl.device_status() == 0
        before = O.FP8_SCALE_FORMAT
        O.FP8_SCALE_FORMAT = fmt
        try:
            ref = O.reference_moe(prob)
        finally:
            O.FP8_SCALE_FORMAT = before
        res = O.verify_output("fp8", out, ref)
        assert res.passed and res.rel_err < 1e-2, (tokens, res.message, res.rel_err)
    capi.use_reference_fp8_scale_format()
