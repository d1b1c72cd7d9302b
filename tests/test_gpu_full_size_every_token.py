"""Every token of the full-size DeepSeek-V3.2 workloads against a plain PyTorch
fp32 reference computed on the GPU.

The CPU oracle is too slow for all 8192 tokens x 256 experts, so the other
full-size tests sample tokens; a wrong tile at one (expert, feature block,
token block) could slip through a sample.  Here the same arithmetic as the
oracle (per expert: gather the rows, fp32 matmuls, SiLU-mul, for fp8 the 1x128
quantiser and one scaled partial product per 128-deep K block in ascending
order, reference.py:65-167) runs in torch on the GPU for every assignment, is
itself pinned to the CPU oracle on sampled tokens, and the library's output is
compared with it over the whole batch at the reference's tolerance."""

import dataclasses

import pytest
import torch
import torch.nn.functional as F

from moe_bench_b200 import problem as P
from moe_bench_b200.plugin import get_implementation
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _silu_mul(h):
    d = h.shape[-1] // 2
    return F.silu(h[..., :d]) * h[..., d:]


def _block_matmul(a_q, a_s, b_q, b_s, block=128):
    """a_q (m, K) e4m3 with scales a_s (m, K/128); b_q (n, K) e4m3 with scales b_s (n/128, K/128)."""
    a, b = a_q.float(), b_q.float()
    m, k = a.shape
    n = b.shape[0]
    col_block = torch.arange(n, device=a.device) // block
    out = torch.zeros(m, n, dtype=torch.float32, device=a.device)
    for i in range(k // block):
        ks = slice(i * block, (i + 1) * block)
        out += (a[:, ks] @ b[:, ks].t()) * (a_s[:, i : i + 1] * b_s[col_block, i].unsqueeze(0))
    return out


def torch_reference_on_gpu(prob):
    """(T, K) fp32 on the GPU; every assignment computed (single GPU: no expert map)."""
    fp8 = prob.config.precision.value == "fp8"
    x = prob.hidden_states
    t, hidden = x.shape
    topk = prob.topk_ids.shape[1]
    flat_ids = prob.topk_ids.reshape(-1)
    tok = torch.arange(t, device=x.device).repeat_interleave(topk)
    per = torch.zeros(t * topk, hidden, dtype=torch.float32, device=x.device)
    if fp8:
        xq, xs = O.group_quant_fp8(x, 128)
        qc = prob.quant_config
    else:
        xf = x.float()
    for e in range(prob.w1.shape[0]):
        sel = (flat_ids == e).nonzero().flatten()
        if sel.numel() == 0:
            continue
        if fp8:
            h = _block_matmul(xq[tok[sel]], xs[tok[sel]], prob.w1[e], qc.w1_scale[e].float())
            aq, a_s = O.group_quant_fp8(_silu_mul(h).to(torch.bfloat16), 128)
            per[sel] = _block_matmul(aq, a_s, prob.w2[e], qc.w2_scale[e].float())
        else:
            per[sel] = _silu_mul(xf[tok[sel]] @ prob.w1[e].float().t()) @ prob.w2[e].float().t()
    return (per.view(t, topk, hidden) * prob.topk_weights.float().unsqueeze(-1)).sum(dim=1)


def _subset(prob, idx):
    return dataclasses.replace(
        prob, num_tokens=len(idx), hidden_states=prob.hidden_states[idx].contiguous(),
        topk_ids=prob.topk_ids[idx].contiguous(), topk_weights=prob.topk_weights[idx].contiguous(),
    )


@pytest.mark.parametrize("precision,tokens", [("bf16", 8192), ("bf16", 2048), ("fp8", 8192), ("fp8", 128)])
def test_every_token_of_the_full_size_workload(precision, tokens):
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False           # the reference must be true fp32
    try:
        cfg = P.deepseek_v32_config(device=DEV, precision=P.Precision(precision))
        prob = P.make_problem(cfg, tokens, weights=P.make_weights(cfg))
        impl = get_implementation("b200")
        impl.setup(prob)
        out = impl.run(prob).clone()
        assert impl.device_status() == 0
        ref = torch_reference_on_gpu(prob)
        # the torch reference itself against the CPU oracle, on sampled tokens
        idx = torch.randperm(tokens, generator=torch.Generator().manual_seed(3))[:8].to(DEV)
        # (fp8: a last-bit difference between the GPU's and the CPU's fp32 sums can move an
        # activation to the neighbouring e4m3 value, hence the wider bound)
        pin = O.verify_output(precision, ref[idx], O.reference_moe(_subset(prob, idx)),
                              atol=3e-3 if precision == "fp8" else 2e-4, rtol=1e-3)
        assert pin.passed, pin.message
        # every token of the batch, at the reference's tolerance for the precision (reference.py:39-43)
        res = O.verify_output(precision, out, ref)
        assert res.passed, res.message
        assert res.rel_err < 1e-2, res.rel_err
        # and row by row: no single token may be far off even if the batch norm hides it
        row_err = (out.float() - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-6)
        assert float(row_err.max()) < 3e-2, float(row_err.max())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32
