"""CPU oracle for the MoE layer forward.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the arithmetic the moe_bench reference defines
for the layer (``reference.py``) and for the routing / sort-and-pad steps that
surround it.  It exists to check the CUDA path; nothing the library ships may
import it.  Only the test-suite, the smoke check and the benchmark's CPU
baseline legs use it.

Parity status
-------------
* bf16 / fp16 layer (``moe_dense``): pinned against outputs of the reference
  itself, generated in a container where the reference imports
  (``tests/golden/make_golden.py`` -> ``tests/golden/golden.pt``).
* sort-and-pad (``align``): pinned against the slot order produced by the
  reference's host schedule builder (``tk_scheme.py:98-126``) for world size 1,
  replayed by ``tests/golden/make_golden.py``.
* fp8 layer (``moe_fp8``): the block matmul, SiLU-mul, bf16 round and combine
  follow ``reference.py:65-95,119-182`` and are pinned by running the
  reference's ``_reference_fp8`` with its activation quantiser replaced by
  ``group_quant_fp8`` (cases ``config1_*_fp8`` of ``golden.pt``).  The activation
  quantiser itself is a call into vLLM 0.22.0 (``moe_kernel_quantize_input`` ->
  ``per_token_group_quant_fp8``), a third-party CUDA/Triton op that cannot run
  on a CPU and that no reference test pins at bit level: on the CPU this oracle
  is "parity unpinned" for it; on a GPU box the test-suite pins the CUDA
  quantiser of this package (which must equal ``group_quant_fp8`` bit for bit)
  against vLLM's op itself.
* top-k routing (``route_topk``): the reference has no router (it draws ids
  directly, ``data.py:178-235``); the oracle is the textbook
  softmax -> top-k -> renormalise and is "parity unpinned".
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0

# Format of the fp8 activation scales: "fp32" (amax/448) or "ue8m0" (rounded up to a power of
# two).  The reference leaves the choice to vLLM, which uses the second on GPUs where its
# DeepGEMM path is enabled (Hopper, Blackwell) and the first elsewhere; callers that check a
# GPU run set this to what the library was told to compute.
FP8_SCALE_FORMAT = "fp32"

# (atol, rtol) per precision: reference.py:39-43.
DEFAULT_TOL = {"bf16": (2e-2, 0.0), "fp16": (1e-2, 0.0), "fp8": (3.5e-2, 3.5e-2)}


# ----------------------------------------------------------------------------
# integer / index stages
# ----------------------------------------------------------------------------
def local_slots(topk_ids, expert_map):
    """Flat ``(T*k,)`` int64 local expert slot per assignment, -1 when the
    expert is not on this rank (reference.py:52-62)."""
    ids = np.asarray(topk_ids, dtype=np.int64).reshape(-1)
    if expert_map is None:
        return ids
    return np.asarray(expert_map, dtype=np.int64)[ids]


def align(topk_ids, expert_map, num_local_experts: int, tile_m: int = 128):
    """Sort assignments by local expert and pad every expert segment to a
    multiple of ``tile_m`` rows.

    The order inside an expert is ascending flat assignment index
    ``n = token * k + kpos`` (a stable sort), which is what the reference's
    schedule builder produces on one rank: cursor advanced over ``src_tok``
    then ``kpos`` (tk_scheme.py:98-126), equal to the argsort key of
    tk_scheme.py:338-342.

    Returns ``(counts[E], offsets[E+1], sorted_ids[P], inverse[T*k])`` as
    int32 numpy arrays: ``offsets`` are padded row offsets, ``sorted_ids[p]``
    is the flat assignment index in row ``p`` or -1 for padding,
    ``inverse[n]`` is the row of assignment ``n`` or -1 if its expert is not
    local.
    """
    slots = local_slots(topk_ids, expert_map)
    n_assign = slots.shape[0]
    counts = np.bincount(slots[slots >= 0], minlength=num_local_experts).astype(np.int64)
    padded = (counts + tile_m - 1) // tile_m * tile_m
    offsets = np.zeros(num_local_experts + 1, dtype=np.int64)
    offsets[1:] = np.cumsum(padded)
    sorted_ids = np.full(int(offsets[-1]), -1, dtype=np.int32)
    inverse = np.full(n_assign, -1, dtype=np.int32)
    order = np.argsort(slots, kind="stable")
    order = order[slots[order] >= 0]
    rank_in_expert = np.arange(order.shape[0]) - np.repeat(
        np.concatenate([[0], np.cumsum(counts)[:-1]]), counts
    )
    rows = offsets[slots[order]] + rank_in_expert
    sorted_ids[rows] = order.astype(np.int32)
    inverse[order] = rows.astype(np.int32)
    return counts.astype(np.int32), offsets.astype(np.int32), sorted_ids, inverse


def route_topk(logits: torch.Tensor, k: int):
    """softmax over experts -> top-k -> weights renormalised to sum to 1.

    Selection is by logit, largest first, lowest expert index on equal logits
    (softmax is monotonic, so this is top-k of the probabilities with an
    explicit tie rule).  Returns (ids int32, weights fp32)."""
    lg = logits.float()
    order = torch.sort(-lg, dim=-1, stable=True).indices[:, :k]
    top = torch.gather(torch.softmax(lg, dim=-1), 1, order)
    return order.to(torch.int32), top / top.sum(dim=-1, keepdim=True)


# ----------------------------------------------------------------------------
# fp8 quantisation
# ----------------------------------------------------------------------------
def group_quant_fp8(x: torch.Tensor, group: int = 128, eps: float = 1e-10, scale_format: str | None = None):
    """Per-row, per-``group`` dynamic e4m3 quantisation of activations.

    Semantics of vLLM 0.22.0 ``per_token_group_quant_fp8`` as the reference
    reaches it on a GPU (reference.py:143-145,157-163 -> the
    ``per_token_group_fp8_quant`` CUDA op): ``amax = max(|x|, eps)`` in fp32,
    ``scale = amax / 448`` (an IEEE division; vLLM's Triton fallback multiplies
    by the reciprocal instead, which differs in the last bit for ~60 % of the
    groups), ``q = clamp(x / scale, -448, 448)`` rounded to nearest-even e4m3.
    With ``scale_format="ue8m0"`` (default: the module's ``FP8_SCALE_FORMAT``) the
    scale is then rounded up to a power of two, ``exp2(ceil(log2(scale)))``, as
    vLLM does when it runs with DeepGEMM's E8M0 scales.
    The GPU test-suite compares the CUDA kernel of this package with vLLM's op
    byte for byte, in both formats, where vLLM is installed.
    Returns ``(q (m, K) e4m3, scales (m, K/group) fp32)``.
    """
    m, k = x.shape
    xf = x.float().view(m, k // group, group)
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    scale = amax / np.float32(FP8_MAX)
    if (scale_format or FP8_SCALE_FORMAT) == "ue8m0":
        scale = torch.exp2(torch.ceil(torch.log2(scale.abs().clamp_min(1e-10))))
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(m, k), scale.view(m, k // group)


def block_matmul(a_q, b_q, a_s, b_s, block_shape):
    """``a @ b.T`` for block-scaled e4m3 operands with fp32 accumulation, one
    partial product per (k-block, n-block) scaled by ``a_s[:, i] * b_s[j, i]``
    and added in ascending k-block order (reference.py:65-95)."""
    bn, bk = block_shape
    a = a_q.float()
    b = b_q.float()  # converted where it lives (a GPU tensor is converted there), multiplied on the CPU
    a, b = a.cpu(), b.cpu()
    a_s, b_s = a_s.float().cpu(), b_s.float().cpu()
    m, k = a.shape
    n = b.shape[0]
    out = torch.zeros(m, n, dtype=torch.float32)
    # scale of every output column for k-block i: b_s[j, i] of the column's n-block j
    col_block = torch.arange(n) // bn
    for i in range(-(-k // bk)):
        ks = slice(i * bk, min((i + 1) * bk, k))
        # all n-blocks of this k-block in one product; each element still receives
        # (partial * (a_s * b_s)) added in ascending k-block order, as in the reference's loop
        out += (a[:, ks] @ b[:, ks].t()) * (a_s[:, i : i + 1] * b_s[col_block, i].unsqueeze(0))
    return out


# ----------------------------------------------------------------------------
# the layer
# ----------------------------------------------------------------------------
def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` with gate = first half of the last dim
    (reference.py:46-49)."""
    d = x.shape[-1] // 2
    return F.silu(x[..., :d]) * x[..., d:]


def moe_dense(hidden_states, w1, w2, topk_ids, expert_map):
    """bf16/fp16 layer, per assignment, everything in fp32 with no
    intermediate rounding (reference.py:98-116).  Returns ``(T, k, K)`` fp32;
    rows of non-local assignments are zero."""
    t, k_dim = hidden_states.shape
    topk = topk_ids.shape[1]
    x = hidden_states.cpu().float()
    slots = torch.from_numpy(local_slots(topk_ids.cpu().numpy(), None if expert_map is None else expert_map.cpu().numpy()))
    tok = torch.arange(t).repeat_interleave(topk)
    out = torch.zeros(t * topk, k_dim, dtype=torch.float32)
    for e in range(w1.shape[0]):
        sel = (slots == e).nonzero().flatten()
        if sel.numel() == 0:
            continue
        # weights may live on another device: only touched experts are copied
        # (converted to fp32 where they live, multiplied on the CPU)
        h = x[tok[sel]] @ w1[e].float().cpu().t()
        out[sel] = silu_and_mul(h) @ w2[e].float().cpu().t()
    return out.view(t, topk, k_dim)


def moe_fp8(hidden_states, w1, w2, w1_scale, w2_scale, topk_ids, expert_map, block_shape, base_dtype=torch.bfloat16):
    """fp8 block-quantised layer per assignment (reference.py:119-167):
    quantise x per 128-group, block matmul with w1, SiLU-mul, round to the base
    dtype, quantise again, block matmul with w2."""
    t, k_dim = hidden_states.shape
    topk = topk_ids.shape[1]
    xq, xs = group_quant_fp8(hidden_states.cpu(), block_shape[1])
    slots = torch.from_numpy(local_slots(topk_ids.cpu().numpy(), None if expert_map is None else expert_map.cpu().numpy()))
    tok = torch.arange(t).repeat_interleave(topk)
    out = torch.zeros(t * topk, k_dim, dtype=torch.float32)
    for e in range(w1.shape[0]):
        sel = (slots == e).nonzero().flatten()
        if sel.numel() == 0:
            continue
        h = block_matmul(xq[tok[sel]], w1[e], xs[tok[sel]], w1_scale[e], block_shape)
        act = silu_and_mul(h).to(base_dtype)
        aq, a_s = group_quant_fp8(act, block_shape[1])
        out[sel] = block_matmul(aq, w2[e], a_s, w2_scale[e], block_shape)
    return out.view(t, topk, k_dim)


def reference_moe(problem) -> torch.Tensor:
    """Layer output ``(T, K)`` fp32 for a problem bundle (any object with the
    ``MoEProblem`` attributes), tensors on the CPU (reference.py:170-182)."""
    prec = problem.config.precision.value
    if prec == "fp8":
        qc = problem.quant_config
        per = moe_fp8(
            problem.hidden_states, problem.w1, problem.w2, qc.w1_scale, qc.w2_scale,
            problem.topk_ids, problem.expert_map, list(problem.config.block_shape),
            problem.config.torch_dtype,
        )
    else:
        per = moe_dense(problem.hidden_states, problem.w1, problem.w2, problem.topk_ids, problem.expert_map)
    return (per * problem.topk_weights.cpu().float().unsqueeze(-1)).sum(dim=1)


@dataclass
class VerificationResult:
    """reference.py:185-204."""

    max_abs_err: float
    rel_err: float
    atol: float
    rtol: float
    passed: bool
    message: str = ""


def verify_output(precision: str, output, reference, atol=None, rtol=None) -> VerificationResult:
    """``assert_close`` at the per-precision tolerance plus relative L2 and
    max-abs error (reference.py:207-250)."""
    d_atol, d_rtol = DEFAULT_TOL[precision]
    atol = d_atol if atol is None else atol
    rtol = d_rtol if rtol is None else rtol
    out, ref = output.float().cpu(), reference.float().cpu()
    diff = out - ref
    passed, message = True, ""
    try:
        torch.testing.assert_close(out, ref, atol=atol, rtol=rtol)
    except AssertionError as err:
        passed = False
        lines = [ln.strip() for ln in str(err).splitlines() if ln.strip()]
        message = next((ln for ln in lines if ln.startswith("Mismatched")), lines[0] if lines else "")
    return VerificationResult(
        float(diff.abs().max()), float(diff.norm() / ref.norm().clamp_min(1e-12)), atol, rtol, passed, message
    )
