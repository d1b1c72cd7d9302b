"""The compute-only plugin: a moe_bench ``MoEImplementation`` backed by the
sm_100a library.

``MoEImplementation`` and the registry mirror reference ``baseline.py:24-44``
and ``baseline.py:80-91`` (same method names, argument meaning and error
behaviour), so ``B200FusedExperts`` can be registered in the reference's own
``IMPLEMENTATIONS`` table unchanged: it only reads the attributes of the
problem bundle it is handed.

``run`` is allocation-stable, has no host synchronisation and reads only from
``problem`` and buffers made in ``setup``, as the reference requires of a
timed, graph-captured implementation (ADDING_IMPLEMENTATIONS.md:48-60).
"""

from __future__ import annotations

from abc import ABC, abstractmethod

import torch

from . import capi
from .problem import MoEProblem, Precision


class MoEImplementation(ABC):
    """Uniform interface of a benchmarked MoE forward (reference baseline.py:24-44)."""

    name: str

    def setup(self, problem: MoEProblem) -> None:
        """Optional one-time, untimed preparation for ``problem``'s shape."""

    @abstractmethod
    def run(self, problem: MoEProblem) -> torch.Tensor:
        """Return the layer output ``(num_tokens, hidden_size)``."""
        raise NotImplementedError


class B200FusedExperts(MoEImplementation):
    """MoE layer forward on hand-written sm_100a kernels (tcgen05 grouped GEMMs
    fed by TMA, fused SiLU-mul, activation re-quantisation and combine weights)
    through the C ABI; bf16, and fp8 with 128x128 weight-block / 1x128
    activation-group fp32 scales."""

    name = "b200"

    # fp8 activation scale format: None = what the reference does on this box (asked of vLLM
    # in setup()), or "fp32" / "ue8m0" to fix it
    fp8_scale_format = None
    # limit of one in-kernel wait in milliseconds (0 = the library's default of 4 s)
    wait_limit_ms = 0

    def __init__(self) -> None:
        self._key = None
        self._workspace = None
        self._out = None
        self._fp8 = False
        self._w1_scale = self._w2_scale = None

    @staticmethod
    def _shape_key(problem: MoEProblem):
        x = problem.hidden_states
        return (
            x.device, tuple(x.shape), tuple(problem.w1.shape), tuple(problem.topk_ids.shape),
            problem.config.precision.value,
        )

    def setup(self, problem: MoEProblem) -> None:
        if not problem.hidden_states.is_cuda:
            raise capi.MB200Error("B200FusedExperts needs CUDA tensors; there is no CPU path")
        prec = Precision(problem.config.precision.value)
        self._fp8 = prec == Precision.FP8
        self._dtype = torch.float16 if prec == Precision.FP16 else torch.bfloat16
        if not self._fp8 and problem.w1.dtype != self._dtype:
            raise capi.MB200Error(f"{prec.value} problem with {problem.w1.dtype} weights")
        if problem.hidden_states.dtype != self._dtype:
            raise capi.MB200Error(f"{prec.value} problem with {problem.hidden_states.dtype} hidden_states")
        if self._fp8:
            qc = problem.quant_config
            if qc is None or qc.w1_scale is None or qc.w2_scale is None:
                raise capi.MB200Error("fp8 problem without quant_config.w1_scale / w2_scale")
            if list(qc.block_shape) != [128, 128]:
                raise capi.MB200Error(f"fp8 block_shape {qc.block_shape} is not supported (only [128, 128])")
            if problem.w1.dtype != torch.float8_e4m3fn:
                raise capi.MB200Error(f"fp8 problem with {problem.w1.dtype} weights")
            # plugin-owned contiguous fp32 copies of the (small) scale tables
            self._w1_scale = qc.w1_scale.to(torch.float32).contiguous()
            self._w2_scale = qc.w2_scale.to(torch.float32).contiguous()
            self._scale_format = self.fp8_scale_format or capi.reference_fp8_scale_format()
        capi.load()
        capi.check_problem_tensors(problem, self._dtype)
        t, hidden = problem.hidden_states.shape
        e_local, two_n, _ = problem.w1.shape
        topk = problem.topk_ids.shape[1]
        code = {Precision.BF16: capi.PRECISION_BF16, Precision.FP8: capi.PRECISION_FP8,
                Precision.FP16: capi.PRECISION_FP16}[prec]
        nbytes = capi.workspace_bytes(code, t, hidden, two_n // 2, e_local, topk)
        dev = problem.hidden_states.device
        # torch's caching allocator hands out 512-byte aligned blocks; over-allocate
        # and slice to the 1024-byte boundary the tile buffers need.
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        shift = (-raw.data_ptr()) % 1024
        self._workspace = raw[shift : shift + nbytes]
        self._workspace[:256].zero_()  # status block: [0] first failure code, [1] wait limit in ms
        self._workspace[:256].view(torch.int32)[1] = int(self.wait_limit_ms)
        self._out = torch.empty(t, hidden, dtype=self._dtype, device=dev)
        self._key = self._shape_key(problem)

    def run(self, problem: MoEProblem) -> torch.Tensor:
        if self._key != self._shape_key(problem):
            raise capi.MB200Error("run() called with a problem of another shape than setup()")
        expert_map = problem.expert_map
        if self._fp8:
            capi.set_fp8_scale_format(self._scale_format)
            capi.moe_forward_fp8(
                problem.hidden_states, problem.w1, problem.w2, self._w1_scale, self._w2_scale,
                problem.topk_ids, problem.topk_weights, expert_map, self._out, self._workspace,
            )
        else:
            capi.moe_forward_bf16(
                problem.hidden_states, problem.w1, problem.w2, problem.topk_ids, problem.topk_weights,
                expert_map, self._out, self._workspace,
            )
        return self._out

    def device_status(self) -> int:
        """Synchronise and return the kernels' status word (0 = every wait completed)."""
        return capi.read_status(self._workspace)


# Registry keyed by the harness's ``--impl`` name (reference baseline.py:80-91).
IMPLEMENTATIONS: dict = {B200FusedExperts.name: B200FusedExperts}


def get_implementation(name: str) -> MoEImplementation:
    if name not in IMPLEMENTATIONS:
        raise ValueError(f"Unknown implementation '{name}'. Available: {sorted(IMPLEMENTATIONS)}")
    return IMPLEMENTATIONS[name]()
