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
    fed by TMA, fused SiLU-mul and combine weights) through the C ABI."""

    name = "b200"

    def __init__(self) -> None:
        self._key = None
        self._workspace = None
        self._out = None

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
        if prec != Precision.BF16:
            raise capi.MB200Error(f"precision {prec.value} is not built in this library version")
        capi.load()
        t, hidden = problem.hidden_states.shape
        e_local, two_n, _ = problem.w1.shape
        topk = problem.topk_ids.shape[1]
        nbytes = capi.workspace_bytes(capi.PRECISION_BF16, t, hidden, two_n // 2, e_local, topk)
        dev = problem.hidden_states.device
        # torch's caching allocator hands out 512-byte aligned blocks; over-allocate
        # and slice to the 1024-byte boundary the tile buffers need.
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        shift = (-raw.data_ptr()) % 1024
        self._workspace = raw[shift : shift + nbytes]
        self._workspace[:256].zero_()  # status word
        self._out = torch.empty(t, hidden, dtype=torch.bfloat16, device=dev)
        self._key = self._shape_key(problem)

    def run(self, problem: MoEProblem) -> torch.Tensor:
        if self._key != self._shape_key(problem):
            raise capi.MB200Error("run() called with a problem of another shape than setup()")
        expert_map = problem.expert_map
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
