"""The distributed plugin: a moe_bench ``DistributedScheme`` (one rank's full
layer including dispatch and combine) backed by the sm_100a library.

``DistContext``, ``DistributedScheme`` and the registry mirror reference
``context.py:18-32`` and ``schemes.py:40-61,147-170``; ``B200Scheme`` can be put
into the reference's own ``SCHEMES`` table (in every spawned worker, since
``mp.spawn`` re-imports modules: ``distributed.py:99``).

Where the reference's serial scheme all-gathers every token and reduce-scatters
a mostly empty result (``schemes.py:117-143``), this scheme keeps each rank's
staged tokens in a buffer all peers have mapped and lets kernels pull exactly
the rows they need over NVLink (fp8 rows + scales for fp8 problems).  Both
parallel modes and all three precisions go through one entry point.
"""

from __future__ import annotations

import ctypes
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist

from . import capi
from .problem import MoEProblem, ParallelMode, Precision


@dataclass(frozen=True)
class DistContext:
    """Handles for one rank (reference context.py:18-32)."""

    rank: int
    world_size: int
    local_rank: int
    device: Any
    group: Optional[Any] = None

    @property
    def is_rank0(self) -> bool:
        return self.rank == 0


class DistributedScheme(ABC):
    """One rank's full MoE layer including communication (reference schemes.py:40-61)."""

    name: str

    def setup(self, problem: MoEProblem, ctx: DistContext) -> None:
        """Optional one-time, untimed setup."""

    @abstractmethod
    def run(self) -> torch.Tensor:
        """Full layer on this rank; returns ``(num_tokens, hidden)``."""
        raise NotImplementedError

    def close(self) -> None:
        """Optional teardown."""


class PeerBuffer:
    """A zero-filled device buffer of identical size on every rank that all
    ranks of the group have mapped.  ``ptrs[r]`` is rank r's buffer as an
    address valid in this process.

    Backend 1: torch's symmetric-memory allocator.  Backend 2 (if that is not
    usable): ``cudaMalloc`` + CUDA IPC handles exchanged over the process group.
    World size 1 needs neither.
    """

    def __init__(self, nbytes: int, ctx: DistContext):
        self.nbytes = nbytes
        self.rank, self.world = ctx.rank, ctx.world_size
        self._tensor = None
        self._ipc_own = None
        self._ipc_opened = []
        self.backend = None
        dev = torch.device(ctx.device)
        group = ctx.group if ctx.group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        if self.world == 1:
            raw = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=dev)
            shift = (-raw.data_ptr()) % 1024
            self._tensor = raw[shift : shift + nbytes]
            self.ptrs = [self._tensor.data_ptr()]
            self.backend = "local"
            return
        err = None
        try:
            import torch.distributed._symmetric_memory as symm

            t = symm.empty(nbytes, dtype=torch.uint8, device=dev)
            hdl = symm.rendezvous(t, group)
            t.zero_()
            self._tensor, self._hdl = t, hdl
            self.ptrs = [int(p) for p in hdl.buffer_ptrs]
            self.backend = "symmetric_memory"
        except Exception as exc:  # noqa: BLE001
            err = exc
        # every rank must take the same branch
        flags = [None] * self.world
        dist.all_gather_object(flags, self.backend is not None, group=group)
        if not all(flags):
            self._tensor = None
            self._init_ipc(nbytes, group, err)
        if any(p % 1024 for p in self.ptrs):
            raise capi.MB200Error("peer buffer is not 1024-byte aligned")
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def _init_ipc(self, nbytes, group, first_error):
        lib = capi.load()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        rc = lib.mb200_ipc_alloc(nbytes, ctypes.byref(ptr), handle)
        if rc != 0:
            raise capi.MB200Error(
                f"no way to share GPU memory between ranks: symmetric memory failed ({first_error!r}) "
                f"and ipc_alloc failed: {lib.mb200_last_error().decode()}"
            )
        self._ipc_own = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self._ipc_own)
                continue
            peer = ctypes.c_void_p()
            rc = lib.mb200_ipc_open(ctypes.create_string_buffer(raw, 64), ctypes.byref(peer))
            if rc != 0:
                raise capi.MB200Error(f"ipc_open for rank {r} failed: {lib.mb200_last_error().decode()}")
            self._ipc_opened.append(peer.value)
            self.ptrs.append(peer.value)
        self.backend = "cuda_ipc"

    def close(self):
        lib = capi.load()
        for p in self._ipc_opened:
            lib.mb200_ipc_close(p)
        self._ipc_opened = []
        if self._ipc_own is not None:
            lib.mb200_ipc_free(self._ipc_own)
            self._ipc_own = None
        self._tensor = None


class B200Scheme(DistributedScheme):
    """EP (dispatch + grouped GEMMs + combine) and TP (gather + GEMMs + output
    reduce) on hand-written sm_100a kernels over NVLink peer memory."""

    name = "b200"

    # fp8 activation scale format: None = what the reference does on this box (asked of vLLM
    # in setup()), or "fp32" / "ue8m0" to fix it
    fp8_scale_format = None
    # limits in milliseconds of one in-kernel wait and of one cross-GPU barrier (0 = the
    # library's defaults of 4 s and 3 s); raise the second where ranks can be further apart
    wait_limit_ms = 0
    barrier_limit_ms = 0

    def __init__(self) -> None:
        self._buf = None
        self._seq = 0

    def setup(self, problem: MoEProblem, ctx: DistContext) -> None:
        if not problem.hidden_states.is_cuda:
            raise capi.MB200Error("B200Scheme needs CUDA tensors; there is no CPU path")
        cfg = problem.config
        prec = Precision(cfg.precision.value)
        capi.load()
        self.ctx, self.problem = ctx, problem
        self._fp8 = prec == Precision.FP8
        self._ep = ParallelMode(cfg.parallel_mode.value) == ParallelMode.EP
        self._precision = {Precision.BF16: capi.PRECISION_BF16, Precision.FP8: capi.PRECISION_FP8,
                           Precision.FP16: capi.PRECISION_FP16}[prec]
        self._dtype = torch.float16 if prec == Precision.FP16 else torch.bfloat16
        if problem.hidden_states.dtype != self._dtype:
            raise capi.MB200Error(f"{prec.value} problem with {problem.hidden_states.dtype} hidden_states")
        self._w1_scale = self._w2_scale = None
        if self._fp8:
            qc = problem.quant_config
            if qc is None or list(qc.block_shape) != [128, 128]:
                raise capi.MB200Error("fp8 needs quant_config with block_shape [128, 128]")
            self._w1_scale = qc.w1_scale.to(torch.float32).contiguous()
            self._w2_scale = qc.w2_scale.to(torch.float32).contiguous()
            self._scale_format = self.fp8_scale_format or capi.reference_fp8_scale_format()
        if self._ep and problem.expert_map is None:
            raise capi.MB200Error("expert-parallel problem without expert_map")
        capi.check_problem_tensors(problem, self._dtype)
        t, hidden = problem.hidden_states.shape
        e_local, two_n, _ = problem.w1.shape
        topk = problem.topk_ids.shape[1]
        world = ctx.world_size
        dev = problem.hidden_states.device
        self._sym_bytes = capi.dist_symmetric_bytes(self._precision, t, hidden, topk, world)
        self._buf = PeerBuffer(self._sym_bytes, ctx)
        self._ptr_array = capi.peer_pointer_array(self._buf.ptrs)
        nbytes = capi.dist_workspace_bytes(self._precision, t, hidden, two_n // 2, e_local, topk, world)
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        shift = (-raw.data_ptr()) % 1024
        self._workspace = raw[shift : shift + nbytes]
        self._workspace[:256].zero_()  # status block: [0] failure code, [1] wait limit, [2] barrier limit (ms)
        head = self._workspace[:256].view(torch.int32)
        head[1], head[2] = int(self.wait_limit_ms), int(self.barrier_limit_ms)
        self._out = torch.empty(t, hidden, dtype=self._dtype, device=dev)
        self._hidden = problem.hidden_states.contiguous()
        self._ids = problem.topk_ids.contiguous()
        self._weights = problem.topk_weights.contiguous()
        self._seq = 0
        torch.cuda.synchronize(dev)

    def run(self) -> torch.Tensor:
        p = self.problem
        if self._fp8:
            capi.set_fp8_scale_format(self._scale_format)
        capi.dist_forward(
            self._precision, self._ep, self._hidden, p.w1, p.w2, self._w1_scale, self._w2_scale, self._ids,
            self._weights, p.expert_map if self._ep else None, self._out, p.config.num_experts, self.ctx.rank,
            self.ctx.world_size, self._ptr_array, self._sym_bytes, self._seq, self._workspace,
        )
        self._seq += capi.DIST_SEQ_STRIDE
        return self._out

    def run_comm_only(self) -> torch.Tensor:
        """One forward with the arithmetic switched off: staging, barriers, routing exchange,
        dispatch of rows and combine traffic only (for the decomposition of a step into
        computation and communication; the returned tensor means nothing)."""
        capi.set_comm_only(True)
        try:
            return self.run()
        finally:
            capi.set_comm_only(False)

    def device_status(self) -> int:
        return capi.read_status(self._workspace)

    def close(self) -> None:
        if self._buf is not None:
            torch.cuda.synchronize()
            if self.ctx.world_size > 1:
                dist.barrier(group=self.ctx.group)
            self._buf.close()
            self._buf = None


SCHEMES: dict = {B200Scheme.name: B200Scheme}


def get_scheme(name: str) -> DistributedScheme:
    if name not in SCHEMES:
        raise ValueError(f"Unknown scheme '{name}'. Available: {sorted(SCHEMES)}")
    return SCHEMES[name]()
