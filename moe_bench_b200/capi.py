"""ctypes binding of ``libmoe_bench_b200.so`` (declared in ``include/moe_bench_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Tensors are passed as raw device pointers and the current torch stream
is used, so calls are ordered with surrounding torch work.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmoe_bench_b200.so")

ABI_VERSION = 5
PRECISION_BF16 = 0
PRECISION_FP8 = 1
PRECISION_FP16 = 2
PAD_ROWS_BF16 = 16
PAD_ROWS_FP8 = 128

c_i32, c_i64, c_vp = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol the header declares.
SIGNATURES = {
    "mb200_abi_version": (c_i32, []),
    "mb200_last_error": (ctypes.c_char_p, []),
    "mb200_route_topk": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp]),
    "mb200_row_capacity": (c_i64, [c_i64, c_i32, c_i32, c_i32]),
    "mb200_align_scratch_bytes": (c_i64, [c_i64, c_i32, c_i32]),
    "mb200_align": (c_i32, [c_vp, c_i64, c_i32, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_vp, c_vp]),
    "mb200_align_noalloc": (c_i32, [c_vp, c_i64, c_i32, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_vp]),
    "mb200_group_quant_fp8": (c_i32, [c_vp, c_i64, c_i32, c_vp, c_vp, c_vp]),
    "mb200_grouped_gemm_bf16": (
        c_i32,
        [c_i32, c_vp, c_i64, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp],
    ),
    "mb200_grouped_gemm_bf16_gated": (
        c_i32,
        [c_vp, c_i64, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_i32, c_vp],
    ),
    "mb200_workspace_bytes": (c_i64, [c_i32, c_i64, c_i32, c_i32, c_i32, c_i32]),
    "mb200_forward_layout": (c_i32, [c_i32, c_i64, c_i32, c_i32, c_i32, c_i32, c_i64, c_vp]),
    "mb200_moe_forward_bf16": (
        c_i32,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp, c_i64, c_i32, c_vp],
    ),
    "mb200_moe_forward_fp16": (
        c_i32,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp, c_i64, c_i32, c_vp],
    ),
    "mb200_grouped_gemm_fp8": (
        c_i32,
        [c_i32, c_vp, c_vp, c_i64, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
         c_i32, c_vp],
    ),
    "mb200_grouped_gemm_fp8_cols": (
        c_i32,
        [c_i32, c_vp, c_vp, c_i64, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
         c_i32, c_vp],
    ),
    "mb200_moe_forward_fp8": (
        c_i32,
        [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32, c_vp, c_i64,
         c_i32, c_vp],
    ),
    "mb200_dist_symmetric_bytes": (c_i64, [c_i32, c_i64, c_i32, c_i32, c_i32]),
    "mb200_dist_workspace_bytes": (c_i64, [c_i32, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32]),
    "mb200_dist_forward": (
        c_i32,
        [c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i32, c_i32, c_i32, c_i32,
         c_i32, c_i32, c_i32, c_vp, c_i64, ctypes.c_uint32, c_vp, c_i64, c_i32, c_vp],
    ),
    "mb200_peer_barrier": (c_i32, [c_vp, c_i32, c_i32, ctypes.c_uint32, c_vp, c_vp]),
    "mb200_ipc_alloc": (c_i32, [c_i64, c_vp, c_vp]),
    "mb200_ipc_open": (c_i32, [c_vp, c_vp]),
    "mb200_ipc_close": (c_i32, [c_vp]),
    "mb200_ipc_free": (c_i32, [c_vp]),
    "mb200_set_stage_events": (c_i32, [c_vp, c_i32]),
    "mb200_set_fp8_scale_format": (c_i32, [c_i32]),
    "mb200_set_comm_only": (c_i32, [c_i32]),
    "mb200_read_status": (c_i32, [c_vp, c_vp, c_vp]),
}


class MB200Error(RuntimeError):
    """A library call returned a non-zero status."""


_lib: Optional[ctypes.CDLL] = None


def load_library(path: str) -> ctypes.CDLL:
    """Open a build of the library, set the prototypes and check its ABI version."""
    if not os.path.exists(path):
        raise MB200Error(
            f"{path} is missing: build it with `python -m moe_bench_b200.build` "
            "(there is no non-CUDA fallback)"
        )
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.mb200_abi_version() != ABI_VERSION:
        raise MB200Error(
            f"{path} has ABI version {lib.mb200_abi_version()}, this package needs {ABI_VERSION}: "
            "rebuild with `python -m moe_bench_b200.build --force`"
        )
    return lib


def load() -> ctypes.CDLL:
    """Load the shared library (once) and set the prototypes."""
    global _lib
    if _lib is None:
        _lib = load_library(LIB_PATH)
    return _lib


def use_library(lib: ctypes.CDLL) -> None:
    """Route every later call of this module to ``lib`` (a result of ``load_library``);
    lets one process compare two builds."""
    global _lib
    _lib = lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise MB200Error(f"{what} failed (status {rc}): {load().mb200_last_error().decode()}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda or not t.is_contiguous() or t.dtype != dtype:
        raise MB200Error(f"{name}: need a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}")


def check_problem_tensors(problem, dtype) -> None:
    """The layer entry points take raw pointers: refuse tensors of another dtype, device or
    layout here instead of computing on garbage (called from ``setup()``, not in the timed path)."""
    _need(problem.hidden_states, dtype, "hidden_states")
    _need(problem.topk_ids, torch.int32, "topk_ids")
    _need(problem.topk_weights, torch.float32, "topk_weights")
    for name in ("w1", "w2"):
        w = getattr(problem, name)
        if not w.is_cuda or not w.is_contiguous():
            raise MB200Error(f"{name}: need a contiguous CUDA tensor")
    if problem.w1.dtype != problem.w2.dtype:
        raise MB200Error(f"w1 is {problem.w1.dtype} but w2 is {problem.w2.dtype}")
    if problem.expert_map is not None:
        _need(problem.expert_map, torch.int32, "expert_map")
        if problem.topk_ids.numel() and int(problem.topk_ids.max()) >= problem.expert_map.numel():
            raise MB200Error("topk_ids holds an expert id beyond the end of expert_map")
    if problem.topk_ids.numel() and int(problem.topk_ids.min()) < 0:
        raise MB200Error("topk_ids holds a negative expert id")


def row_capacity(tokens: int, topk: int, local_experts: int, pad_rows: int = PAD_ROWS_BF16) -> int:
    return int(load().mb200_row_capacity(tokens, topk, local_experts, pad_rows))


def workspace_bytes(precision: int, tokens: int, hidden: int, intermediate: int, local_experts: int, topk: int) -> int:
    n = int(load().mb200_workspace_bytes(precision, tokens, hidden, intermediate, local_experts, topk))
    if n < 0:
        raise MB200Error(f"workspace_bytes: {load().mb200_last_error().decode()}")
    return n


LAYOUT_FIELDS = ("pad_rows", "row_capacity", "counts", "mtile_prefix", "sorted_ids", "inverse", "rows", "row_scales",
                 "act", "y")


def forward_layout(precision: int, tokens: int, hidden: int, intermediate: int, local_experts: int, topk: int,
                   expected_rows: int) -> dict:
    """Padding, row capacity and the byte offsets of the forward's tables inside its workspace."""
    out = (ctypes.c_int64 * 10)()
    _check(load().mb200_forward_layout(precision, tokens, hidden, intermediate, local_experts, topk, expected_rows,
                                       out), "forward_layout")
    return dict(zip(LAYOUT_FIELDS, [int(v) for v in out]))


def route_topk(logits: torch.Tensor, topk: int):
    """softmax -> top-k -> renormalise on the GPU; returns (ids int32, weights fp32)."""
    _need(logits, torch.float32, "logits")
    t, e = logits.shape
    ids = torch.empty(t, topk, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, topk, dtype=torch.float32, device=logits.device)
    _check(load().mb200_route_topk(_ptr(logits), t, e, topk, _ptr(ids), _ptr(w), _stream(logits.device)), "route_topk")
    return ids, w


def align(topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor], local_experts: int,
          pad_rows: int = PAD_ROWS_BF16):
    """Sort-and-pad to ``pad_rows``; returns (counts[E], mtile_prefix[E+1], sorted_ids[cap], inverse[T*k])."""
    _need(topk_ids, torch.int32, "topk_ids")
    if expert_map is not None:
        _need(expert_map, torch.int32, "expert_map")
    t, k = topk_ids.shape
    dev = topk_ids.device
    cap = row_capacity(t, k, local_experts, pad_rows)
    counts = torch.empty(local_experts, dtype=torch.int32, device=dev)
    prefix = torch.empty(local_experts + 1, dtype=torch.int32, device=dev)
    sorted_ids = torch.full((max(cap, 1),), -2, dtype=torch.int32, device=dev)[:cap]
    inverse = torch.empty(max(t * k, 1), dtype=torch.int32, device=dev)
    scratch = torch.empty(load().mb200_align_scratch_bytes(t, k, local_experts), dtype=torch.uint8, device=dev)
    _check(
        load().mb200_align(
            _ptr(topk_ids), t, k, _ptr(expert_map), local_experts, _ptr(counts), _ptr(prefix),
            _ptr(sorted_ids), _ptr(inverse), cap, pad_rows, _ptr(scratch), _stream(dev),
        ),
        "align",
    )
    return counts, prefix, sorted_ids, inverse[: t * k]


def align_noalloc(topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor], local_experts: int, outputs=None,
                  pad_rows: int = PAD_ROWS_BF16):
    """Sort-and-pad through the entry point that needs no scratch buffer.

    For hosts that may not allocate device memory while running (a server
    whose pool owns all of HBM, a latency-bound decode loop): the library's
    built-in 1 MiB array replaces the scratch tensor.  Pass ``outputs`` =
    ``(counts, mtile_prefix, sorted_ids, inverse)`` preallocated to make the
    whole call allocation-free; without it the four output tensors are created
    here for convenience.  Limits: 256 local experts, 2**20 assignments; calls
    on one device must not overlap.
    """
    _need(topk_ids, torch.int32, "topk_ids")
    if expert_map is not None:
        _need(expert_map, torch.int32, "expert_map")
    t, k = topk_ids.shape
    dev = topk_ids.device
    if outputs is None:
        cap = row_capacity(t, k, local_experts, pad_rows)
        outputs = (
            torch.empty(local_experts, dtype=torch.int32, device=dev),
            torch.empty(local_experts + 1, dtype=torch.int32, device=dev),
            torch.full((cap,), -2, dtype=torch.int32, device=dev),
            torch.empty(max(t * k, 1), dtype=torch.int32, device=dev),
        )
    counts, prefix, sorted_ids, inverse = outputs
    _check(
        load().mb200_align_noalloc(
            _ptr(topk_ids), t, k, _ptr(expert_map), local_experts, _ptr(counts), _ptr(prefix),
            _ptr(sorted_ids), _ptr(inverse), sorted_ids.shape[0], pad_rows, _stream(dev),
        ),
        "align_noalloc",
    )
    return counts, prefix, sorted_ids, inverse[: t * k]


def group_quant_fp8(x: torch.Tensor):
    """Per-row, per-128 e4m3 quantisation; returns (q e4m3 [m,K], scales fp32 [m,K/128])."""
    _need(x, torch.bfloat16, "x")
    m, k = x.shape
    q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(m, k // 128, dtype=torch.float32, device=x.device)
    _check(load().mb200_group_quant_fp8(_ptr(x), m, k, _ptr(q), _ptr(s), _stream(x.device)), "group_quant_fp8")
    return q, s


def grouped_gemm_bf16(mode, a, w, hidden, intermediate, counts, prefix, sorted_ids, row_scale, out, status):
    """One grouped GEMM stage (mode 0 gate/up + SiLU-mul, mode 1 down + weight)."""
    dev = a.device
    _check(
        load().mb200_grouped_gemm_bf16(
            mode, _ptr(a), a.shape[0], _ptr(w), w.shape[0], hidden, intermediate, _ptr(counts),
            _ptr(prefix), _ptr(sorted_ids), _ptr(row_scale), _ptr(out), _ptr(status), dev.index or 0, _stream(dev),
        ),
        "grouped_gemm_bf16",
    )


def grouped_gemm_bf16_gated(a, w, hidden, intermediate, counts, prefix, sorted_ids, granule_done, granule_target,
                            out, status):
    """The gate/up stage for rows delivered by someone else: a token block is loaded once
    ``granule_done`` of each of its 16-row granules has reached ``granule_target``."""
    dev = a.device
    _need(granule_done, torch.int32, "granule_done")
    _need(status, torch.int32, "status")
    if status.numel() < 2:
        raise MB200Error("status: need the two-word head of a status block")
    _check(
        load().mb200_grouped_gemm_bf16_gated(
            _ptr(a), a.shape[0], _ptr(w), w.shape[0], hidden, intermediate, _ptr(counts), _ptr(prefix),
            _ptr(sorted_ids), _ptr(granule_done), granule_target, _ptr(out), _ptr(status), dev.index or 0,
            _stream(dev),
        ),
        "grouped_gemm_bf16_gated",
    )


def moe_forward_bf16(x, w1, w2, topk_ids, topk_weights, expert_map, out, workspace):
    """Enqueue the 16-bit layer forward on the current stream: bf16 tensors, or
    fp16 when ``x`` is ``torch.float16`` (weights and output must match)."""
    t, hidden = x.shape
    e_local, two_n, _ = w1.shape
    dev = x.device
    if not (x.dtype == w1.dtype == w2.dtype == out.dtype) or x.dtype not in (torch.bfloat16, torch.float16):
        raise MB200Error(f"moe_forward: tensors must all be bf16 or all fp16, got {x.dtype}/{w1.dtype}/{w2.dtype}/{out.dtype}")
    fn = load().mb200_moe_forward_fp16 if x.dtype == torch.float16 else load().mb200_moe_forward_bf16
    _check(
        fn(
            _ptr(x), _ptr(w1), _ptr(w2), _ptr(topk_ids), _ptr(topk_weights), _ptr(expert_map), _ptr(out),
            t, hidden, two_n // 2, e_local, topk_ids.shape[1], _ptr(workspace), workspace.numel(),
            dev.index or 0, _stream(dev),
        ),
        "moe_forward_bf16",
    )


def grouped_gemm_fp8(mode, a, a_scale_t, w, w_scale, hidden, intermediate, counts, prefix, sorted_ids,
                     row_scale, out, out_scale_t, status, cols: bool = False):
    """One fp8 grouped GEMM stage (mode 0 gate/up + SiLU-mul + re-quantise, mode 1 down + weight).
    ``cols``: schedule padded to 16 rows, tokens-on-columns kernel; else 128-row token tiles."""
    dev = a.device
    fn = load().mb200_grouped_gemm_fp8_cols if cols else load().mb200_grouped_gemm_fp8
    _check(
        fn(
            mode, _ptr(a), _ptr(a_scale_t), a.shape[0], _ptr(w), _ptr(w_scale), w.shape[0], hidden, intermediate,
            _ptr(counts), _ptr(prefix), _ptr(sorted_ids), _ptr(row_scale), _ptr(out), _ptr(out_scale_t),
            _ptr(status), dev.index or 0, _stream(dev),
        ),
        "grouped_gemm_fp8",
    )


def moe_forward_fp8(x, w1, w2, w1_scale, w2_scale, topk_ids, topk_weights, expert_map, out, workspace):
    """Enqueue the fp8 block-quantised layer forward on the current stream."""
    t, hidden = x.shape
    e_local, two_n, _ = w1.shape
    dev = x.device
    _check(
        load().mb200_moe_forward_fp8(
            _ptr(x), _ptr(w1), _ptr(w2), _ptr(w1_scale), _ptr(w2_scale), _ptr(topk_ids), _ptr(topk_weights),
            _ptr(expert_map), _ptr(out), t, hidden, two_n // 2, e_local, topk_ids.shape[1], _ptr(workspace),
            workspace.numel(), dev.index or 0, _stream(dev),
        ),
        "moe_forward_fp8",
    )


DIST_SEQ_STRIDE = 4


def dist_symmetric_bytes(precision: int, tokens: int, hidden: int, topk: int, world: int) -> int:
    n = int(load().mb200_dist_symmetric_bytes(precision, tokens, hidden, topk, world))
    if n < 0:
        raise MB200Error("dist_symmetric_bytes: bad shape")
    return n


def dist_workspace_bytes(precision, tokens, hidden, intermediate, local_experts, topk, world) -> int:
    n = int(load().mb200_dist_workspace_bytes(precision, tokens, hidden, intermediate, local_experts, topk, world))
    if n < 0:
        raise MB200Error(f"dist_workspace_bytes: {load().mb200_last_error().decode()}")
    return n


def peer_pointer_array(ptrs):
    """ctypes ``void*[world]`` from a list of integer device addresses."""
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def peer_barrier(ptr_array, rank: int, world: int, seq: int, status: Optional[torch.Tensor], device) -> None:
    if status is not None:
        _need(status, torch.int32, "status")
        if status.numel() < 4:
            raise MB200Error("status: need the four-word head of a status block")
    _check(load().mb200_peer_barrier(ptr_array, rank, world, seq, _ptr(status), _stream(device)), "peer_barrier")


def dist_forward(precision, expert_parallel, x, w1, w2, w1_scale, w2_scale, topk_ids, topk_weights, expert_map,
                 out, global_experts, rank, world, ptr_array, symmetric_bytes, seq_base, workspace):
    """Enqueue one distributed layer forward (EP or TP) on the current stream."""
    t, hidden = x.shape
    e_local, two_n, _ = w1.shape
    dev = x.device
    _check(
        load().mb200_dist_forward(
            precision, 1 if expert_parallel else 0, _ptr(x), _ptr(w1), _ptr(w2), _ptr(w1_scale), _ptr(w2_scale),
            _ptr(topk_ids), _ptr(topk_weights), _ptr(expert_map), _ptr(out), t, hidden, two_n // 2, e_local,
            global_experts, topk_ids.shape[1], rank, world, ptr_array, symmetric_bytes, seq_base & 0xFFFFFFFF,
            _ptr(workspace), workspace.numel(), dev.index or 0, _stream(dev),
        ),
        "dist_forward",
    )


def read_status(workspace: torch.Tensor) -> int:
    """Synchronise and return the workspace status word (0 = ok)."""
    val = ctypes.c_int32(0)
    _check(load().mb200_read_status(_ptr(workspace), ctypes.byref(val), _stream(workspace.device)), "read_status")
    return int(val.value)


STAGE_NAMES = ("align", "gather_rows", "gate_up_gemm", "down_gemm", "combine")


def set_stage_events(events) -> None:
    """Have forward calls from this thread record ``events`` (six
    ``torch.cuda.Event(enable_timing=True)``, already recorded once so their
    handles exist) around the five stages; ``None`` switches it off."""
    if not events:
        _check(load().mb200_set_stage_events(None, 0), "set_stage_events")
        return
    arr = (ctypes.c_void_p * len(events))(*[ev.cuda_event for ev in events])
    _check(load().mb200_set_stage_events(arr, len(events)), "set_stage_events")


FP8_SCALE_FORMATS = {"fp32": 0, "ue8m0": 1}


def set_fp8_scale_format(fmt: str) -> None:
    """Format of the fp8 activation scales computed by later calls from this thread:
    ``"fp32"`` (amax/448) or ``"ue8m0"`` (rounded up to a power of two)."""
    if fmt not in FP8_SCALE_FORMATS:
        raise MB200Error(f"fp8 scale format {fmt!r}: expected one of {sorted(FP8_SCALE_FORMATS)}")
    _check(load().mb200_set_fp8_scale_format(FP8_SCALE_FORMATS[fmt]), "set_fp8_scale_format")


def reference_fp8_scale_format() -> str:
    """What the reference's activation quantiser does on this box.  The reference calls
    vLLM's ``per_token_group_quant_fp8`` without saying which scale format it wants
    (reference.py:143-145), and vLLM then follows ``is_deep_gemm_e8m0_used()``: power-of-two
    scales on GPUs where its DeepGEMM path is enabled (Hopper, Blackwell), fp32 elsewhere.
    Without vLLM there is no reference to match and the plain fp32 format applies."""
    if not torch.cuda.is_available():
        return "fp32"
    try:
        from vllm.utils.deep_gemm import is_deep_gemm_e8m0_used

        return "ue8m0" if is_deep_gemm_e8m0_used() else "fp32"
    except Exception:  # noqa: BLE001
        return "fp32"


def use_reference_fp8_scale_format() -> str:
    """Select, for this thread's direct calls, the scale format the reference uses on this
    box; returns it ("fp32" or "ue8m0") so that a checker can compute in the same format."""
    fmt = reference_fp8_scale_format()
    set_fp8_scale_format(fmt)
    return fmt


def set_comm_only(enabled: bool) -> None:
    """Forward calls from this thread move data only (GEMM kernels run with zero K steps)."""
    _check(load().mb200_set_comm_only(1 if enabled else 0), "set_comm_only")


def read_kernel_clocks(workspace: torch.Tensor) -> dict:
    """SM clock (MHz) the two GEMM kernels of the last forward ran at, from the
    cycle/nanosecond pairs the kernels leave in the workspace head.  Synchronises."""
    torch.cuda.synchronize(workspace.device)
    vals = workspace[32:64].view(torch.int64).cpu().tolist()
    out = {}
    for name, (cyc, ns) in (("gate_up_gemm", vals[0:2]), ("down_gemm", vals[2:4])):
        out[name] = None if ns <= 0 else round(cyc / ns * 1e3, 1)
    return out
