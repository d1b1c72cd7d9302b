"""Workload description and seeded input generation for the MoE layer.

Host-side mirror of the moe_bench contract that every implementation of the
layer is fed from: the configuration schema (reference ``config.py:72-216``),
the ``MoEProblem`` / ``MoEWeights`` bundles (``data.py:24-75``) and the seeded
generators (``data.py:78-410``).  Names, argument meaning, tensor shapes and the
order in which random numbers are drawn are the reference's, so a problem built
here is byte-identical to one built by the reference on the same device with
the same seed; the code itself is written for this package.

The only intended difference: fp8 weight quantisation and the quant-config
record are restated here in plain torch (the reference takes them from vLLM,
``data.py:147-174``), so this module imports nothing but torch.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Optional

import torch

FP8_DTYPE = torch.float8_e4m3fn
FP8_MAX = 448.0


class ParallelMode(str, Enum):
    """TP shards every expert's intermediate dim; EP shards the expert set
    (reference ``config.py:18-35``)."""

    TP = "tp"
    EP = "ep"


class Distribution(str, Enum):
    """Token -> expert load shape (reference ``config.py:38-48``)."""

    BALANCED = "balanced"
    UNIFORM = "uniform"
    SKEWED = "skewed"
    SINGLE = "single"


class Precision(str, Enum):
    """GEMM operand precision (reference ``config.py:51-57``)."""

    BF16 = "bf16"
    FP16 = "fp16"
    FP8 = "fp8"


@dataclass
class RoutingConfig:
    """Reference ``config.py:60-69``."""

    distribution: Distribution = Distribution.BALANCED
    skew_alpha: float = 1.0
    num_active_experts: Optional[int] = None


_BASE_DTYPE = {
    Precision.BF16: torch.bfloat16,
    Precision.FP16: torch.float16,
    Precision.FP8: torch.bfloat16,  # fp8 keeps bf16 activations in and out
}


@dataclass
class MoEBenchConfig:
    """One benchmark workload (reference ``config.py:72-216``).

    Field names, defaults and the validation errors follow the reference so a
    YAML/dict written for it loads here unchanged.
    """

    hidden_size: int = 4096
    intermediate_size: int = 3072
    num_experts: int = 64
    topk: int = 8
    parallel_mode: ParallelMode = ParallelMode.TP
    world_size: int = 8
    precision: Precision = Precision.BF16
    block_shape: list = field(default_factory=lambda: [128, 128])
    num_tokens: list = field(default_factory=lambda: [1, 4, 16, 64, 256, 1024, 4096])
    routing: RoutingConfig = field(default_factory=RoutingConfig)
    distributed: bool = False
    all2all_backend: str = "allgather_reducescatter"
    warmup_iters: int = 10
    bench_iters: int = 50
    use_cuda_graph: bool = True
    seed: int = 0
    verify: bool = True
    verify_atol: Optional[float] = None
    verify_rtol: Optional[float] = None
    device: str = "cuda"
    output_json: Optional[str] = None

    def __post_init__(self) -> None:
        for key in ("hidden_size", "intermediate_size", "num_experts", "topk", "world_size"):
            if getattr(self, key) <= 0:
                raise ValueError(f"{key} must be positive")
        if self.all2all_backend == "naive":
            self.all2all_backend = "allgather_reducescatter"
        if self.topk > self.num_experts:
            raise ValueError(f"topk={self.topk} > num_experts={self.num_experts}")
        active = self.routing.num_active_experts
        if active is not None and not 1 <= active <= self.num_experts:
            raise ValueError(
                f"num_active_experts={active} out of range [1, num_experts={self.num_experts}]"
            )
        pool = self.num_experts if active is None else active
        if self.topk > pool:
            raise ValueError(
                f"topk={self.topk} > num_active_experts={pool}; "
                "cannot route to that many distinct experts"
            )
        if self.parallel_mode == ParallelMode.TP:
            if self.intermediate_size % self.world_size:
                raise ValueError(
                    f"intermediate_size={self.intermediate_size} not divisible "
                    f"by world_size={self.world_size} for TP mode"
                )
        elif self.num_experts % self.world_size:
            raise ValueError(
                f"num_experts={self.num_experts} not divisible by "
                f"world_size={self.world_size} for EP mode"
            )
        if self.precision == Precision.FP8 and len(self.block_shape) != 2:
            raise ValueError("block_shape must be [block_n, block_k] for fp8")

    @property
    def num_local_experts(self) -> int:
        if self.parallel_mode == ParallelMode.EP:
            return self.num_experts // self.world_size
        return self.num_experts

    @property
    def intermediate_shard(self) -> int:
        if self.parallel_mode == ParallelMode.TP:
            return self.intermediate_size // self.world_size
        return self.intermediate_size

    @property
    def torch_dtype(self) -> torch.dtype:
        return _BASE_DTYPE[self.precision]

    @classmethod
    def from_dict(cls, data: dict) -> "MoEBenchConfig":
        raw = dict(data)
        unknown = set(raw) - {f.name for f in dataclasses.fields(cls)}
        if unknown:
            raise ValueError(f"Unknown config keys: {sorted(unknown)}")
        if "parallel_mode" in raw:
            raw["parallel_mode"] = ParallelMode(raw["parallel_mode"])
        if "precision" in raw:
            raw["precision"] = Precision(raw["precision"])
        if isinstance(raw.get("routing"), dict):
            r = dict(raw["routing"])
            if "distribution" in r:
                r["distribution"] = Distribution(r["distribution"])
            raw["routing"] = RoutingConfig(**r)
        return cls(**raw)

    @classmethod
    def from_file(cls, path) -> "MoEBenchConfig":
        import yaml

        with open(path, encoding="utf-8") as fh:
            return cls.from_dict(yaml.safe_load(fh) or {})

    def to_dict(self) -> dict:
        out = dataclasses.asdict(self)
        out["parallel_mode"] = self.parallel_mode.value
        out["precision"] = self.precision.value
        out["routing"]["distribution"] = self.routing.distribution.value
        return out


def deepseek_v32_config(**overrides: Any) -> MoEBenchConfig:
    """The DeepSeek-V3.2 layer shape of reference ``configs/deepseek_v32.yaml:8-11``
    as a single-GPU compute-only workload (all 256 experts local, full
    intermediate size)."""
    base = dict(
        hidden_size=7168,
        intermediate_size=2048,
        num_experts=256,
        topk=8,
        parallel_mode=ParallelMode.TP,
        world_size=1,
        precision=Precision.BF16,
        routing=RoutingConfig(distribution=Distribution.UNIFORM),
        seed=0,
    )
    base.update(overrides)
    return MoEBenchConfig(**base)


@dataclass
class BlockQuantConfig:
    """fp8 block-quant metadata carried by a problem.

    Exposes the attributes the layer reads off vLLM's ``FusedMoEQuantConfig``
    in the reference (``reference.py:126-127``, ``data.py:169-174``):
    ``w1_scale`` ``(E, 2N/bn, K/bk)`` and ``w2_scale`` ``(E, K/bn, N/bk)`` in
    fp32, plus ``block_shape``.  A vLLM ``FusedMoEQuantConfig`` can be passed
    anywhere this type is accepted.
    """

    w1_scale: torch.Tensor
    w2_scale: torch.Tensor
    block_shape: list
    quant_dtype: torch.dtype = FP8_DTYPE


@dataclass
class MoEProblem:
    """Everything one forward of the layer consumes (reference ``data.py:24-61``).

    ``hidden_states (T, K)`` base dtype; ``w1 (E_local, 2*N_shard, K)`` with the
    gate rows first and the up rows second; ``w2 (E_local, K, N_shard)``;
    ``topk_ids (T, k)`` int32 global expert ids, distinct within a row;
    ``topk_weights (T, k)`` fp32; ``expert_map (E,)`` int32 global id -> local
    slot or -1 (EP only, else ``None``); ``quant_config`` for fp8, else ``None``.
    """

    config: MoEBenchConfig
    num_tokens: int
    hidden_states: torch.Tensor
    w1: torch.Tensor
    w2: torch.Tensor
    topk_ids: torch.Tensor
    topk_weights: torch.Tensor
    expert_map: Optional[torch.Tensor]
    quant_config: Optional[Any]

    @property
    def global_num_experts(self) -> int:
        return self.config.num_experts

    @property
    def num_local_assignments(self) -> int:
        """Assignments whose expert lives on this rank (synchronises the
        device, so call it outside timed code; reference ``data.py:56-61``)."""
        if self.expert_map is None:
            return self.topk_ids.numel()
        return int((self.expert_map[self.topk_ids.long()] >= 0).sum().item())


@dataclass
class MoEWeights:
    """Token-count independent part of a problem (reference ``data.py:64-75``)."""

    w1: torch.Tensor
    w2: torch.Tensor
    quant_config: Optional[Any]


_STREAM_INPUT = 0
_STREAM_WEIGHT = 1


def _mix_seed(*parts: int) -> int:
    """31-bit polynomial hash of the seed components (reference ``data.py:78-87``)."""
    acc = 0
    for part in parts:
        acc = (acc * 1_000_003 + part) & 0x7FFF_FFFF
    return acc


def per_block_cast_to_fp8(w: torch.Tensor, block_shape) -> tuple:
    """Block-quantise a 2-D weight to e4m3 with one fp32 scale per block.

    Restates what the reference obtains from vLLM 0.22.0
    ``vllm.utils.deep_gemm.per_block_cast_to_fp8`` (call sites
    ``data.py:157-158,359-360``) without power-of-two scales: zero-pad to whole
    blocks, ``sf = max(amax, 1e-4) / 448`` per block in fp32,
    ``q = (w * (1 / sf))`` rounded to nearest-even e4m3.
    """
    bm, bn = block_shape
    m, n = w.shape
    mp, np_ = -(-m // bm) * bm, -(-n // bn) * bn
    padded = torch.zeros(mp, np_, dtype=w.dtype, device=w.device)
    padded[:m, :n] = w
    blocks = padded.view(mp // bm, bm, np_ // bn, bn)
    amax = blocks.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    sf = amax / FP8_MAX
    q = (blocks * (1.0 / sf)).to(FP8_DTYPE)
    return q.view(mp, np_)[:m, :n].contiguous(), sf.view(mp // bm, np_ // bn)


def _gen_expert_chunk(config: MoEBenchConfig, global_e: int, shard: int, generator):
    """One expert's weight chunk for one shard, seeded by ``(seed, expert,
    shard)`` only (reference ``data.py:96-124``): ``w1 (2n, K) / sqrt(K)`` then
    ``w2 (K, n) / sqrt(n)`` from the same generator."""
    k, n = config.hidden_size, config.intermediate_shard
    generator.manual_seed(_mix_seed(config.seed, _STREAM_WEIGHT, global_e, shard))
    kw = dict(device=config.device, dtype=config.torch_dtype, generator=generator)
    w1 = torch.randn(2 * n, k, **kw) / (k**0.5)
    w2 = torch.randn(k, n, **kw) / (n**0.5)
    return w1, w2


def _pack_weights(config, w1_parts, w2_parts, s1_parts, s2_parts) -> MoEWeights:
    w1, w2 = torch.stack(w1_parts), torch.stack(w2_parts)
    if config.precision != Precision.FP8:
        return MoEWeights(w1, w2, None)
    qc = BlockQuantConfig(torch.stack(s1_parts), torch.stack(s2_parts), list(config.block_shape))
    return MoEWeights(w1, w2, qc)


def make_weights(config: MoEBenchConfig, rank: int = 0) -> MoEWeights:
    """``rank``'s expert weights (reference ``data.py:127-175``).  EP: rank r
    owns global experts ``[r*E_l, (r+1)*E_l)`` (shard 0); TP: every rank holds
    shard ``rank`` of every expert."""
    tp = config.parallel_mode == ParallelMode.TP
    fp8 = config.precision == Precision.FP8
    gen = torch.Generator(device=config.device)
    w1s, w2s, s1s, s2s = [], [], [], []
    for slot in range(config.num_local_experts):
        ge = slot if tp else rank * config.num_local_experts + slot
        w1, w2 = _gen_expert_chunk(config, ge, rank if tp else 0, gen)
        if fp8:
            w1, s1 = per_block_cast_to_fp8(w1, config.block_shape)
            w2, s2 = per_block_cast_to_fp8(w2, config.block_shape)
            s1s.append(s1)
            s2s.append(s2)
        w1s.append(w1)
        w2s.append(w2)
    return _pack_weights(config, w1s, w2s, s1s, s2s)


def _make_routing(config: MoEBenchConfig, num_tokens: int, generator):
    """``topk_ids`` (int32, distinct per row) by distribution and
    ``topk_weights = softmax(rand(T, k))`` (reference ``data.py:178-235``)."""
    dev, k = config.device, config.topk
    active = config.routing.num_active_experts
    active = config.num_experts if active is None else min(active, config.num_experts)
    dist = config.routing.distribution
    if dist == Distribution.SINGLE:
        ids = torch.arange(k, device=dev, dtype=torch.int32).repeat(num_tokens, 1)
    elif dist == Distribution.BALANCED:
        flat = torch.arange(num_tokens * k, device=dev, dtype=torch.int64) % active
        shift = (torch.arange(num_tokens, device=dev) % active).view(-1, 1)
        ids = ((flat.view(num_tokens, k) + shift) % active).to(torch.int32)
    else:
        if dist == Distribution.SKEWED:
            p = torch.arange(1, active + 1, device=dev, dtype=torch.float32) ** (
                -config.routing.skew_alpha
            )
        else:
            p = torch.ones(active, device=dev, dtype=torch.float32)
        p = (p / p.sum()).unsqueeze(0).expand(num_tokens, active)
        ids = torch.multinomial(p, k, replacement=False, generator=generator).to(torch.int32)
    logits = torch.rand(num_tokens, k, device=dev, dtype=torch.float32, generator=generator)
    return ids, torch.softmax(logits, dim=-1)


def _make_expert_map(config: MoEBenchConfig, rank: int):
    """EP global id -> local slot table (reference ``data.py:238-253``)."""
    if config.parallel_mode != ParallelMode.EP:
        return None
    el = config.num_local_experts
    table = torch.full((config.num_experts,), -1, device=config.device, dtype=torch.int32)
    table[rank * el : (rank + 1) * el] = torch.arange(el, device=config.device, dtype=torch.int32)
    return table


def _input_rank(config: MoEBenchConfig, rank: int) -> int:
    """Reference ``data.py:256-265``."""
    return rank if (config.distributed or config.parallel_mode == ParallelMode.EP) else 0


def _gen_input(config: MoEBenchConfig, num_tokens: int, input_rank: int):
    """Hidden states, then routing, from one generator (reference
    ``data.py:268-288``; the draw order is part of the contract)."""
    gen = torch.Generator(device=config.device)
    gen.manual_seed(_mix_seed(config.seed, _STREAM_INPUT, num_tokens, input_rank))
    x = torch.randn(
        num_tokens, config.hidden_size, device=config.device, dtype=config.torch_dtype, generator=gen
    )
    ids, wts = _make_routing(config, num_tokens, gen)
    return x, ids, wts


def make_problem(config, num_tokens: int, rank: int = 0, weights: Optional[MoEWeights] = None):
    """Reference ``data.py:291-321``."""
    x, ids, wts = _gen_input(config, num_tokens, _input_rank(config, rank))
    if weights is None:
        weights = make_weights(config, rank)
    return MoEProblem(
        config, num_tokens, x, weights.w1, weights.w2, ids, wts,
        _make_expert_map(config, rank), weights.quant_config,
    )


def make_logical_weights(config: MoEBenchConfig) -> MoEWeights:
    """All global experts, unsharded (reference ``data.py:324-376``): TP
    concatenates the per-shard gate rows, then the per-shard up rows, and the
    ``w2`` column blocks."""
    shards = range(config.world_size) if config.parallel_mode == ParallelMode.TP else (0,)
    fp8 = config.precision == Precision.FP8
    gen = torch.Generator(device=config.device)
    w1s, w2s, s1s, s2s = [], [], [], []
    for e in range(config.num_experts):
        chunks = [_gen_expert_chunk(config, e, s, gen) for s in shards]
        halves = [c[0].chunk(2, dim=0) for c in chunks]
        w1 = torch.cat([h[0] for h in halves] + [h[1] for h in halves], dim=0)
        w2 = torch.cat([c[1] for c in chunks], dim=1)
        if fp8:
            w1, s1 = per_block_cast_to_fp8(w1, config.block_shape)
            w2, s2 = per_block_cast_to_fp8(w2, config.block_shape)
            s1s.append(s1)
            s2s.append(s2)
        w1s.append(w1)
        w2s.append(w2)
    return _pack_weights(config, w1s, w2s, s1s, s2s)


def make_golden_problem(config, num_tokens: int, rank: int, weights: Optional[MoEWeights] = None):
    """``rank``'s own tokens through the full model (reference ``data.py:379-410``)."""
    if weights is None:
        weights = make_logical_weights(config)
    x, ids, wts = _gen_input(config, num_tokens, rank)
    return MoEProblem(config, num_tokens, x, weights.w1, weights.w2, ids, wts, None, weights.quant_config)
