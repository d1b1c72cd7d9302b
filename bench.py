"""Benchmark of the MoE layer forward (DeepSeek-V3.2 shape, bf16, compute-only).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl b200|reference]

One step = one forward of the layer over one batch of T tokens per GPU
(hidden 7168, intermediate 2048, 256 experts, top-8, uniform routing, seed 0;
synthetic inputs from the package's seeded generator).  The metric is the
harness's TFLOP/s: 6*N*K flops per computed assignment divided by the layer
latency; ``ms_per_step`` is that latency.  Prints ONE JSON line on rank 0.

* ``value``     inputs resident in HBM, device-timed with CUDA events.
* ``e2e``       the same metric through the plugin call with the step's inputs
                copied from pinned host memory and the output copied back, all
                inside the timed region.  ``e2e.value`` is the throughput with two
                steps in flight (copies on their own streams overlap the
                neighbouring steps' kernels, as a server feeds the layer);
                ``e2e.serial_*`` is one step at a time (copy in, run, copy out).
* ``roofline``  the gate/up grouped GEMM (the dominant kernel), its duration read
                from events recorded around it inside the timed region.
* ``cpu_baseline`` / ``--impl reference``: the CPU oracle (a port of the
                reference's torch forward) on a bounded sample of the workload.

With N > 1 the layer runs expert-parallel over the N GPUs (the reference's
distributed EP mode): rank r owns 256/N experts and its own shard of T tokens,
token dispatch (pulls) and the weighted combine (pushes) cross NVLink inside the
library's GEMM kernels.  Per-GPU work is fixed (weak scaling); the value is the sum over ranks
divided by the slowest rank's time.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, EXPERTS, TOPK = 7168, 2048, 256, 8  # EXPERTS can be lowered with --experts for profiling
METRIC, UNIT = "moe_layer_tflops", "TFLOP/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.errors, self.power_w, self._index = set(), 0.0, index
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self._nv = None

    _NAMES = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
    }

    def _reason_bits(self):
        """Current clock-event (throttle) reason bitmask; NVML renamed the call, so try both."""
        nv = self._nv
        for fn in ("nvmlDeviceGetCurrentClocksEventReasons", "nvmlDeviceGetCurrentClocksThrottleReasons"):
            if hasattr(nv, fn):
                try:
                    return int(getattr(nv, fn)(self._h))
                except Exception as exc:  # noqa: BLE001
                    self.errors.add(f"{fn}: {exc}")
        return None

    def _reasons_from_smi(self):
        """Fallback when NVML does not answer: the same flags through nvidia-smi (read-only query)."""
        import subprocess

        fields = ["sw_power_cap", "hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]
        try:
            out = subprocess.run(
                ["nvidia-smi", "-i", str(self._index), "--format=csv,noheader",
                 "--query-gpu=" + ",".join("clocks_event_reasons." + f for f in fields)],
                capture_output=True, text=True, timeout=5).stdout.strip().split(",")
            for name, val in zip(fields, out):
                if val.strip().lower() == "active":
                    self.reasons.add(name)
        except Exception as exc:  # noqa: BLE001
            self.errors.add(f"nvidia-smi: {exc}")

    def _loop(self):
        nv = self._nv
        n = 0
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.power_w = max(self.power_w, nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception as exc:  # noqa: BLE001
                self.errors.add(f"clock/power: {exc}")
            bits = self._reason_bits()
            if bits is None:
                if n % 20 == 0:
                    self._reasons_from_smi()
            else:
                for bit, name in self._NAMES.items():
                    if bits & bit:
                        self.reasons.add(name)
            n += 1
            time.sleep(0.01)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        out = {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
               "samples": len(s), "power_w_max": round(self.power_w, 1)}
        if self.errors:
            out["sampler_errors"] = sorted(self.errors)[:3]
        return out


def _touched_experts(topk_ids) -> int:
    import torch

    return int(torch.unique(topk_ids).numel())


def _cpu_sample_problem(tokens: int):
    """Bounded CPU sample: the first four experts of the layer with every
    assignment the T-token batch routes to them (the compute-only share of rank
    0 of a 64-way expert split, as the reference defines it)."""
    from moe_bench_b200 import problem as P

    cfg = P.MoEBenchConfig(
        hidden_size=HIDDEN, intermediate_size=INTER, num_experts=EXPERTS, topk=TOPK,
        parallel_mode=P.ParallelMode.EP, world_size=64, precision=P.Precision.BF16,
        routing=P.RoutingConfig(distribution=P.Distribution.UNIFORM), seed=0, device="cpu",
    )
    prob = P.make_problem(cfg, tokens, rank=0)
    # weights pre-converted to fp32 once, outside the timed loop
    prob = dataclasses.replace(prob, w1=prob.w1.float(), w2=prob.w2.float())
    return prob


def _staged_reference():
    """The reference's own harness modules, if the build staged them next to the oracle
    (they import vLLM, so this is slow the first time); None when they are not there or do
    not import on this box."""
    from oracle.stage_reference import staged_parent

    parent = staged_parent()
    if parent is None:
        return None
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    if parent not in sys.path:
        sys.path.insert(0, parent)
    try:
        import moe_bench.config as rc
        import moe_bench.data as rd
        import moe_bench.reference as rr
    except Exception:  # noqa: BLE001
        return None
    return rc, rd, rr


def _time_cpu_oracle(tokens: int, steps: int, warmup: int, budget_s: float = 25.0):
    """The reference's CPU forward on a bounded sample, all host cores: the reference's own
    ``reference_moe`` on its own generator's problem when its modules are staged
    (kind "reference"), else the oracle port on the package's byte-identical problem (kind "port")."""
    import torch

    from oracle import moe_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = _staged_reference()
    if ref is not None:
        rc, rd, rr = ref
        cfg = rc.MoEBenchConfig(
            hidden_size=HIDDEN, intermediate_size=INTER, num_experts=EXPERTS, topk=TOPK,
            parallel_mode=rc.ParallelMode.EP, world_size=64, precision=rc.Precision.BF16,
            routing=rc.RoutingConfig(distribution=rc.Distribution.UNIFORM), seed=0, device="cpu",
        )
        prob = rd.make_problem(cfg, tokens, rank=0)
        forward, kind = (lambda: rr.reference_moe(prob)), "reference"
        what = "the reference's own reference_moe on its own generator's problem"
    else:
        prob = _cpu_sample_problem(tokens)
        forward, kind = (lambda: O.reference_moe(prob)), "port"
        what = "the oracle port, weights pre-converted to fp32"
    assignments = prob.num_local_assignments
    flops = 6.0 * INTER * HIDDEN * assignments
    for _ in range(warmup):
        forward()
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        forward()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    avg = sum(times) / len(times)
    return {
        "value": flops / avg / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
        "sample": f"experts 0-3 of 256 with all {assignments} assignments of a {tokens}-token batch "
                  f"(DSv3.2 dims; {what}), {len(times)} passes, {avg * 1e3:.1f} ms each; the sample is one "
                  "host's work and does not grow with the GPU count",
        "ms_per_pass": avg * 1e3, "passes": len(times),
    }


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    res = _time_cpu_oracle(args.tokens, args.steps, min(args.warmup, 3), budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": res["passes"], "warmup": min(args.warmup, 3), "ms_per_step": res["ms_per_pass"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config_dict(args.tokens, world, "bf16", args.mode, args.distribution),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


class _LazyExperts:
    """Indexable stand-in for a stacked ``[E, ...]`` weight tensor that builds
    expert ``e`` when asked (the oracle only touches routed experts)."""

    def __init__(self, count, make):
        self.shape = (count,)
        self._make = make

    def __getitem__(self, e):
        return self._make(int(e))


def _lazy_logical_weights(cfg, P):
    import torch

    gen = torch.Generator(device=cfg.device)
    cache = {}

    tp = cfg.parallel_mode == P.ParallelMode.TP
    shards = range(cfg.world_size) if tp else (0,)

    def expert(e):
        if e not in cache:
            cache.clear()  # one expert at a time
            # the logical expert: TP concatenates the shards' gate rows, then their up rows, and
            # the w2 column blocks (reference data.py:340-357)
            chunks = [P._gen_expert_chunk(cfg, e, s, gen) for s in shards]
            halves = [c[0].chunk(2, dim=0) for c in chunks]
            w1 = torch.cat([h[0] for h in halves] + [h[1] for h in halves], dim=0)
            w2 = torch.cat([c[1] for c in chunks], dim=1)
            if cfg.precision == P.Precision.FP8:
                w1, s1 = P.per_block_cast_to_fp8(w1, cfg.block_shape)
                w2, s2 = P.per_block_cast_to_fp8(w2, cfg.block_shape)
                cache[e] = (w1, w2, s1, s2)
            else:
                cache[e] = (w1, w2, None, None)
        return cache[e]

    n = cfg.num_experts
    w1 = _LazyExperts(n, lambda e: expert(e)[0])
    w2 = _LazyExperts(n, lambda e: expert(e)[1])
    qc = None
    if cfg.precision == P.Precision.FP8:
        qc = P.BlockQuantConfig(_LazyExperts(n, lambda e: expert(e)[2]), _LazyExperts(n, lambda e: expert(e)[3]),
                                list(cfg.block_shape))
    return w1, w2, qc


def _time_vllm_baseline(prob, world, dev, flops_step, barrier, max_over_ranks, ours):
    """vLLM's Triton fused_experts (N=1) or the reference's serial scheme
    all-gather -> fused_experts -> reduce-scatter (N>1), timed like the main arm.
    A baseline, not an optimisation target; any failure is reported, not fatal."""
    import torch
    import torch.distributed as dist

    from moe_bench_b200 import baselines as B

    def agree(flag: float) -> bool:
        """True only if every rank says so (no collective of the baseline runs otherwise)."""
        if world == 1:
            return flag > 0
        t = torch.tensor([flag], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0)

    reason, run = "", None
    try:
        local = B.vllm_compute_only(prob)
        local()  # compiles the Triton kernels; a failure here involves no other rank
        torch.cuda.synchronize()
        run = local if world == 1 else B.vllm_serial_scheme(prob, world)
    except Exception as exc:  # noqa: BLE001
        reason, run = f"{type(exc).__name__}: {str(exc)[:200]}", None
    if not agree(1.0 if run is not None else 0.0):
        return {"unavailable": reason or "vLLM baseline could not be set up on another rank"}
    ms = diff = 0.0
    ok = 1.0
    try:
        for _ in range(3):
            res = run()
        barrier()
        n = 5
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            res = run()
        e.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(s.elapsed_time(e) / n)
        diff = float((res.float() - ours.float()).norm() / ours.float().norm().clamp_min(1e-12))
    except Exception as exc:  # noqa: BLE001
        ok, reason = 0.0, f"{type(exc).__name__}: {str(exc)[:200]}"
        if world > 1:
            raise  # a rank that fails inside the collectives cannot be recovered from
    if not ok:
        return {"unavailable": reason}
    return {
        "impl": "vLLM fused_experts (Triton)" if world == 1 else
                "all_gather + vLLM fused_experts + reduce_scatter (reference serial scheme)",
        "ms_per_step": ms, "value": flops_step * world / (ms * 1e-3) / 1e12, "unit": UNIT,
        "rel_diff_vs_b200": diff,
    }


def _config_dict(tokens: int, world: int, precision: str = "bf16", mode: str = "ep", distribution: str = "uniform"):
    wgb = 11.3 if precision == "fp8" else 22.5
    return {
        "workload": f"dsv32_{precision}_compute_only_T{tokens}" + ("" if EXPERTS == 256 else f"_E{EXPERTS}"),
        "tokens_per_gpu": tokens, "hidden": HIDDEN,
        "intermediate": INTER, "experts": EXPERTS, "topk": TOPK, "routing": distribution, "seed": 0,
        "parallelism": "single GPU, all experts local" if world == 1 else
                       (f"ep{world}: {EXPERTS // world} experts and {tokens} own tokens per GPU, "
                        "dispatch by P2P pulls and combine by P2P pushes over NVLink, both inside the GEMM kernels" if mode == "ep" else
                        f"tp{world}: all experts, intermediate/{world} columns and {tokens} own tokens per GPU, "
                        "token gather and output reduce by P2P pulls over NVLink"),
        "l2": f"inputs larger than L2: {wgb} GB of expert weights are streamed every step",
    }


PREC_CODE = {"bf16": 0, "fp8": 1, "fp16": 2}
DIST_STAGES = ("stage_routing_align", "dispatch", "gate_up_gemm", "down_gemm", "combine")


class Env:
    """This process's place in the job: rank, device, and the two collectives the timing needs."""

    def __init__(self, rank: int, local_rank: int, world: int):
        import torch

        self.rank, self.local_rank, self.world = rank, local_rank, world
        self.dev = torch.device("cuda", local_rank)
        self.t_start = time.time()

    def barrier(self):
        import torch
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, v: float) -> float:
        import torch
        import torch.distributed as dist

        if self.world == 1:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def all_agree(self, flag: bool) -> bool:
        return self.max_over_ranks(0.0 if flag else 1.0) == 0.0

    def elapsed(self) -> float:
        """Seconds since the bench started, the same number on every rank."""
        return self.max_over_ranks(time.time() - self.t_start)


class Leg:
    """One workload on this rank: the problem bundle, the plugin (N = 1) or scheme
    (N > 1) instance set up for it, and ``run()`` = one forward."""

    def __init__(self, env: Env, precision: str, tokens: int, mode: str = "ep", distribution: str = "uniform",
                 weights=None, routing: str = "data"):
        from moe_bench_b200 import capi
        from moe_bench_b200 import gating as G
        from moe_bench_b200 import problem as P
        from moe_bench_b200.plugin import get_implementation

        self.env, self.precision, self.tokens, self.mode, self.distribution = env, precision, tokens, mode, distribution
        world, dev = env.world, env.dev
        kw = dict(device=str(dev), num_tokens=[tokens], num_experts=EXPERTS, precision=P.Precision(precision),
                  routing=P.RoutingConfig(distribution=P.Distribution(distribution)))
        if world == 1:
            self.cfg = P.deepseek_v32_config(**kw)
            self.weights = weights if weights is not None else P.make_weights(self.cfg)
            x, ids, wts = P._gen_input(self.cfg, tokens, 0)
            if routing == "logits":
                # gating front end: router logits -> top-k kernel instead of the generator's direct draw
                ids, wts = capi.route_topk(G.router_logits(self.cfg, tokens, 0), TOPK)
            self.prob = P.MoEProblem(self.cfg, tokens, x, self.weights.w1, self.weights.w2, ids, wts, None,
                                     self.weights.quant_config)
            self.impl = get_implementation("b200")
            self.impl.setup(self.prob)
            self.run = lambda: self.impl.run(self.prob)
            self.stage_names = capi.STAGE_NAMES
        else:
            from moe_bench_b200.scheme import DistContext, get_scheme

            self.cfg = P.deepseek_v32_config(parallel_mode=P.ParallelMode(mode), world_size=world, distributed=True,
                                             **kw)
            self.weights = weights if weights is not None else P.make_weights(self.cfg, env.rank)
            if routing == "logits":
                self.prob, _ = G.make_routed_problem(self.cfg, tokens, env.rank, weights=self.weights)
            else:
                self.prob = P.make_problem(self.cfg, tokens, env.rank, weights=self.weights)
            self.impl = get_scheme("b200")
            self.impl.setup(self.prob, DistContext(rank=env.rank, world_size=world, local_rank=env.local_rank,
                                                   device=dev))
            self.run = self.impl.run
            self.stage_names = DIST_STAGES
        self.x, self.ids, self.wts = self.prob.hidden_states, self.prob.topk_ids, self.prob.topk_weights
        self.tp = world > 1 and mode == "tp"
        self.n_local = INTER // world if self.tp else INTER      # intermediate columns this rank computes
        self.e_local = EXPERTS if (world == 1 or self.tp) else EXPERTS // world
        # whole-job flops of one step by the harness's formula (6*n*k per computed assignment, summed over ranks)
        self.flops_step = 6.0 * INTER * HIDDEN * tokens * TOPK

    def close(self):
        if self.env.world > 1:
            self.impl.close()
        self.impl = self.run = self.prob = None

    def workload(self) -> str:
        w = self.env.world
        par = "compute_only" if w == 1 else f"{self.mode}{w}"
        tag = "" if self.distribution == "uniform" else f"_{self.distribution}"
        return f"dsv32_{self.precision}_{par}_T{self.tokens}{tag}" + ("" if EXPERTS == 256 else f"_E{EXPERTS}")


def _time_leg(leg: Leg, steps: int, warmup: int, sample_clocks: bool = False):
    """W warm-up forwards, then K timed ones between a barrier + synchronize on both sides,
    CUDA events on the launching stream, the library's per-stage events inside; max over ranks."""
    import torch

    from moe_bench_b200 import capi

    env = leg.env
    for _ in range(warmup):
        leg.run()
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(steps)]
    for evs in stage_ev:
        for ev in evs:
            ev.record()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    clocks = ClockSampler(env.local_rank) if sample_clocks else None
    if clocks:
        clocks.__enter__()
    start.record()
    for i in range(steps):
        capi.set_stage_events(stage_ev[i])
        leg.run()
    end.record()
    torch.cuda.synchronize()
    if clocks:
        clocks.__exit__()
    capi.set_stage_events(None)
    env.barrier()
    ms_step = env.max_over_ranks(start.elapsed_time(end) / steps)
    status = leg.impl.device_status()
    if status != 0:
        raise RuntimeError(f"{leg.workload()}: device status {status}")
    stage_ms = [sum(evs[j].elapsed_time(evs[j + 1]) for evs in stage_ev) / steps for j in range(5)]
    return ms_step, stage_ms, (clocks.summary() if clocks else None)


def _verify_leg(leg: Leg, n_tokens: int = 256) -> dict:
    """Parity outside any timed region: ``n_tokens`` sampled tokens of this rank against the
    CPU oracle.  N > 1: the rank's tokens through ALL experts with the logical weights, built
    expert by expert on demand (reference distributed.py:64-84).  FAIL if any rank fails."""
    import torch

    from moe_bench_b200 import problem as P
    from oracle import moe_oracle as O

    env = leg.env
    out = leg.run().clone()
    n = min(n_tokens, leg.tokens)
    idx = torch.randperm(leg.tokens, generator=torch.Generator().manual_seed(0))[:n].to(env.dev)
    if env.world == 1:
        ref_w1, ref_w2, ref_qc = leg.weights.w1, leg.weights.w2, leg.weights.quant_config
    else:
        ref_w1, ref_w2, ref_qc = _lazy_logical_weights(leg.cfg, P)
    sub = P.MoEProblem(leg.cfg, n, leg.x[idx].contiguous(), ref_w1, ref_w2, leg.ids[idx].contiguous(),
                       leg.wts[idx].contiguous(), None, ref_qc)
    check = O.verify_output(leg.precision, out[idx], O.reference_moe(sub))
    passed = env.all_agree(check.passed)
    return {"verify": "ok" if passed else "FAIL", "verify_tokens": n, "rel_err": env.max_over_ranks(check.rel_err),
            "max_abs_err": env.max_over_ranks(check.max_abs_err), "_out": out,
            "verify_message": None if passed else check.message}


def _ring_tokens(leg: Leg):
    """All ranks' hidden states in this rank's ring order (own rank first), as the schedule numbers them."""
    import torch
    import torch.distributed as dist

    env = leg.env
    if env.world == 1:
        return leg.x
    full = torch.empty(env.world * leg.tokens, HIDDEN, dtype=leg.x.dtype, device=env.dev)
    dist.all_gather_into_tensor(full, leg.x.contiguous())
    blocks = full.view(env.world, leg.tokens, HIDDEN)
    order = [(env.rank + r) % env.world for r in range(env.world)]
    return blocks[order].reshape(env.world * leg.tokens, HIDDEN)


def _dispatch_exact(leg: Leg) -> dict:
    """The data-movement check the reference does before it looks at any output
    (tools/validate_push3.py:90-95): after a forward, the sorted row buffer the GEMM read must
    equal ``x_all[sorted_ids // k]`` byte for byte (fp8: the e4m3 bytes and the 1x128 scales of
    the quantised tokens).  Also counts the rows that crossed NVLink."""
    import torch

    from moe_bench_b200 import capi

    env = leg.env
    world, t = env.world, leg.tokens
    all_tokens = t * world
    expected = all_tokens * TOPK // world if (world > 1 and not leg.tp) else all_tokens * TOPK
    lay = capi.forward_layout(PREC_CODE[leg.precision], all_tokens, HIDDEN, leg.n_local, leg.e_local, TOPK, expected)
    leg.run()
    torch.cuda.synchronize()
    ws = leg.impl._workspace
    cap = lay["row_capacity"]
    sorted_ids = ws[lay["sorted_ids"]: lay["sorted_ids"] + cap * 4].view(torch.int32)
    prefix = ws[lay["mtile_prefix"]: lay["mtile_prefix"] + (leg.e_local + 1) * 4].view(torch.int32)
    used = int(prefix[-1].item()) * lay["pad_rows"]
    sorted_ids = sorted_ids[:used]
    valid = (sorted_ids >= 0).nonzero().flatten()
    tok = (sorted_ids[valid] // TOPK).long()
    x_ring = _ring_tokens(leg)
    fp8 = leg.precision == "fp8"
    eb = 1 if fp8 else 2
    rows = ws[lay["rows"]: lay["rows"] + cap * HIDDEN * eb]
    rows = rows.view(torch.uint8).view(cap, HIDDEN) if fp8 else rows.view(leg.x.dtype).view(cap, HIDDEN)
    if fp8:
        q, s = capi.group_quant_fp8(x_ring)
        q = q.view(torch.uint8)
        scales_t = ws[lay["row_scales"]: lay["row_scales"] + (HIDDEN // 128) * cap * 4].view(torch.float32)
        scales_t = scales_t.view(HIDDEN // 128, cap)
    ok = True
    for c0 in range(0, valid.numel(), 16384):  # bounded temporaries
        v, tk = valid[c0:c0 + 16384], tok[c0:c0 + 16384]
        if fp8:
            ok = ok and bool(torch.equal(rows[v], q[tk])) and bool(torch.equal(scales_t[:, v].t(), s[tk]))
        else:
            ok = ok and bool(torch.equal(rows[v], x_ring[tk]))
    remote_rows = int((tok >= t).sum().item()) if world > 1 else 0
    row_bytes = HIDDEN * eb + (HIDDEN // 128 * 4 if fp8 else 0)
    return {"exact": env.all_agree(ok), "rows": int(valid.numel()), "remote_rows": remote_rows,
            "remote_bytes": remote_rows * row_bytes, "pad_rows": lay["pad_rows"]}


def _repeat_identical(leg: Leg, first, n: int = 30) -> bool:
    """Race hunt: ``n`` more forwards, each compared bit for bit with the first result."""
    import torch

    same = True
    for _ in range(n):
        same = same and bool(torch.equal(leg.run(), first))
    return leg.env.all_agree(same)


def _measure_fp8_peak(dev) -> float:
    """Dense e4m3 x e4m3 tensor throughput of this GPU, TFLOP/s: cuBLASLt through
    ``torch._scaled_mm`` at 8192^3, a burst of 20 calls after 5 warm-ups.  The fp8
    counterpart of the measured bf16 figure the other rooflines use."""
    import torch

    n = 8192
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
    one = torch.ones((), device=dev)
    for _ in range(5):
        torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(20):
        torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    e.record()
    torch.cuda.synchronize()
    return 2.0 * n ** 3 / (s.elapsed_time(e) / 20 * 1e-3) / 1e12


_FP8_PEAK = {}


def _tensor_peak(precision: str, peaks: dict, dev):
    """(TFLOP/s, source) of the tensor roofline for a precision."""
    if precision != "fp8":
        return peaks["bf16_tflops"], peaks["source"] + " (burst)"
    if "v" not in _FP8_PEAK:
        try:
            _FP8_PEAK["v"] = (_measure_fp8_peak(dev), "measured in this run: torch._scaled_mm e4m3 8192^3, burst")
        except Exception as exc:  # noqa: BLE001
            _FP8_PEAK["v"] = (2.0 * peaks["bf16_tflops"],
                              f"2 x the bf16 figure (nominal ratio): fp8 GEMM probe failed: {type(exc).__name__}")
    return _FP8_PEAK["v"]


def _rank_work(leg: Leg):
    """(experts touched on this rank, assignments computed on this rank) from the actual routing."""
    import torch
    import torch.distributed as dist

    env = leg.env
    if env.world == 1:
        return _touched_experts(leg.ids), leg.tokens * TOPK
    ids_all = torch.empty(env.world * leg.tokens, TOPK, dtype=leg.ids.dtype, device=env.dev)
    dist.all_gather_into_tensor(ids_all, leg.ids.contiguous())
    if leg.tp:
        return int(torch.unique(ids_all).numel()), env.world * leg.tokens * TOPK
    lo = env.rank * leg.e_local
    mine = ids_all[(ids_all >= lo) & (ids_all < lo + leg.e_local)]
    return int(torch.unique(mine).numel()), int(mine.numel())


def _layer_roofline(leg: Leg, ms_step: float, peaks: dict) -> dict:
    """Roofline of the whole layer on the busiest rank: max(algorithmic bytes / measured HBM
    copy bandwidth, flops / measured tensor peak).  Algorithmic bytes = the weights of the
    experts the rank touches + its tokens in and out + routing; intermediates are not counted."""
    env = leg.env
    fp8 = leg.precision == "fp8"
    wb = 1 if fp8 else 2
    touched, local_assign = _rank_work(leg)
    tc_peak, tc_src = _tensor_peak(leg.precision, peaks, env.dev)
    nbytes = touched * 3 * leg.n_local * HIDDEN * wb + 2 * leg.tokens * HIDDEN * 2 + leg.tokens * TOPK * 8
    if fp8:
        nbytes += touched * 3 * (leg.n_local // 128) * (HIDDEN // 128) * 4
    flops = 6.0 * leg.n_local * HIDDEN * local_assign
    t_hbm, t_tc = nbytes / (peaks["hbm_gbs"] * 1e9), flops / (tc_peak * 1e12)
    roof_ms = env.max_over_ranks(max(t_hbm, t_tc) * 1e3)
    bound = "hbm" if t_hbm >= t_tc else "tensor"
    return {"layer_roofline_ms": roof_ms, "layer_roofline_frac": roof_ms / ms_step, "bound_rank0": bound,
            "tensor_peak_tflops": tc_peak, "tensor_peak_source": tc_src,
            "rank0": {"experts_touched": touched, "assignments": local_assign, "algorithmic_bytes": nbytes,
                      "algorithmic_flops": flops}}


def _ncu_traffic(kernel: str, precision: str, tokens: int, distribution: str, world: int):
    """DRAM bytes of one launch of ``kernel`` from the committed table of ncu captures
    (dram__bytes_read.sum + dram__bytes_write.sum of a small case), scaled by the expert
    count where the rows per expert match the capture; None when no capture applies."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
    if world != 1 or distribution != "uniform" or not os.path.exists(path):
        return None, None
    with open(path) as fh:
        table = json.load(fh)
    for cap in table.get("captures", []):
        if cap["kernel"] == kernel and cap["precision"] == precision and \
                tokens * cap["experts"] == EXPERTS * cap["tokens"]:
            scale = EXPERTS / cap["experts"]
            return cap["dram_bytes_per_launch"] * scale, (
                f"ncu capture of the {cap['experts']}-expert / {cap['tokens']}-token case ({cap['captured']}), "
                f"x{scale:g} by expert count (same rows per expert; weights and rows both grow in proportion)")
    return None, None


def _nvlink_report(leg: Leg, disp: dict, stage_ms) -> dict:
    """Bytes that crossed NVLink into this rank per forward and the rate over the stage that
    moved them (rank 0's numbers; the 770 GB/s per direction peer copy is the yardstick)."""
    import torch

    env = leg.env
    if env.world == 1:
        return None
    names = dict(zip(leg.stage_names, stage_ms))
    fp8 = leg.precision == "fp8"
    eb = 1 if fp8 else 2
    row_bytes = HIDDEN * eb + (HIDDEN // 128 * 4 if fp8 else 0)
    fused = not fp8 or disp["pad_rows"] == 128   # kernels with dispatch / push warps
    if leg.tp:
        d_bytes = (env.world - 1) * leg.tokens * row_bytes
        d_ms, d_note = names["dispatch"], "token blocks of all peers pulled once, before the GEMM"
        c_bytes = leg.tokens * (env.world - 1) * HIDDEN * 2
        c_ms, c_note = names["combine"], ("one row per own token from every peer (its sum over the token's k "
                                          "assignments), pushed by the peer; the stage = that kernel, the "
                                          "barrier and the sum of the W planes")
    else:
        owner = (leg.ids // leg.e_local).long()
        remote_assign = int((owner != env.rank).sum().item())
        d_bytes = disp["remote_bytes"]
        if fused:
            d_ms, d_note = names["gate_up_gemm"], ("rows pulled by the dispatch warps inside the gate/up GEMM kernel: "
                                                   "rate over the whole kernel, a lower bound")
            c_bytes = remote_assign * HIDDEN * 2
            c_ms, c_note = names["down_gemm"], ("one weighted row per assignment of an own token whose expert is "
                                                "remote, pushed by the down GEMM kernel of the expert rank while it "
                                                "computes: rate over the whole kernel, a lower bound")
        else:
            d_ms, d_note = names["dispatch"], "e4m3 rows + scales pulled by the dispatch stage"
            mask = torch.zeros(leg.tokens, env.world, dtype=torch.bool, device=env.dev)
            mask.scatter_(1, owner, True)
            mask[:, env.rank] = False
            c_bytes = int(mask.sum().item()) * HIDDEN * 2
            c_ms, c_note = names["combine"], ("one pre-reduced row per (own token, remote expert rank), pulled and "
                                              "summed; the stage includes its barriers")
    return {
        "peak_gbs_per_direction": 770.0,
        "dispatch": {"bytes_in": d_bytes, "ms": d_ms, "gbs": d_bytes / (d_ms * 1e-3) / 1e9, "note": d_note},
        "combine": {"bytes_in": c_bytes, "ms": c_ms, "gbs": c_bytes / (c_ms * 1e-3) / 1e9, "note": c_note},
    }


def _secondary_entry(leg: Leg, steps: int, warmup: int, peaks: dict, baseline: bool) -> dict:
    """Time, verify and describe one secondary workload."""
    env = leg.env
    ms, stage_ms, _ = _time_leg(leg, steps, warmup)
    ver = _verify_leg(leg)
    out = ver.pop("_out")
    disp = _dispatch_exact(leg)
    same = _repeat_identical(leg, out)
    entry = {
        "workload": leg.workload(), "precision": leg.precision, "tokens_per_gpu": leg.tokens,
        "mode": "single" if env.world == 1 else leg.mode, "routing": leg.distribution,
        "ms": ms, "latency_us": ms * 1e3, "tflops": leg.flops_step * env.world / (ms * 1e-3) / 1e12,
        "steps": steps, "warmup": warmup, "stage_ms": dict(zip(leg.stage_names, stage_ms)),
        **{k: v for k, v in _layer_roofline(leg, ms, peaks).items() if k != "rank0"},
        **ver, "dispatch_bytes_exact": disp["exact"], "repeat30_identical": same,
        "nvlink": _nvlink_report(leg, disp, stage_ms),
    }
    if baseline:
        entry["gpu_baseline"] = _time_vllm_baseline(leg.prob, env.world, env.dev, leg.flops_step, env.barrier,
                                                    env.max_over_ranks, out)
    return entry


def _secondary_legs(env: Env, args, peaks: dict, headline: Leg, headline_entry: dict) -> list:
    """The other configurations of the benchmark next to the headline one, each timed, verified
    (256 tokens per rank against the oracle, byte-exact dispatch, 30 repeats bit for bit) and set
    against its roofline and the reference's vLLM path.  Bounded by ``--secondary-budget`` seconds
    of wall clock: legs that would start after it are listed as skipped."""
    from moe_bench_b200 import problem as P

    out, steps, warmup = [], 10, 3
    plan = []
    if env.world == 1:
        for prec in ("bf16", "fp8"):
            for t in (1, 8, 128, 2048, 8192):
                plan.append((prec, t, "ep", "uniform"))
    else:
        plan += [("fp8", t, "ep", "uniform") for t in (128, 1024, 4096)]     # EP fp8 sweep
        plan.append(("fp8", 4096, "ep", "single"))                           # every token on rank 0's experts 0-7
        plan.append(("bf16", 4096, "tp", "uniform"))                         # tensor parallel
    weights_cache = {(headline.precision, headline.mode): headline.weights}
    for prec, t, mode, dist_name in plan:
        name_key = (prec, t, mode, dist_name)
        if name_key == (headline.precision, headline.tokens, headline.mode, headline.distribution):
            out.append(headline_entry)
            continue
        if env.elapsed() > args.secondary_budget:
            out.append({"workload": f"{prec} T{t} {mode} {dist_name}", "skipped": "time budget of the default run"})
            continue
        wkey = (prec, mode)
        if wkey not in weights_cache:
            weights_cache.clear()  # one set of weights at a time beside the headline's
            weights_cache[(headline.precision, headline.mode)] = headline.weights
            kw = dict(device=str(env.dev), num_tokens=[t], num_experts=EXPERTS, precision=P.Precision(prec))
            if env.world == 1:
                weights_cache[wkey] = P.make_weights(P.deepseek_v32_config(**kw))
            else:
                weights_cache[wkey] = P.make_weights(P.deepseek_v32_config(
                    parallel_mode=P.ParallelMode(mode), world_size=env.world, distributed=True, **kw), env.rank)
        leg = Leg(env, prec, t, mode, dist_name, weights=weights_cache[wkey])
        try:
            baseline = not args.no_gpu_baseline and (env.world > 1 or t >= 2048)
            out.append(_secondary_entry(leg, steps, warmup, peaks, baseline))
        finally:
            leg.close()
    return out


def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    from moe_bench_b200 import capi
    from moe_bench_b200 import gating as G
    from moe_bench_b200 import problem as P
    from moe_bench_b200.plugin import get_implementation

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local_rank)
    env = Env(rank, local_rank, world)
    dev = env.dev
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # fp8 activation scales: the format the reference uses on this box (vLLM decides), in the
    # library and in the oracle that checks it
    from oracle import moe_oracle as O

    O.FP8_SCALE_FORMAT = capi.use_reference_fp8_scale_format()
    tokens, steps, warmup = args.tokens, args.steps, args.warmup
    fp8 = args.precision == "fp8"
    leg = Leg(env, args.precision, tokens, args.mode, args.distribution, routing=args.routing)
    run, x, ids, wts, prob, impl = leg.run, leg.x, leg.ids, leg.wts, leg.prob, leg.impl
    stage_names = leg.stage_names
    assignments = tokens * TOPK
    flops_step = leg.flops_step
    barrier, max_over_ranks = env.barrier, env.max_over_ranks

    # -------- device-resident timing, with per-stage events --------
    ms_step, stage_ms, clock_summary = _time_leg(leg, steps, warmup, sample_clocks=True)
    kernel_clocks = capi.read_kernel_clocks(impl._workspace)  # SM clock inside the GEMM kernels of the last step
    stage_by_rank = None
    if world > 1:  # barriers sit inside the first and the last stage: show every rank's split
        stage_by_rank = [None] * world
        dist.all_gather_object(stage_by_rank, [round(v, 4) for v in stage_ms] + [kernel_clocks["gate_up_gemm"]])

    if args.skip_extras:
        if rank == 0:
            _emit({"ms_per_step": ms_step, "stage_ms": dict(zip(stage_names, stage_ms)),
                   "config": _config_dict(tokens, world, args.precision, args.mode, args.distribution),
                   "note": "profiling run, extras skipped"})
        if world > 1:
            impl.close()
            dist.destroy_process_group()
        return

    # -------- end to end: host buffers in, host buffer out --------
    out_dtype = run().dtype
    hx, hi, hw = x.cpu().pin_memory(), ids.cpu().pin_memory(), wts.cpu().pin_memory()
    hout = [torch.empty(tokens, HIDDEN, dtype=out_dtype).pin_memory() for _ in range(2)]
    h2d = hx.numel() * hx.element_size() + hi.numel() * 4 + hw.numel() * 4
    d2h = hout[0].numel() * hout[0].element_size()

    def e2e_serial_step():
        # the step's inputs arrive from pinned host memory into the tensors the plugin reads
        x.copy_(hx, non_blocking=True)
        ids.copy_(hi, non_blocking=True)
        wts.copy_(hw, non_blocking=True)
        hout[0].copy_(run(), non_blocking=True)

    def copy_only_step():
        # the same copies with no kernels between them: what the host link alone costs
        x.copy_(hx, non_blocking=True)
        ids.copy_(hi, non_blocking=True)
        wts.copy_(hw, non_blocking=True)
        hout[0].copy_(leg.impl._out, non_blocking=True)

    def timed(step_fn, finish):
        for _ in range(max(3, warmup // 2)):
            step_fn()
        finish()
        barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for _ in range(steps):
            step_fn()
        finish()
        e2.record()
        torch.cuda.synchronize()
        barrier()
        return max_over_ranks(s2.elapsed_time(e2) / steps)

    ms_e2e_serial = timed(e2e_serial_step, lambda: None)
    ms_copy_only = timed(copy_only_step, lambda: None)

    # The same work as a pipeline, the way a server feeds the layer: every step still copies its
    # inputs host->device and its result device->host inside the timed region, but on copy
    # streams, through `depth` sets of device staging buffers, so that the copies of
    # neighbouring steps overlap the kernels.  The kernels read and write the same tensors as
    # before; a device-to-device copy on the compute stream moves the staged data in and out.
    main = torch.cuda.current_stream(dev)
    depth = 3
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    st_x = [torch.empty_like(x) for _ in range(depth)]
    st_i = [torch.empty_like(ids) for _ in range(depth)]
    st_w = [torch.empty_like(wts) for _ in range(depth)]
    st_o = [torch.empty(tokens, HIDDEN, dtype=out_dtype, device=dev) for _ in range(depth)]
    hout = [torch.empty(tokens, HIDDEN, dtype=out_dtype).pin_memory() for _ in range(depth)]
    in_ready = [torch.cuda.Event() for _ in range(depth)]
    in_free = [torch.cuda.Event() for _ in range(depth)]
    out_ready = [torch.cuda.Event() for _ in range(depth)]
    out_free = [torch.cuda.Event() for _ in range(depth)]
    for ev in in_free + out_free:
        ev.record(main)
    counter = [0]

    def e2e_pipelined_step():
        b = counter[0] % depth
        counter[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[b])          # the kernels of `depth` steps ago have consumed this buffer
            st_x[b].copy_(hx, non_blocking=True)
            st_i[b].copy_(hi, non_blocking=True)
            st_w[b].copy_(hw, non_blocking=True)
            in_ready[b].record(s_in)
        main.wait_event(in_ready[b])
        x.copy_(st_x[b], non_blocking=True)
        ids.copy_(st_i[b], non_blocking=True)
        wts.copy_(st_w[b], non_blocking=True)
        in_free[b].record(main)
        res = run()
        main.wait_event(out_free[b])             # the device->host copy of `depth` steps ago is done
        st_o[b].copy_(res, non_blocking=True)
        out_ready[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(out_ready[b])
            hout[b].copy_(st_o[b], non_blocking=True)
            out_free[b].record(s_out)

    def drain():
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    ms_e2e = timed(e2e_pipelined_step, drain)
    del st_x, st_i, st_w, st_o

    # -------- gating front end as its own stage (not part of the step) --------
    r_logits = G.router_logits(leg.cfg, tokens, rank)
    for _ in range(3):
        capi.route_topk(r_logits, TOPK)
    rs, re_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rs.record()
    for _ in range(20):
        capi.route_topk(r_logits, TOPK)
    re_.record()
    torch.cuda.synchronize()
    route_ms = rs.elapsed_time(re_) / 20
    route_bytes = r_logits.numel() * 4 + tokens * TOPK * 8
    front_end = {"kernel": "route_topk_kernel", "ms": route_ms, "bytes": route_bytes,
                 "achieved_gbs": route_bytes / (route_ms * 1e-3) / 1e9,
                 "note": "softmax -> top-k -> renormalise over [tokens, experts] fp32 logits; inputs fit L2",
                 "used_for_step_routing": args.routing == "logits"}
    del r_logits

    # -------- parity (outside any timed region) --------
    ver = _verify_leg(leg)
    out = ver.pop("_out")
    disp = _dispatch_exact(leg)
    same30 = _repeat_identical(leg, out)

    # -------- reported GPU baseline: the reference's own vLLM path on the same box --------
    gpu_base = {"unavailable": "skipped (--no-gpu-baseline)"}
    if not args.no_gpu_baseline:
        gpu_base = _time_vllm_baseline(prob, world, dev, flops_step, barrier, max_over_ranks, out)
    # -------- decomposition: computation alone, communication alone, fused --------
    decomposition = None
    if args.decompose and world > 1:
        decomposition = _decompose(leg, ms_step, stage_ms, steps, warmup)

    peaks = _peaks()
    layer = _layer_roofline(leg, ms_step, peaks)
    nvlink = _nvlink_report(leg, disp, stage_ms)
    line = None
    if True:  # every rank builds the line (collectives inside), rank 0 prints it
        tc_peak, tc_src = _tensor_peak(args.precision, peaks, dev)
        touched, rows = layer["rank0"]["experts_touched"], layer["rank0"]["assignments"]
        n_local = leg.n_local
        wb = 1 if fp8 else 2  # bytes per weight / activation element on the GEMM's operands
        own_rows = tokens * (world if leg.tp else 1)   # token rows whose bytes the rank reads once
        # algorithmic bytes of the gate/up launch: its weights, every token row once, the activations it writes
        gemm_bytes = touched * 2 * n_local * HIDDEN * wb + own_rows * HIDDEN * wb + rows * n_local * wb
        gemm_flops = 4.0 * n_local * HIDDEN * rows
        gemm_ms = stage_ms[2]
        t_hbm = gemm_bytes / (peaks["hbm_gbs"] * 1e9)
        t_tc = gemm_flops / (tc_peak * 1e12)
        if t_hbm >= t_tc:
            roof = {"bound": "hbm", "achieved": gemm_bytes / (gemm_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s"}
        else:
            roof = {"bound": "tensor", "achieved": gemm_flops / (gemm_ms * 1e-3) / 1e12,
                    "peak": tc_peak, "unit": "TFLOP/s"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        kernel_name = f"grouped_gemm_{'fp8' if fp8 else 'bf16'}_kernel<gate_up_swiglu>"
        traffic, traffic_src = _ncu_traffic("gate_up_gemm", "fp8" if fp8 else "bf16", tokens, args.distribution, world)
        roof.update({
            "traffic": traffic, "traffic_source": traffic_src, "kernel": kernel_name, "kernel_ms": gemm_ms,
            "peak_source": peaks["source"] + " (burst)" if roof["bound"] == "hbm" else tc_src,
            "algorithmic_bytes": gemm_bytes, "algorithmic_flops": gemm_flops, "t_hbm_ms": t_hbm * 1e3,
            "t_tensor_ms": t_tc * 1e3,
        })
        # the other stages against the same peaks (single GPU; the multi-GPU stages contain barriers)
        stage_roofline = None
        if world == 1:
            def _entry(ms, nbytes, flops):
                t_b, t_f = nbytes / (peaks["hbm_gbs"] * 1e9), flops / (tc_peak * 1e12)
                return {"ms": ms, "algorithmic_bytes": nbytes, "algorithmic_flops": flops,
                        "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "achieved_tflops": flops / (ms * 1e-3) / 1e12,
                        "bound": "hbm" if t_b >= t_f else "tensor", "frac": max(t_b, t_f) / (ms * 1e-3)}
            # down GEMM: its weights, the activations it reads, one 16-bit output row per token
            down_bytes = touched * n_local * HIDDEN * wb + rows * n_local * wb + tokens * HIDDEN * 2
            stage_roofline = {
                "align": _entry(stage_ms[0], assignments * 12, 0.0),
                "gather_rows": _entry(stage_ms[1], tokens * HIDDEN * 2 + rows * HIDDEN * wb, 0.0),
                "gate_up_gemm": _entry(stage_ms[2], gemm_bytes, gemm_flops),
                "down_gemm": _entry(stage_ms[3], down_bytes, 2.0 * n_local * HIDDEN * rows),
                "combine": _entry(stage_ms[4], (assignments + tokens) * HIDDEN * 2, 0.0),
            }
            if not fp8:
                stage_roofline.pop("gather_rows")  # the 16-bit gather runs inside the gate/up kernel
        # kernels of this library launched per step (memsets and copies are not kernels); derived
        # from the call sequence of the entry points, checked against the committed ncu launch list
        total_assignments = assignments * world
        n_align = 3 if total_assignments > 8192 else 1
        if world == 1:      # align, [fp8: quantise + row gather], gate/up GEMM (16-bit: gather fused), down GEMM, combine
            kernels_per_step = n_align + 3 + (2 if fp8 else 0)
        else:
            kernels_per_step = _dist_kernels_per_step(n_align, fp8, leg.tp, not fp8 or disp["pad_rows"] == 128)
        line = {
            "metric": METRIC, "value": flops_step * world / (ms_step * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.precision,
            "data": "synthetic", "config": _config_dict(tokens, world, args.precision, args.mode, args.distribution),
            "e2e": {"value": flops_step * world / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                    "mode": f"{depth} steps in flight: copy streams and {depth} device staging buffers overlap each "
                            "step's host<->device copies with the neighbouring steps' kernels",
                    "serial_ms_per_step": ms_e2e_serial,
                    "serial_value": flops_step * world / (ms_e2e_serial * 1e-3) / 1e12,
                    "copy_only_ms": ms_copy_only,
                    "copy_only_note": "the step's pinned host<->device copies alone, no kernels, all ranks at once",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": kernels_per_step * steps,
            "gpu_launches_note": "derived: kernels per forward of the call sequence x steps",
            "front_end": front_end, "decomposition": decomposition,
            "clocks": dict(clock_summary, in_kernel_sm_mhz=kernel_clocks),
            "roofline": roof,
            "stage_ms": dict(zip(stage_names, stage_ms)),
            "stage_ms_by_rank": stage_by_rank, "stage_roofline": stage_roofline,
            "layer_roofline_ms": layer["layer_roofline_ms"], "layer_roofline_frac": layer["layer_roofline_frac"],
            "latency_us": ms_step * 1e3,
            **ver, "dispatch_bytes_exact": disp["exact"], "repeat30_identical": same30, "nvlink": nvlink,
            "fp8_activation_scales": O.FP8_SCALE_FORMAT,
            "fp8_activation_scales_note": "fp8 legs: the format vLLM's quantiser (which the reference calls) uses "
                                          "on this box: ue8m0 = amax/448 rounded up to a power of two",
        }
        line["gpu_baseline"] = gpu_base
    default_workload = (tokens == 8192 and args.precision == "bf16" and args.mode == "ep"
                        and args.distribution == "uniform" and args.routing == "data" and EXPERTS == 256)
    if default_workload and not args.no_secondary:
        headline_entry = {
            "workload": leg.workload(), "precision": leg.precision, "tokens_per_gpu": tokens,
            "mode": "single" if world == 1 else leg.mode, "routing": leg.distribution, "ms": ms_step,
            "latency_us": ms_step * 1e3, "tflops": line["value"], "steps": steps, "warmup": warmup,
            "stage_ms": line["stage_ms"], "layer_roofline_ms": line["layer_roofline_ms"],
            "layer_roofline_frac": line["layer_roofline_frac"], **ver,
            "dispatch_bytes_exact": disp["exact"], "repeat30_identical": same30, "nvlink": nvlink,
            "gpu_baseline": gpu_base, "note": "the headline workload of this line",
        }
        line["secondary"] = _secondary_legs(env, args, peaks, leg, headline_entry)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and not fp8:  # the CPU leg times the bf16 oracle
            res = _time_cpu_oracle(tokens, 20, 2)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        _emit(line)
    leg.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _dist_kernels_per_step(n_align: int, fp8: bool, tp: bool, fused: bool) -> int:
    """Kernels of one distributed forward.  Expert parallel with the fused kernels: 2 barriers,
    routing gather, align, [fp8: quantise], gate/up GEMM (with the dispatch), down GEMM (with the
    combine push), final sum.  Otherwise: 3 barriers, routing gather, align, [fp8: quantise, row
    gather], [TP: block gathers], two GEMMs, local pre-reduce, partial reduce."""
    if not tp and fused:
        return n_align + 2 + 1 + 2 + 1 + (1 if fp8 else 0)
    if tp:  # 2 barriers, routing gather, align, [quantise], block gather(s), [row gather], 2 GEMMs, sum+push, plane sum
        return n_align + 2 + 1 + (1 if fp8 else 0) + (2 if fp8 else 1) + (0 if fused else 1) + 2 + 2
    return n_align + 3 + 5 + 2   # fp8 with few rows per expert: separate gather, pre-reduce and pull


def _decompose(leg: Leg, ms_fused: float, stage_ms, steps: int, warmup: int) -> dict:
    """T_fused next to T_comp alone (this rank's GEMM work with every token already local) and
    T_comm alone (the exchange steps with no GEMM between them), the three legs of the
    reference's tools/analyze_overlap.py:88-100 and tools/time_dispatch.py."""
    import torch
    import torch.distributed as dist

    from moe_bench_b200 import problem as P
    from moe_bench_b200.plugin import get_implementation

    env = leg.env
    world, tokens, dev = env.world, leg.tokens, env.dev
    full_x = torch.empty(world * tokens, HIDDEN, dtype=leg.x.dtype, device=dev)
    full_ids = torch.empty(world * tokens, TOPK, dtype=leg.ids.dtype, device=dev)
    full_w = torch.empty(world * tokens, TOPK, dtype=leg.wts.dtype, device=dev)
    dist.all_gather_into_tensor(full_x, leg.x.contiguous())
    dist.all_gather_into_tensor(full_ids, leg.ids.contiguous())
    dist.all_gather_into_tensor(full_w, leg.wts.contiguous())
    comp_prob = P.MoEProblem(leg.cfg, world * tokens, full_x, leg.prob.w1, leg.prob.w2, full_ids, full_w,
                             None if leg.tp else leg.prob.expert_map, leg.prob.quant_config)
    comp = get_implementation("b200")
    comp.setup(comp_prob)
    for _ in range(max(3, warmup)):
        comp.run(comp_prob)
    env.barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(steps):
        comp.run(comp_prob)
    c1.record()
    torch.cuda.synchronize()
    env.barrier()
    ms_comp = env.max_over_ranks(c0.elapsed_time(c1) / steps)
    del comp, comp_prob, full_x, full_ids, full_w
    # communication alone: the same forward with the GEMM stages switched off
    ms_comm = None
    if hasattr(leg.impl, "run_comm_only"):
        for _ in range(max(3, warmup)):
            leg.impl.run_comm_only()
        env.barrier()
        c0.record()
        for _ in range(steps):
            leg.impl.run_comm_only()
        c1.record()
        torch.cuda.synchronize()
        env.barrier()
        ms_comm = env.max_over_ranks(c0.elapsed_time(c1) / steps)
    return {
        "t_fused_ms": ms_fused, "t_comp_alone_ms": ms_comp, "t_comm_alone_ms": ms_comm,
        "t_comm_exposed_ms": ms_fused - ms_comp,
        "exposed_fraction_of_fused": (ms_fused - ms_comp) / ms_fused,
        "overlap_efficiency": None if ms_comm is None else 1.0 - (ms_fused - ms_comp) / max(ms_comm, 1e-9),
        "comm_stage_ms_in_fused": stage_ms[0] + stage_ms[1] + stage_ms[4],
        "note": "comp alone = the single-GPU forward of this rank's experts (EP) or weight shard (TP) over all "
                "W*T tokens gathered beforehand; comm alone = staging, barriers, routing exchange, dispatch of "
                "rows and combine of partial rows with the GEMM kernels skipped; exposed = fused - comp alone",
    }


_RESULT_STREAM = None


def _claim_stdout() -> None:
    """Keep the real stdout for the one JSON line and send everything else that
    writes to file descriptor 1 (vLLM and Triton log there) to stderr."""
    global _RESULT_STREAM
    if _RESULT_STREAM is None:
        sys.stdout.flush()
        _RESULT_STREAM = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        sys.stdout = sys.stderr


def _emit(line: dict) -> None:
    stream = _RESULT_STREAM or sys.stdout
    stream.write(json.dumps(line) + "\n")
    stream.flush()


def main() -> None:
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per GPU")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp8", "fp16"],
                    help="bf16 = the headline workload; fp8 = the block-quantised config of the same shape; "
                         "fp16 = the bf16 kernels with IEEE-half tensors")
    ap.add_argument("--mode", default="ep", choices=["ep", "tp"], help="parallel mode when --gpus > 1")
    ap.add_argument("--distribution", default="uniform", choices=["uniform", "single", "skewed", "balanced"])
    ap.add_argument("--routing", default="data", choices=["data", "logits"],
                    help="data = topk_ids/topk_weights drawn as the reference's generator does (the headline); "
                         "logits = router logits through the library's top-k kernel")
    ap.add_argument("--decompose", action="store_true",
                    help="N > 1: also time the rank's computation alone (all tokens local) next to the fused step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gpu-baseline", action="store_true", help="skip the vLLM fused_experts baseline leg")
    ap.add_argument("--experts", type=int, default=256, help="expert count (lower it only to size a profiler capture)")
    ap.add_argument("--skip-extras", action="store_true", help="timed region only: no e2e, parity or CPU legs")
    ap.add_argument("--no-secondary", action="store_true",
                    help="default workload only: skip the secondary list (token sweep, fp8, EP-fp8 / single / TP legs)")
    ap.add_argument("--secondary-budget", type=float, default=420.0,
                    help="seconds of wall clock after which no further secondary leg is started")
    args = ap.parse_args()
    global EXPERTS
    EXPERTS = args.experts
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
