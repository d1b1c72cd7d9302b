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
token dispatch and the weighted combine cross NVLink inside the library's
kernels.  Per-GPU work is fixed (weak scaling); the value is the sum over ranks
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


def _time_cpu_oracle(tokens: int, steps: int, warmup: int, budget_s: float = 25.0):
    import torch

    from oracle import moe_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    prob = _cpu_sample_problem(tokens)
    assignments = prob.num_local_assignments
    flops = 6.0 * INTER * HIDDEN * assignments
    for _ in range(warmup):
        O.reference_moe(prob)
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        O.reference_moe(prob)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    avg = sum(times) / len(times)
    return {
        "value": flops / avg / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"experts 0-3 of 256 with all {assignments} assignments of a {tokens}-token batch "
                  f"(DSv3.2 dims, weights pre-converted to fp32), {len(times)} passes, {avg * 1e3:.1f} ms each",
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
                        "dispatch/combine by P2P pulls over NVLink" if mode == "ep" else
                        f"tp{world}: all experts, intermediate/{world} columns and {tokens} own tokens per GPU, "
                        "token gather and output reduce by P2P pulls over NVLink"),
        "l2": f"inputs larger than L2: {wgb} GB of expert weights are streamed every step",
    }


def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    from moe_bench_b200 import capi
    from moe_bench_b200 import gating as G
    from moe_bench_b200 import problem as P
    from moe_bench_b200.plugin import get_implementation
    from oracle import moe_oracle as O

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    tokens, steps, warmup = args.tokens, args.steps, args.warmup
    fp8 = args.precision == "fp8"
    prec = P.Precision(args.precision)
    if world == 1:
        cfg = P.deepseek_v32_config(device=str(dev), num_tokens=[tokens], num_experts=EXPERTS, precision=prec,
                                    routing=P.RoutingConfig(distribution=P.Distribution(args.distribution)))
        weights = P.make_weights(cfg)
        x, ids, wts = P._gen_input(cfg, tokens, 0)
        if args.routing == "logits":
            # gating front end: router logits -> top-k kernel instead of the generator's direct draw
            ids, wts = capi.route_topk(G.router_logits(cfg, tokens, 0), TOPK)
        prob = P.MoEProblem(cfg, tokens, x, weights.w1, weights.w2, ids, wts, None, weights.quant_config)
        impl = get_implementation("b200")
        impl.setup(prob)
        run = lambda: impl.run(prob)  # noqa: E731
        stage_names = capi.STAGE_NAMES
    else:
        # expert parallel over the N GPUs: rank r owns experts [r*E/N, (r+1)*E/N) and its own token shard
        from moe_bench_b200.scheme import DistContext, get_scheme

        cfg = P.deepseek_v32_config(device=str(dev), num_tokens=[tokens], num_experts=EXPERTS, precision=prec,
                                    parallel_mode=P.ParallelMode(args.mode), world_size=world, distributed=True,
                                    routing=P.RoutingConfig(distribution=P.Distribution(args.distribution)))
        weights = P.make_weights(cfg, rank)
        if args.routing == "logits":
            prob, _ = G.make_routed_problem(cfg, tokens, rank, weights=weights)
        else:
            prob = P.make_problem(cfg, tokens, rank, weights=weights)
        x, ids, wts = prob.hidden_states, prob.topk_ids, prob.topk_weights
        impl = get_scheme("b200")
        impl.setup(prob, DistContext(rank=rank, world_size=world, local_rank=local_rank, device=dev))
        run = impl.run
        stage_names = ("stage_routing_align", "dispatch", "gate_up_gemm", "down_gemm", "combine")
    assignments = tokens * TOPK
    # TP: every rank computes all W*T*k assignments on intermediate/W columns = the same flops per rank
    flops_step = 6.0 * INTER * HIDDEN * assignments

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(warmup):
        run()
    # -------- device-resident timing, with per-stage events --------
    stage_ev = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(steps)]
    for evs in stage_ev:
        for ev in evs:
            ev.record()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        start.record()
        for i in range(steps):
            capi.set_stage_events(stage_ev[i])
            run()
        end.record()
        torch.cuda.synchronize()
    capi.set_stage_events(None)
    barrier()
    ms_step = max_over_ranks(start.elapsed_time(end) / steps)
    if impl.device_status() != 0:
        raise RuntimeError(f"device status {impl.device_status()}")
    stage_ms = [sum(evs[j].elapsed_time(evs[j + 1]) for evs in stage_ev) / steps for j in range(5)]
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

    # The same work as a two-deep pipeline, the way a server feeds the layer: every step still
    # copies its inputs host->device and its result device->host inside the timed region, but
    # on copy streams, through two sets of device staging buffers, so that the copies of
    # neighbouring steps overlap the kernels.  The kernels read and write the same tensors as
    # before; a device-to-device copy on the compute stream moves the staged data in and out.
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    st_x = [torch.empty_like(x) for _ in range(2)]
    st_i = [torch.empty_like(ids) for _ in range(2)]
    st_w = [torch.empty_like(wts) for _ in range(2)]
    st_o = [torch.empty(tokens, HIDDEN, dtype=out_dtype, device=dev) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]
    for ev in in_free + out_free:
        ev.record(main)
    counter = [0]

    def e2e_pipelined_step():
        b = counter[0] & 1
        counter[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[b])          # the kernels of two steps ago have consumed this buffer
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
        main.wait_event(out_free[b])             # the device->host copy of two steps ago is done
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

    # -------- gating front end as its own stage (not part of the step) --------
    r_logits = G.router_logits(cfg, tokens, rank)
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

    # -------- parity spot check (outside any timed region) --------
    out = run().clone()
    idx = torch.randperm(tokens, generator=torch.Generator().manual_seed(0))[: min(8, tokens)].to(dev)
    if world == 1:
        ref_w1, ref_w2, ref_qc = weights.w1, weights.w2, weights.quant_config
    else:
        # ground truth of a distributed rank: its tokens through ALL experts (reference distributed.py:64-84);
        # experts are generated on demand, only the ones the sampled tokens touch
        ref_w1, ref_w2, ref_qc = _lazy_logical_weights(cfg, P)
    sub = P.MoEProblem(cfg, len(idx), x[idx].contiguous(), ref_w1, ref_w2, ids[idx].contiguous(),
                       wts[idx].contiguous(), None, ref_qc)
    check = O.verify_output(args.precision, out[idx], O.reference_moe(sub))

    # -------- reported GPU baseline: the reference's own vLLM path on the same box --------
    gpu_base = {"unavailable": "skipped (--no-gpu-baseline)"}
    if not args.no_gpu_baseline:
        gpu_base = _time_vllm_baseline(prob, world, dev, flops_step, barrier, max_over_ranks, out)
    # -------- decomposition: the rank's GEMM work with every token already local --------
    decomposition = None
    if args.decompose and world > 1:
        full_x = torch.empty(world * tokens, HIDDEN, dtype=x.dtype, device=dev)
        full_ids = torch.empty(world * tokens, TOPK, dtype=ids.dtype, device=dev)
        full_w = torch.empty(world * tokens, TOPK, dtype=wts.dtype, device=dev)
        dist.all_gather_into_tensor(full_x, x.contiguous())
        dist.all_gather_into_tensor(full_ids, ids.contiguous())
        dist.all_gather_into_tensor(full_w, wts.contiguous())
        ep = args.mode == "ep"
        comp_prob = P.MoEProblem(cfg, world * tokens, full_x, prob.w1, prob.w2, full_ids, full_w,
                                 prob.expert_map if ep else None, prob.quant_config)
        comp = get_implementation("b200")
        comp.setup(comp_prob)
        for _ in range(max(3, warmup)):
            comp.run(comp_prob)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(steps):
            comp.run(comp_prob)
        c1.record()
        torch.cuda.synchronize()
        barrier()
        ms_comp = max_over_ranks(c0.elapsed_time(c1) / steps)
        decomposition = {
            "t_fused_ms": ms_step, "t_comp_alone_ms": ms_comp, "t_comm_exposed_ms": ms_step - ms_comp,
            "comm_stage_ms_in_fused": stage_ms[0] + stage_ms[1] + stage_ms[4],
            "note": "comp alone = the single-GPU forward of this rank's experts (EP) or weight shard (TP) over "
                    "all W*T tokens gathered beforehand; exposed communication = fused - comp alone; the stage "
                    "sum is routing exchange + dispatch + combine/reduce incl. their barriers in the fused run",
        }
        del comp, comp_prob, full_x, full_ids, full_w

    if world > 1:
        ok = torch.tensor([1.0 if check.passed else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        passed = bool(ok.item() > 0)
    else:
        passed = check.passed

    if rank == 0:
        peaks = _peaks()
        # world == 1: experts this batch touches; EP: every local expert is hit, rows = this rank's share
        tp = world > 1 and args.mode == "tp"
        if world == 1:
            touched, rows, n_local = _touched_experts(ids), assignments, INTER
        elif tp:   # all experts, intermediate/W columns, every rank computes all W*T tokens
            touched, rows, n_local = EXPERTS, assignments * world, INTER // world
        else:      # EP, uniform routing: every local expert is hit, rows = this rank's share on average
            touched, rows, n_local = EXPERTS // world, assignments, INTER
        wb = 1 if fp8 else 2  # bytes per weight / activation element on the GEMM's operands
        gemm_bytes = touched * 2 * n_local * HIDDEN * wb + rows * HIDDEN * wb + rows * n_local * wb
        gemm_flops = 4.0 * INTER * HIDDEN * assignments
        gemm_ms = stage_ms[2]
        t_hbm = gemm_bytes / (peaks["hbm_gbs"] * 1e9)
        # no fp8 peak is measured on this pool: the bf16 burst figure is doubled (nominal ratio)
        tc_peak = peaks["bf16_tflops"] * (2.0 if fp8 else 1.0)
        t_tc = gemm_flops / (tc_peak * 1e12)
        if t_hbm >= t_tc:
            roof = {"bound": "hbm", "achieved": gemm_bytes / (gemm_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s"}
        else:
            roof = {"bound": "tensor", "achieved": gemm_flops / (gemm_ms * 1e-3) / 1e12,
                    "peak": tc_peak, "unit": "TFLOP/s"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        # DRAM bytes of one gate/up launch from the committed ncu capture of the 32-expert /
        # 1024-token case (2.075 GB read + 0.151 GB written), scaled by the expert count; only
        # for workloads with the capture's 32 tokens per expert, where traffic grows in proportion
        traffic = None
        if not fp8 and world == 1 and tokens * 32 == EXPERTS * 1024 and args.distribution == "uniform":
            traffic = 2.226e9 * EXPERTS / 32
        roof.update({
            "traffic": traffic,
            "traffic_source": "profiles/grouped_gemm_bf16_E32_T1024_ncu_full.md x experts/32" if traffic else None, "kernel": f"grouped_gemm_{'fp8' if fp8 else 'bf16'}_kernel<gate_up_swiglu>", "kernel_ms": gemm_ms,
            "peak_source": peaks["source"] + " (burst)", "algorithmic_bytes": gemm_bytes,
            "algorithmic_flops": gemm_flops, "t_hbm_ms": t_hbm * 1e3, "t_tensor_ms": t_tc * 1e3,
        })
        # the other stages against the same peaks (single GPU; the multi-GPU stages contain barriers)
        stage_roofline = None
        if world == 1:
            def _entry(ms, nbytes, flops):
                t_b, t_f = nbytes / (peaks["hbm_gbs"] * 1e9), flops / (tc_peak * 1e12)
                return {"ms": ms, "algorithmic_bytes": nbytes, "algorithmic_flops": flops,
                        "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "achieved_tflops": flops / (ms * 1e-3) / 1e12,
                        "bound": "hbm" if t_b >= t_f else "tensor", "frac": max(t_b, t_f) / (ms * 1e-3)}
            down_bytes = touched * n_local * HIDDEN * wb + rows * n_local * wb + rows * HIDDEN * 2
            stage_roofline = {
                "align": _entry(stage_ms[0], assignments * 12, 0.0),
                "gate_up_gemm": _entry(stage_ms[2], gemm_bytes, gemm_flops),
                "down_gemm": _entry(stage_ms[3], down_bytes, 2.0 * INTER * HIDDEN * assignments),
                "combine": _entry(stage_ms[4], (assignments + tokens) * HIDDEN * 2, 0.0),
            }
        layer_bytes = touched * 3 * n_local * HIDDEN * wb + 2 * tokens * HIDDEN * 2 + assignments * 8
        layer_roof_ms = max(layer_bytes / (peaks["hbm_gbs"] * 1e9), flops_step / (tc_peak * 1e12)) * 1e3
        # kernels of this library launched per step (memsets and copies are not kernels)
        total_assignments = assignments * world
        n_align = 3 if total_assignments > 16384 else 1
        if world == 1:      # align, [fp8: gather+quantise], gate/up GEMM (bf16: with the gather fused), down GEMM, combine
            kernels_per_step = n_align + 3 + (1 if fp8 else 0)
        else:               # + 3 barriers, routing gather, partial reduce; fp8: quantise + dispatch gather; TP: block gather(s)
            kernels_per_step = n_align + 3 + 5 + (2 if fp8 else 0)
            if args.mode == "tp":
                kernels_per_step += 2 if fp8 else 1
        line = {
            "metric": METRIC, "value": flops_step * world / (ms_step * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.precision,
            "data": "synthetic", "config": _config_dict(tokens, world, args.precision, args.mode, args.distribution),
            "e2e": {"value": flops_step * world / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                    "mode": "two steps in flight: copy streams and two device staging buffers overlap each "
                            "step's host<->device copies with the neighbouring steps' kernels",
                    "serial_ms_per_step": ms_e2e_serial,
                    "serial_value": flops_step * world / (ms_e2e_serial * 1e-3) / 1e12,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": kernels_per_step * steps, "front_end": front_end, "decomposition": decomposition,
            "clocks": dict(clocks.summary(), in_kernel_sm_mhz=kernel_clocks),
            "roofline": roof,
            "stage_ms": dict(zip(stage_names, stage_ms)),
            "stage_ms_by_rank": stage_by_rank, "stage_roofline": stage_roofline,
            "layer_roofline_ms": layer_roof_ms, "layer_roofline_frac": layer_roof_ms / ms_step,
            "latency_us": ms_step * 1e3,
            "verify": "ok" if passed else "FAIL", "rel_err": check.rel_err,
        }
        line["gpu_baseline"] = gpu_base
        if world == 1 and not args.no_cpu_baseline and not fp8:  # the CPU leg times the bf16 oracle
            res = _time_cpu_oracle(tokens, 20, 2)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        _emit(line)
    if world > 1:
        impl.close()
        dist.barrier()
        dist.destroy_process_group()


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
