"""Diagnostics for the grouped GEMM kernels (need a B200; nothing here is on the
product path and nothing imports this module).

    python -m moe_bench_b200.diagnostics waits [--tokens 8192 4096 --distribution uniform balanced]
    python -m moe_bench_b200.diagnostics ab --a PATH_A.so --b PATH_B.so [--tokens ...]
    python -m moe_bench_b200.diagnostics mma-rate

``waits``     runs the layer with the probe build of the library (compiled with
              ``-DMB200_PROBE_WAITS``): the MMA-issuing warp of CTA 0 counts the SM
              cycles it spends waiting for a stage to arrive, waiting for a free
              accumulator, and in total, for both GEMM kernels, next to the clock the
              kernels really ran at (cycles / nanoseconds).
``ab``        loads two builds of the library side by side and alternates bursts of
              forwards between them in ONE process, so that the clock drift of a
              power-capped GPU cancels; prints time, in-kernel clock and cycle counts
              and whether the outputs are bit-identical.  The environment is read by
              each copy at its first GEMM launch (``--env-a`` / ``--env-b`` set
              ``MB200_PAIR_MIN_ROWS`` for that moment).
``mma-rate``  runs the stand-alone ``tcgen05.mma`` issue-rate microbenchmark.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

import torch

from . import build as B
from . import capi
from . import problem as P
from .plugin import get_implementation

# int64 words of the workspace head (starting at byte 32) the probe build fills
_G1_CYC, _G1_NS, _G2_CYC, _G2_NS = 0, 1, 2, 3
_G1_WAIT_FULL, _G1_WAIT_ACC, _G1_TOTAL = 4, 5, 6
_G2_WAIT_FULL, _G2_WAIT_ACC, _G2_TOTAL = 9, 10, 11


def _probe_words(impl) -> list:
    return impl._workspace[32:160].view(torch.int64).cpu().tolist()


def _problem(weights, tokens: int, distribution: str):
    cfg = P.deepseek_v32_config(device="cuda:0", routing=P.RoutingConfig(distribution=P.Distribution(distribution)))
    return P.make_problem(cfg, tokens, weights=weights)


def waits(tokens_list, distributions) -> None:
    probe, _ = B.build_diagnostics()
    capi.use_library(capi.load_library(probe))
    weights = P.make_weights(P.deepseek_v32_config(device="cuda:0"))
    for dist in distributions:
        for tokens in tokens_list:
            prob = _problem(weights, tokens, dist)
            impl = get_implementation("b200")
            impl.setup(prob)
            for _ in range(12):
                impl.run(prob)
            torch.cuda.synchronize()
            d = _probe_words(impl)
            for name, cyc, ns, wf, wa, tot in (
                ("gate/up", _G1_CYC, _G1_NS, _G1_WAIT_FULL, _G1_WAIT_ACC, _G1_TOTAL),
                ("down", _G2_CYC, _G2_NS, _G2_WAIT_FULL, _G2_WAIT_ACC, _G2_TOTAL),
            ):
                total = max(d[tot], 1)
                print(f"{dist:9s} T={tokens:<5d} {name:8s} {d[ns] / 1e6:7.3f} ms @ {d[cyc] / max(d[ns], 1):.3f} GHz  "
                      f"MMA warp: {total / 1e6:.2f} M cycles, waiting for data {100 * d[wf] / total:4.1f} %, "
                      f"for a free accumulator {100 * d[wa] / total:4.1f} %")
            del impl


def ab(path_a: str, path_b: str, env_a: str, env_b: str, tokens_list, distributions) -> None:
    tmp = tempfile.mkdtemp(prefix="mb200_ab_")
    libs = {}
    small = P.MoEBenchConfig(hidden_size=256, intermediate_size=128, num_experts=8, topk=2, world_size=1,
                             device="cuda:0")
    for name, path, env in (("A", path_a, env_a), ("B", path_b, env_b)):
        copy = os.path.join(tmp, f"lib_{name}.so")   # a second path = a second instance with its own statics
        shutil.copy(path, copy)
        if env is None:
            os.environ.pop("MB200_PAIR_MIN_ROWS", None)
        else:
            os.environ["MB200_PAIR_MIN_ROWS"] = env
        libs[name] = capi.load_library(copy)
        capi.use_library(libs[name])
        prob = P.make_problem(small, 64)             # first GEMM launch of this copy: it reads the environment now
        impl = get_implementation("b200")
        impl.setup(prob)
        impl.run(prob)
        torch.cuda.synchronize()
    weights = P.make_weights(P.deepseek_v32_config(device="cuda:0"))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for dist in distributions:
        for tokens in tokens_list:
            prob = _problem(weights, tokens, dist)
            impls, res, outs = {}, {n: [] for n in libs}, {}
            for name, lib in libs.items():
                capi.use_library(lib)
                impls[name] = get_implementation("b200")
                impls[name].setup(prob)
                impls[name].run(prob)
            torch.cuda.synchronize()
            for _ in range(7):
                for name, lib in libs.items():
                    capi.use_library(lib)
                    for _ in range(3):
                        impls[name].run(prob)
                    ev[0].record()
                    for _ in range(5):
                        outs[name] = impls[name].run(prob)
                    ev[1].record()
                    torch.cuda.synchronize()
                    d = _probe_words(impls[name])
                    res[name].append((ev[0].elapsed_time(ev[1]) / 5, d[_G1_NS] / 1e6, d[_G1_CYC] / max(d[_G1_NS], 1),
                                      d[_G2_NS] / 1e6, d[_G1_TOTAL], d[_G2_TOTAL]))
            same = torch.equal(outs["A"], outs["B"])
            for name in libs:
                r = res[name][1:]
                a = [sum(x[i] for x in r) / len(r) for i in range(6)]
                print(f"{dist:9s} T={tokens:<5d} {name}  layer {a[0]:.3f} ms | gate/up {a[1]:.3f} ms @ {a[2]:.3f} GHz "
                      f"({a[4] / 1e6:.2f} M cyc) | down {a[3]:.3f} ms ({a[5] / 1e6:.2f} M cyc) | bit-identical: {same}")
    shutil.rmtree(tmp, ignore_errors=True)


def mma_rate() -> None:
    _, tool = B.build_diagnostics()
    sys.stdout.write(subprocess.run([tool], capture_output=True, text=True, timeout=120).stdout)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m moe_bench_b200.diagnostics")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("waits", "ab"):
        sp = sub.add_parser(name)
        sp.add_argument("--tokens", type=int, nargs="+", default=[8192])
        sp.add_argument("--distribution", nargs="+", default=["uniform", "balanced"],
                        choices=["uniform", "balanced", "skewed", "single"])
        if name == "ab":
            sp.add_argument("--a", required=True, help="library build A (cycle counts need a probe build)")
            sp.add_argument("--b", required=True)
            sp.add_argument("--env-a", default=None, help="MB200_PAIR_MIN_ROWS while copy A starts")
            sp.add_argument("--env-b", default=None)
    sub.add_parser("mma-rate")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the diagnostics need a CUDA device")
    if args.cmd == "waits":
        waits(args.tokens, args.distribution)
    elif args.cmd == "ab":
        ab(args.a, args.b, args.env_a, args.env_b, args.tokens, args.distribution)
    else:
        mma_rate()


if __name__ == "__main__":
    main()
