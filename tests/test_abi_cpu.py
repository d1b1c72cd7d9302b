"""The C-ABI library loads without a GPU and exports every declared symbol."""

import ctypes
import os
import re

import pytest

from moe_bench_b200 import build as mb_build
from moe_bench_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moe_bench_b200.h")


@pytest.fixture(scope="module")
def lib():
    mb_build.build()
    return capi.load()


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes prototype"
    assert sorted(capi.SIGNATURES) == names


def test_abi_version_and_pure_host_queries(lib):
    assert lib.mb200_abi_version() == capi.ABI_VERSION == 5
    # 8 assignments can hit at most 8 experts: 8 + 8*127 rows, rounded to 128
    assert lib.mb200_row_capacity(1, 8, 256, 128) == 1024
    assert lib.mb200_row_capacity(1, 8, 256, 16) == 128
    assert lib.mb200_row_capacity(8192, 8, 256, 128) == (65536 + 256 * 127 + 127) // 128 * 128
    assert lib.mb200_row_capacity(8192, 8, 256, 16) == (65536 + 256 * 15 + 15) // 16 * 16
    assert lib.mb200_row_capacity(0, 8, 256, 16) == 0
    n = lib.mb200_workspace_bytes(capi.PRECISION_BF16, 128, 7168, 2048, 256, 8)
    assert n > 128 * 8 * 7168 * 2
    assert n % 1024 == 0
    assert lib.mb200_workspace_bytes(capi.PRECISION_FP16, 128, 7168, 2048, 256, 8) == n


def test_argument_errors_are_reported_not_fatal(lib):
    assert lib.mb200_workspace_bytes(capi.PRECISION_BF16, 4, 100, 128, 8, 2) == -1
    assert b"hidden" in lib.mb200_last_error()
    rc = lib.mb200_route_topk(None, 4, 8, 9, None, None, None)
    assert rc != 0
    rc = lib.mb200_align(None, 4, 2, None, 4096, None, None, None, None, 0, 16, None, None)
    assert rc != 0


def test_plugin_refuses_cpu_tensors():
    import torch

    from moe_bench_b200 import problem as P
    from moe_bench_b200.plugin import B200FusedExperts, get_implementation

    cfg = P.MoEBenchConfig(hidden_size=256, intermediate_size=128, num_experts=8, topk=2, world_size=1, device="cpu")
    prob = P.make_problem(cfg, 4)
    impl = get_implementation("b200")
    assert isinstance(impl, B200FusedExperts)
    with pytest.raises(capi.MB200Error):
        impl.setup(prob)
    with pytest.raises(ValueError):
        get_implementation("nope")
