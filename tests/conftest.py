"""Shared pytest configuration: the ``gpu`` marker and import paths."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "golden.pt")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(GOLDEN, weights_only=False)


@pytest.fixture(scope="session", autouse=True)
def _fp8_scale_format_of_this_box():
    """On a GPU box the library quantises activations the way the reference does THERE (vLLM
    uses power-of-two scales where its DeepGEMM path is enabled); the oracle and the library's
    direct calls from the test thread follow.  Without a GPU: the plain fp32 format."""
    import torch

    if not torch.cuda.is_available():
        yield "fp32"
        return
    from moe_bench_b200 import capi
    from oracle import moe_oracle as O

    O.FP8_SCALE_FORMAT = capi.use_reference_fp8_scale_format()
    yield O.FP8_SCALE_FORMAT
    O.FP8_SCALE_FORMAT = "fp32"
