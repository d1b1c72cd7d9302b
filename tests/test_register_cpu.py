"""Drop-in check against the reference package itself, where it is present next to
this repository (directory ``reference`` beside the repository root); skipped
elsewhere.  No compute: the point is that the reference's own registries, factory
functions and problem objects accept the plugin."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PARENT = os.path.dirname(ROOT)


@pytest.mark.skipif(not os.path.isfile(os.path.join(PARENT, "reference", "baseline.py")),
                    reason="the reference package is not present beside the repository")
def test_plugin_registers_with_the_reference_and_takes_its_problem_objects():
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    sys.path.insert(0, PARENT)
    try:
        import moe_bench_b200.register as R
        from moe_bench_b200 import capi

        regs = R.register("reference")
        assert "b200" in regs["IMPLEMENTATIONS"] and "b200" in regs["SCHEMES"]
        assert "naive" in regs["IMPLEMENTATIONS"]          # the reference's own entry is untouched

        from reference import baseline, schemes
        from reference.config import MoEBenchConfig
        from reference.data import make_problem

        impl = baseline.get_implementation("b200")          # the reference's factory builds the plugin
        assert impl.name == "b200" and callable(impl.setup) and callable(impl.run)
        scheme = schemes.get_scheme("b200")
        assert scheme.name == "b200" and callable(scheme.close)

        # a problem made by the reference itself (CPU tensors): the plugin reads it and refuses
        # loudly, because there is no CPU path
        cfg = MoEBenchConfig(hidden_size=256, intermediate_size=128, num_experts=8, topk=2, world_size=1,
                             device="cpu")
        prob = make_problem(cfg, 16)
        with pytest.raises(capi.MB200Error, match="no CPU path"):
            impl.setup(prob)
    finally:
        sys.path.remove(PARENT)
