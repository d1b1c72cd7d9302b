"""Registration with an installed moe_bench: one call instead of editing its sources.

    import moe_bench_b200.register as R
    R.register("moe_bench")            # the importable name of the reference package

adds ``B200FusedExperts`` to the package's ``IMPLEMENTATIONS`` registry
(reference ``baseline.py:80-91``, selected with ``--impl b200``) and
``B200Scheme`` to its ``SCHEMES`` registry (``schemes.py:147-170``, ``--scheme
b200``).  ``mp.spawn`` workers re-import modules, so a distributed run must make
the same call in every worker before ``get_scheme`` (reference
``distributed.py:99``).  The classes only read attributes of the ``MoEProblem`` /
``DistContext`` objects they are handed, so the reference's own objects work.
"""

from __future__ import annotations

import importlib

from .plugin import B200FusedExperts
from .scheme import B200Scheme


def register(package: str = "moe_bench") -> dict:
    """Returns the two registries after the insertion."""
    baseline = importlib.import_module(f"{package}.baseline")
    schemes = importlib.import_module(f"{package}.schemes")
    baseline.IMPLEMENTATIONS[B200FusedExperts.name] = B200FusedExperts
    schemes.SCHEMES[B200Scheme.name] = B200Scheme
    return {"IMPLEMENTATIONS": baseline.IMPLEMENTATIONS, "SCHEMES": schemes.SCHEMES}
