"""pytest plugin (``-p reference_alias_plugin``): run a checkout of the reference's OWN test suite
against this package.

It makes ``import brute`` resolve to ``brute_b200`` and binds the CPU dispatch key of
``torch.ops.brute.*`` to the oracle (the product has CUDA kernels only), then the reference's
tests/unit, tests/fuzz and tests/stress run unchanged. Used by tests/test_reference_suite.py.
"""
import importlib
import sys
from pathlib import Path

_TESTS = Path(__file__).resolve().parent
for _p in (str(_TESTS.parent), str(_TESTS)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import __graft_entry__ as _entry  # noqa: E402

_entry.build()
import brute_b200  # noqa: E402

sys.modules["brute"] = brute_b200
for _sub in ("tensor", "dtype", "functional", "fast", "streams", "cuda_graphs"):
    sys.modules["brute." + _sub] = importlib.import_module("brute_b200." + _sub)

import conftest as _repo_conftest  # noqa: E402

_repo_conftest.install_oracle_cpu_ops()
