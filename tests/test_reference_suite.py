"""The reference's own unit / fuzz / stress tests, run against this package as ``brute``.

Needs a checkout of the reference: set ``BRUTE_REFERENCE_CHECKOUT`` to its root (the directory that
holds ``tests/unit``). Skipped when the variable is not set. The suite runs in a child pytest
process from that checkout, with tests/reference_alias_plugin.py loaded first; nothing is written
into the checkout.
"""
import os
import re
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent


@pytest.mark.timeout(1800)
def test_reference_suite_passes_against_this_package(lib_built):
    root = os.environ.get("BRUTE_REFERENCE_CHECKOUT")
    if not root:
        pytest.skip("BRUTE_REFERENCE_CHECKOUT is not set")
    root = Path(root)
    assert (root / "tests" / "unit").is_dir(), f"{root} does not look like a checkout of the reference"
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(HERE), env.get("PYTHONPATH", "")])
    env["HYPOTHESIS_STORAGE_DIRECTORY"] = tempfile.mkdtemp(prefix="hyp")
    res = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "reference_alias_plugin", "-p", "no:cacheprovider",
         "tests/unit", "tests/fuzz", "tests/stress", "-q", "--no-header", "--tb=line", "-rf"],
        cwd=root, env=env, capture_output=True, text=True)
    tail = "\n".join(res.stdout.splitlines()[-40:])
    summary = res.stdout.strip().splitlines()[-1] if res.stdout.strip() else ""
    assert res.returncode == 0 and " failed" not in summary, f"reference suite did not pass:\n{tail}\n{res.stderr[-2000:]}"
    passed = re.search(r"(\d+) passed", summary)
    assert passed and int(passed.group(1)) >= 1000, summary
