"""(Collected late on purpose: it re-runs whole suites in a child process.) The two bindings of
torch.ops.brute.* to the C ABI: the compiled one (csrc_host/cbrute.cpp, the default) and the ctypes one
(BRUTE_B200_BINDING=ctypes).

The binding is chosen when the package is imported, so each check runs in a child process with the
variable set. Without a GPU: the compiled functions are registered on the CUDA key of every schema.
With one (marked gpu): the suites that the rest of the run executes through the default binding pass
through the other one as well, and the stream tests run through the ctypes binding, whose ops take
part in the rotation of ``parallel_streams``.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(code_or_args, env_extra, timeout=1500):
    env = dict(os.environ)
    env.update(env_extra)
    return subprocess.run(code_or_args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_compiled_binding_registers_every_schema(lib_built):
    code = (
        "import torch, brute_b200\n"
        "from brute_b200 import ops\n"
        "assert ops.BINDING == 'cpp'\n"
        "missing = [n for n in ops._CUDA_IMPLS if not torch._C._dispatch_has_kernel_for_dispatch_key('brute::' + n, 'CUDA')]\n"
        "assert not missing, missing\n"
        "try:\n"
        "    torch.ops.brute.pack_bool(torch.zeros(4, dtype=torch.bool))\n"
        "except NotImplementedError:\n"
        "    print('no-cpu-kernel')\n"
        "print('ok', len(ops._CUDA_IMPLS))\n")
    res = _run([sys.executable, "-c", code], {"BRUTE_B200_BINDING": "cpp"})
    assert res.returncode == 0, res.stderr[-2000:]
    assert "no-cpu-kernel" in res.stdout and "ok" in res.stdout


def test_status_codes_become_runtime_errors_with_their_number(lib_built):
    # formatting the number goes through the C++ iostream locale: a module that carries its own copy
    # of libstdc++ (a toolchain that links it statically) crashes here instead of raising
    from brute_b200 import _cbrute
    _cbrute._check_status(0)
    with pytest.raises(RuntimeError, match=r"not supported.*status -3"):
        _cbrute._check_status(-3)


def test_unknown_binding_name_is_rejected(lib_built):
    res = _run([sys.executable, "-c", "import brute_b200"], {"BRUTE_B200_BINDING": "jit"})
    assert res.returncode != 0 and "BRUTE_B200_BINDING" in res.stderr


def test_default_binding_is_the_compiled_one(lib_built):
    res = _run([sys.executable, "-c", "from brute_b200 import ops; print(ops.BINDING)"], {"BRUTE_B200_BINDING": ""})
    assert res.returncode == 0 and res.stdout.strip() == "cpp", res.stderr[-1000:]


@pytest.mark.gpu
def test_gpu_suites_pass_through_the_other_binding(lib_built):
    from brute_b200 import ops
    other = "ctypes" if ops.BINDING == "cpp" else "cpp"
    res = _run([sys.executable, "-m", "pytest", "tests/test_gpu_parity.py", "tests/test_frontend.py", "tests/test_gpu_streams.py",
                "tests/test_zz_no_alloc.py", "-m", "gpu", "-q", "-x", "-p", "no:cacheprovider"], {"BRUTE_B200_BINDING": other})
    tail = "\n".join(res.stdout.splitlines()[-25:])
    assert res.returncode == 0, tail + res.stderr[-1500:]
    assert " passed" in tail and " failed" not in tail
