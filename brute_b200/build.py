"""Build the native parts in-tree: ``python -m brute_b200.build``.

* ``csrc/*.cu`` are compiled for sm_100a only and linked into ``brute_b200/libbrute_b200.so``
  (a plain C-ABI shared library, no torch or Python types in it). nvcc cross-compiles without a
  GPU; objects are rebuilt only when a source or header is newer.
* ``csrc_host/cbrute.cpp`` becomes the Python extension module ``brute_b200/_cbrute.so`` (g++
  against the installed torch): the front end's tensor-implementation helpers and the compiled
  ``torch.ops.brute`` binding, which calls the C ABI of the library above.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OBJ_DIR = PKG / "build"
LIB = PKG / "libbrute_b200.so"
HOST_SRC = PKG / "csrc_host" / "cbrute.cpp"
HOST_MOD = PKG / "_cbrute.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _headers_mtime()):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile and link; returns the path of the shared library."""
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    build_host_module(force)
    return LIB


def build_host_module(force: bool = False) -> Path:
    """Compile ``_cbrute`` (pybind11 + torch headers, host code only) and link it to the library."""
    deps = [HOST_SRC, *INCLUDE.glob("*.h")]
    if not force and HOST_MOD.exists() and HOST_MOD.stat().st_mtime > max(d.stat().st_mtime for d in deps):
        return HOST_MOD
    import sysconfig
    import torch
    tdir = Path(torch.__file__).resolve().parent
    # The system g++, not $CXX: a toolchain that links libstdc++ statically (some CI wrappers do)
    # would put a second copy of the iostream locale state into this module, and formatting a
    # number in an error message would then crash. Checked below.
    cxx = next((c for c in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")) if c and Path(c).exists()), "g++")
    cuda_home = Path(_nvcc()).resolve().parent.parent
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-attributes",
           "-DTORCH_EXTENSION_NAME=_cbrute", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
           f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}", f"-I{cuda_home / 'include'}",
           str(HOST_SRC), "-o", str(HOST_MOD),
           f"-L{tdir / 'lib'}", "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python",
           f"-L{PKG}", "-l:libbrute_b200.so",
           f"-Wl,-rpath,{tdir / 'lib'}", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building _cbrute failed:\n{res.stdout}\n{res.stderr}")
    syms = subprocess.run(["nm", "-D", "--defined-only", str(HOST_MOD)], capture_output=True, text=True).stdout
    if "_ZNKSt6locale2id5_M_idEv" in syms:
        HOST_MOD.unlink()
        raise RuntimeError(f"{cxx} linked libstdc++ statically into _cbrute.so; build it with a g++ that links "
                           "libstdc++.so (the system compiler)")
    return HOST_MOD


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
