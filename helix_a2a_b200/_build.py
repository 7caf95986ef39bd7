"""In-tree build of the native extension ``helix_a2a_b200/_C*.so`` for sm_100a.

Kernels (``csrc/*.cu``) are compiled by nvcc with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and include only CUDA headers, so
they build in seconds; the two binding files are compiled by g++ against the torch
headers.  Objects land in ``build/`` and are rebuilt only when a source or header is newer.
The reference builds through ``setup.py`` with sm_90/sm_90a/sm_100 (``setup.py:14-20``);
this library targets B200 only.

``python -m helix_a2a_b200._build`` builds from the command line.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
PKG = ROOT / "helix_a2a_b200"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = PKG / f"_C{EXT_SUFFIX}"
HOST_TARGET = PKG / "_ll128_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wno-deprecated-declarations"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _headers() -> List[Path]:
    return sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")))


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    if src.stat().st_mtime > t or Path(__file__).stat().st_mtime > t:
        return True
    return any(h.stat().st_mtime > t for h in _headers())


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def cuda_sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def cpp_sources() -> List[Path]:
    return sorted(p for p in CSRC.glob("*.cpp") if not p.name.startswith("host_"))


def build_host_lib(force: bool = False) -> Path:
    """g++-only library with the LL128 / FIFO protocol arithmetic for CPU unit tests."""
    src = CSRC / "host_protocol.cpp"
    if force or _stale(HOST_TARGET, src):
        BUILD.mkdir(exist_ok=True)
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", str(CSRC), "-isystem", str(_cuda_home() / "include"),
              str(src), "-o", str(HOST_TARGET)])
    return HOST_TARGET


def build(force: bool = False, verbose: bool = False) -> Path:
    import torch  # noqa: F401  (needed for include / library paths)
    from torch.utils import cpp_extension as ce

    BUILD.mkdir(exist_ok=True)
    cuda_home = _cuda_home()
    jobs = []
    objs: List[Path] = []
    for src in cuda_sources():
        obj = BUILD / (src.stem + ".cu.o")
        objs.append(obj)
        if force or _stale(obj, src):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-isystem", str(cuda_home / "include")]
    defs = ["-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for src in cpp_sources():
        obj = BUILD / (src.stem + ".cpp.o")
        objs.append(obj)
        if force or _stale(obj, src):
            jobs.append(["g++", *CXX_FLAGS, *defs, "-I", str(CSRC), *inc, "-c", str(src), "-o", str(obj)])
    if jobs:
        if verbose:
            for j in jobs:
                print(" ".join(j), file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    if jobs or not TARGET.exists():
        torch_lib = Path(torch.__file__).parent / "lib"
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objs),
                f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}",
                "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                f"-L{cuda_home / 'lib64'}", "-lcudart"]
        _run(link)
    build_host_lib(force)
    return TARGET


def is_built() -> bool:
    return TARGET.exists()


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose=True)
    print(out)
