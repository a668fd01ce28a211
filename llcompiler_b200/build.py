"""Builds the native parts in-tree: ``lib/libllc_cuda.so`` (compiler + CUDA kernel
library + executor behind the C ABI of include/llc_runtime.h and include/llc_cuda.h)
and the ``llcompiler_`` pybind11 module that binds it with the reference's class names.

The reference builds LLVM/MLIR, StableHLO, SymEngine and spdlog through a CMake
superbuild before its own sources (CMakeLists.txt:28-176, setup.py:86-186); nothing of
that is needed here: every source is in ``csrc/`` and is compiled with nvcc / g++ only.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
OBJ_DIR = ROOT / "build"
LIB = LIB_DIR / "libllc_cuda.so"
INCLUDE = ROOT.parent / "include"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", f"-I{INCLUDE}", f"-I{CSRC}"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", f"-I{INCLUDE}", f"-I{CSRC}",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"] + ARCH


def _headers() -> List[Path]:
    return list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(INCLUDE.glob("*.h"))


def _digest(deps: List[Path], extra: str = "") -> str:
    import hashlib
    h = hashlib.sha1(extra.encode())
    for d in sorted(deps):
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def _stale(target: Path, deps: List[Path], extra: str = "") -> bool:
    """A target is rebuilt when the content of its inputs changed (a content stamp, not mtimes:
    a copied tree keeps the built objects valid)."""
    stamp = target.with_name(target.name + ".stamp")
    if not target.exists() or not stamp.exists():
        return True
    return stamp.read_text() != _digest(deps, extra)


def _mark(target: Path, deps: List[Path], extra: str = "") -> None:
    target.with_name(target.name + ".stamp").write_text(_digest(deps, extra))


def _compile_one(src: Path, obj: Path, verbose: bool) -> str:
    if src.suffix == ".cu":
        cmd = [NVCC] + NVCC_FLAGS + ["-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++"] + CXX_FLAGS + ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    (obj.with_suffix(".log")).write_text(" ".join(cmd) + "\n" + log)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src.name} failed:\n{log[-6000:]}")
    return log


def build_library(verbose: bool = False, force: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sorted(p for p in CSRC.rglob("*") if p.suffix in (".cpp", ".cu") and "pybind" not in p.parts)
    hdrs = _headers()
    jobs = []
    objs = []
    flags = " ".join(NVCC_FLAGS + CXX_FLAGS)
    for s in srcs:
        o = OBJ_DIR / (s.relative_to(CSRC).as_posix().replace("/", "_") + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs, flags):
            jobs.append((s, o))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            for log in ex.map(lambda j: _compile_one(j[0], j[1], verbose), jobs):
                if verbose:
                    print(log)
        for s, o in jobs:
            _mark(o, [s] + hdrs, flags)
    if jobs or not LIB.exists():
        cmd = [NVCC, "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ARCH + ["-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("linking libllc_cuda.so failed:\n" + r.stdout + r.stderr)
    return LIB


def pybind_module_path() -> Path:
    return ROOT.parent / ("llcompiler_" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_pybind(force: bool = False) -> Path:
    import pybind11
    src = CSRC / "pybind" / "entrance.cpp"
    out = pybind_module_path()
    deps = [src] + _headers()
    if force or _stale(out, deps) or out.stat().st_mtime < LIB.stat().st_mtime - 1e9:
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-I{pybind11.get_include()}",
               f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}", str(src), "-o", str(out),
               f"-L{LIB_DIR}", "-lllc_cuda", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN/llcompiler_b200/lib"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the llcompiler_ module failed:\n" + r.stdout + r.stderr)
        _mark(out, deps)
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_library(verbose, force)
    if (CSRC / "pybind" / "entrance.cpp").exists():
        build_pybind(force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", LIB)
