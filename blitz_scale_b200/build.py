"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host-side C++ cores.

Everything lands in ``blitz_scale_b200/_lib`` so the shared objects travel with
the source tree.  ``python -m blitz_scale_b200.build`` rebuilds what is stale;
``build_all(force=True)`` rebuilds everything.  The reference builds with
CMake for sm_80 (CMakeLists.txt:42-102); this build targets sm_100a only.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"
OBJ = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wno-sign-compare", "-pthread", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_files, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_files)


def _run(cmd, log: Path | None = None):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))


def build_kernels(force: bool = False) -> Path:
    """Compile every .cu under csrc/kernels and csrc/comm into libblitz_kernels.so."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "kernels").glob("*.h")) + \
        list((CSRC / "comm").glob("*.cuh"))
    srcs = kernel_sources()
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or _newer([s] + headers, o):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC / "kernels"), "-I", str(CSRC / "comm"), "-c", str(s),
                         "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = [ex.submit(_run, j, OBJ / (Path(j[-1]).stem + ".ptxas.log")) for j in jobs]
        for f in futs:
            f.result()
    out = LIB / "libblitz_kernels.so"
    if force or jobs or not out.exists():
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def _pybind_includes():
    import pybind11
    return ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]


def build_host(force: bool = False):
    """Compile the C++ cores (runtime, router, simulator) and their pybind11 module."""
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    bind = CSRC / "bindings" / "core_module.cpp"
    if not bind.exists():
        return None
    dirs = [CSRC / "runtime", CSRC / "router", CSRC / "sim", CSRC / "bindings"]
    srcs = [p for d in dirs for p in sorted(d.glob("*.cpp"))]
    headers = [p for d in dirs for p in d.glob("*.h*")]
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = LIB / f"blitz_core{ext}"
    cxx = os.environ.get("CXX", "g++")
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / (s.parent.name + "_" + s.stem + ".o")
        objs.append(o)
        if force or _newer([s] + headers, o):
            jobs.append([cxx, *CXX_FLAGS, *_pybind_includes(), "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for f in [ex.submit(_run, j) for j in jobs]:
            f.result()
    if force or jobs or not out.exists():
        # static libstdc++ with local symbol binding: the module must not resolve C++ runtime symbols against
        # whichever libstdc++ another extension (torch) loaded first
        _run([cxx, "-shared", "-o", str(out), *map(str, objs), "-pthread", "-static-libstdc++", "-static-libgcc",
              "-Wl,-Bsymbolic", "-Wl,--exclude-libs,ALL"])
    return out


def build_all(force: bool = False):
    k = build_kernels(force)
    h = build_host(force)
    return k, h


def main() -> int:
    k, h = build_all(force="--force" in sys.argv)
    print("built", k, h)
    return 0


if __name__ == "__main__":
    sys.exit(main())
