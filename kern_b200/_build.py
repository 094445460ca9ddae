"""In-tree build of the native pieces: sm_100a cubins (one per kernel source) and the C++ core.

The cubins are *built-in modules* of the package format: a manifest names them by file and sha256
exactly like any other pinned module (reference: crates/kern-runtime/src/cubin.rs:70-155 loads
modules by content hash). ``kernels/index.json`` is written at build time with the hash of every
cubin, so nothing hand-committed can go stale.

Everything is rebuilt only when a source is newer than its product; the products stay in the tree
(``kern_b200/kernels/*.cubin``, ``kern_b200/_native*.so``) so a copy of the tree runs without a
build step.
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import re
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "kern_b200"
CSRC = ROOT / "csrc"
KSRC = CSRC / "kernels" / "sm100"
KOUT = PKG / "kernels"
KOUT_CHECKED = PKG / "kernels_checked"
BUILD = ROOT / "build"

NVCC = os.environ.get("KERN_NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xptxas", "-v"]

# sources with host code for nvcc (C entry points reached through ctypes), one library per file
HSRC = CSRC / "kernels" / "host"


def _newer(src: list[Path], out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in src)


def _run(cmd: list[str], log: Path | None = None) -> str:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.parent.mkdir(parents=True, exist_ok=True)
        log.write_text(p.stdout)
    if p.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd) + "\n" + p.stdout[-4000:])
    return p.stdout


def kernel_sources() -> list[Path]:
    return sorted(KSRC.glob("*.cu"))


def checked() -> bool:
    """KERN_B200_CHECKED=1 selects the checked kernel build (``kernels_checked/``: every data-derived address is
    looked up in the runtime's table of allocations before it is used; common.cuh, KERN_CHECK)."""
    return os.environ.get("KERN_B200_CHECKED", "0") not in ("", "0")


def kernels_dir(checked_build: bool | None = None) -> Path:
    return KOUT_CHECKED if (checked() if checked_build is None else checked_build) else KOUT


def build_kernels(force: bool = False, verbose: bool = False, checked_build: bool = False) -> dict[str, dict]:
    """Compile every kernel source to ``kernels/<stem>.cubin`` (``kernels_checked/`` with -DKERN_CHECKED for the checked
    build); return the module index."""
    KOUT = kernels_dir(checked_build)
    KOUT.mkdir(parents=True, exist_ok=True)
    headers = sorted(KSRC.glob("*.cuh"))
    jobs = []
    for src in kernel_sources():
        out = KOUT / (src.stem + ".cubin")
        # a source that includes another kernel source (the GEMM body shared by several modules) depends on it too
        included = [KSRC / m for m in re.findall(r'#include\s+"([\w.]+\.cu)"', src.read_text())]
        if force or _newer([src, *headers, *included], out):
            jobs.append((src, out))

    def one(job):
        src, out = job
        cmd = [NVCC, *ARCH, *NVCC_FLAGS, *(["-DKERN_CHECKED"] if checked_build else []), "-cubin", "-I", str(KSRC), "-o", str(out), str(src)]
        text = _run(cmd, BUILD / ("ptxas_checked" if checked_build else "ptxas") / (src.stem + ".log"))
        if verbose:
            print(text)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(one, jobs))
    index = {}
    for src in kernel_sources():
        out = KOUT / (src.stem + ".cubin")
        data = out.read_bytes()
        index[src.stem] = {"source": out.name, "sha256": hashlib.sha256(data).hexdigest()}
    (KOUT / "index.json").write_text(json.dumps(index, indent=1, sort_keys=True))
    return index


def native_sources() -> list[Path]:
    out = sorted((CSRC / "bindings").glob("*.cpp"))
    for sub in ("manifest", "pool", "runtime"):
        out += sorted((CSRC / sub).glob("*.cpp"))
    return out


def native_path() -> Path:
    return PKG / ("_native" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_native(force: bool = False) -> Path:
    """Compile the C++ core (manifest, pool, runtime, bindings) into ``kern_b200/_native*.so``."""
    import pybind11

    out = native_path()
    srcs = native_sources()
    headers = [p for p in CSRC.rglob("*.hpp")]
    if not force and not _newer([*srcs, *headers], out):
        return out
    objdir = BUILD / "native"
    objdir.mkdir(parents=True, exist_ok=True)
    defs = []
    if (CSRC / "bindings" / "bind_manifest.cpp").exists():
        defs.append("-DKERN_WITH_MANIFEST")
    if (CSRC / "bindings" / "bind_pool.cpp").exists():
        defs.append("-DKERN_WITH_POOL")
    if (CSRC / "bindings" / "bind_runtime.cpp").exists():
        defs.append("-DKERN_WITH_RUNTIME")
    inc = [
        "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
        "-I", "/usr/local/cuda/include", "-I", str(CSRC),
    ]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", *defs]

    def one(src: Path):
        obj = objdir / (src.parent.name + "_" + src.stem + ".o")
        if force or _newer([src, *headers], obj):
            _run([CXX, *flags, *inc, "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(one, srcs))
    _run([CXX, "-shared", "-o", str(out), *map(str, objs), "-ldl", "-lpthread"])
    return out


def build_cli(force: bool = False) -> Path:
    """The native `kern` binary (verify / cut / print): the manifest library and a main, nothing else."""
    out = PKG / "bin" / "kern"
    srcs = [CSRC / "cli" / "kern_main.cpp", *sorted((CSRC / "manifest").glob("*.cpp"))]
    headers = [p for p in (CSRC / "manifest").glob("*.hpp")] + [p for p in (CSRC / "common").glob("*.hpp")]
    if not force and not _newer([*srcs, *headers], out):
        return out
    out.parent.mkdir(exist_ok=True)
    _run([CXX, "-O2", "-std=c++17", "-Wall", "-Wno-unused-function", "-I", str(CSRC), "-o", str(out), *map(str, srcs)])
    return out


def build_runner(force: bool = False) -> Path:
    """The native `kern-run` binary: manifest + pool + runtime (the CUDA driver and NCCL are reached by dlopen at run
    time, so it builds and links without a GPU) behind a single-sequence caller."""
    out = PKG / "bin" / "kern-run"
    srcs = [CSRC / "cli" / "kern_run.cpp", *sorted((CSRC / "manifest").glob("*.cpp")), *sorted((CSRC / "runtime").glob("*.cpp"))]
    headers = [p for p in CSRC.rglob("*.hpp")]
    if not force and not _newer([*srcs, *headers], out):
        return out
    out.parent.mkdir(exist_ok=True)
    _run([CXX, "-O2", "-std=c++17", "-Wall", "-Wno-unused-function", "-I", str(CSRC), "-I", "/usr/local/cuda/include", "-o", str(out),
          *map(str, srcs), "-ldl", "-lpthread"])
    return out


def build_capture(force: bool = False) -> Path:
    """`libkern_capture.so`, the injection library that records a process's module loads, allocations, descriptor encodes
    and launches (`csrc/capture/kern_capture.cpp`; read by `kern_b200/capture.py`). Opens the driver and the profiling
    interface at run time, so it builds and loads anywhere."""
    out = PKG / "libkern_capture.so"
    src = CSRC / "capture" / "kern_capture.cpp"
    if force or _newer([src, CSRC / "common" / "sha256.hpp"], out):
        _run([CXX, "-O2", "-std=c++17", "-Wall", "-shared", "-fPIC", "-I", str(CSRC), "-o", str(out), str(src), "-ldl", "-lpthread"])
    return out


def build_host_libs(force: bool = False) -> list[Path]:
    """Shared libraries with host code compiled by nvcc (C entry points reached through ctypes)."""
    outs = []
    for src in sorted(HSRC.glob("*.cu")):
        out = PKG / ("lib" + src.stem + ".so")
        if force or _newer([src, *HSRC.glob("*.h"), *KSRC.glob("*.cuh"), *KSRC.glob("*.cu")], out):   # host sources include kernel sources
            _run([NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
                  "-I", str(KSRC), "-o", str(out), str(src), "-lcudart"])
        outs.append(out)
    return outs


def build_all(force: bool = False, verbose: bool = False) -> None:
    BUILD.mkdir(exist_ok=True)
    with open(BUILD / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            build_kernels(force, verbose)
            if checked() or "--checked" in sys.argv:
                build_kernels(force, verbose, checked_build=True)
            build_native(force)
            build_cli(force)
            build_runner(force)
            build_capture(force)
            build_host_libs(force)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def ensure_built() -> None:
    """Build whatever is missing or stale. Cheap when everything is current."""
    try:
        build_all(False)
    except FileNotFoundError as e:  # no compiler on this machine: use what is in the tree
        if not native_path().exists():
            raise RuntimeError(f"native core is not built and no toolchain was found: {e}")


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", native_path().name, "+", len(kernel_sources()), "cubins")
