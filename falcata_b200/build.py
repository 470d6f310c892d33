"""In-tree build of the native core (``falcata_b200/lib/libfalcata_core.so``).

Host sources are compiled with g++, device sources with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``); objects are cached by mtime under
``csrc/build`` and compiled in parallel. The library links the CUDA runtime statically so it
also loads on a machine without a GPU (the CPU learner and the model code work there).

Run ``python -m falcata_b200.build`` (add ``--force`` to rebuild everything, ``--ptxas`` to
print register / shared-memory usage of every kernel).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
BUILD = CSRC / "build"
LIB = ROOT / "lib" / "libfalcata_core.so"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", f"-I{CSRC / 'include'}"]
HOST_FLAGS = ["-fPIC", "-fopenmp", "-ffp-contract=off", "-Wall", "-Wno-sign-compare", "-Wno-unused-function"]


def _sources():
    cpp = sorted(CSRC.glob("core/*.cpp")) + sorted(CSRC.glob("cuda/*.cpp"))
    cu = sorted(CSRC.glob("cuda/*.cu"))
    return cpp, cu


def _newest_header() -> float:
    return max((p.stat().st_mtime for p in list(CSRC.glob("include/fb/*.h")) + list(CSRC.glob("cuda/*.cuh")) + list(CSRC.glob("cuda/*.h"))), default=0.0)


def _compile(src: Path, obj: Path, ptxas: bool) -> str:
    if src.suffix == ".cu":
        cmd = [NVCC, *ARCH, "-lineinfo", *COMMON, "--expt-relaxed-constexpr", "-Xcompiler", ",".join(HOST_FLAGS),
               "-Xcudafe", "--diag_suppress=177", "-c", str(src), "-o", str(obj)]
        if ptxas:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = [CXX, *COMMON, *HOST_FLAGS, "-I/usr/local/cuda/include", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stderr if ptxas else ""


def build_sanitized() -> Path:
    """Host-only build of the core library with AddressSanitizer and UndefinedBehaviorSanitizer, for running the CPU
    tests under sanitizers (``FALCATA_LIB=<path> python -m pytest tests -m "not gpu"`` with libasan preloaded).
    The CUDA translation units are left out: device_type=cpu only."""
    out_dir = BUILD / "asan"; out_dir.mkdir(parents=True, exist_ok=True)
    cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else CXX   # the system compiler ships libasan / libubsan / libgomp
    cpp = sorted(CSRC.glob("core/*.cpp"))
    objs = []
    for src in cpp:
        obj = out_dir / (src.stem + ".o"); objs.append(obj)
        cmd = [cxx, "-std=c++17", "-O1", "-g", f"-I{CSRC / 'include'}", "-I/usr/local/cuda/include", "-fPIC", "-fopenmp", "-ffp-contract=off",
               "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-DFB_NO_CUDA=1", "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stderr}")
    lib = LIB.parent / "libfalcata_core_asan.so"
    r = subprocess.run([cxx, "-shared", "-fsanitize=address,undefined", "-fopenmp", "-o", str(lib), *map(str, objs), "-lz"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed\n{r.stderr}")
    return lib


def build(force: bool = False, ptxas: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    cpp, cu = _sources()
    hdr_time = _newest_header()
    jobs = []
    objs = []
    for src in cpp + cu:
        obj = BUILD / (src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        stale = force or ptxas or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            futs = {ex.submit(_compile, s, o, ptxas and s.suffix == ".cu"): s for s, o in jobs}
            for fut in cf.as_completed(futs):
                out = fut.result()
                if verbose:
                    print(f"compiled {futs[fut].name}", file=sys.stderr)
                if out:
                    logs.append(f"==== {futs[fut].name}\n{out}")
    if jobs or not LIB.exists():
        # link beside the target and rename: a reader (an import, a copy of the tree) never sees a half-written library
        tmp = LIB.with_name(LIB.name + ".tmp")
        cmd = [NVCC, *ARCH, "-shared", "-Xcompiler", "-fPIC,-fopenmp", "-o", str(tmp), *map(str, objs), "-lz", "-lgomp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    if ptxas:
        print("\n".join(logs))
    _build_cli()
    _build_native_tests()
    return LIB


def _build_cli() -> Path:
    """The command-line application (train / predict / convert_model / refit / save_binary), linked against the core library."""
    src = CSRC / "cli" / "main.cpp"
    exe = LIB.parent.parent / "bin" / "falcata"
    exe.parent.mkdir(parents=True, exist_ok=True)
    if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, LIB.stat().st_mtime):
        return exe
    cmd = [CXX, *COMMON, "-ffp-contract=off", str(src), "-o", str(exe), f"-L{LIB.parent}", "-lfalcata_core", "-Wl,-rpath,$ORIGIN/../lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"CLI build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return exe


def _build_native_tests() -> Path:
    """Native unit tests of the core (plain asserts), linked against the core library: bin/falcata_core_tests."""
    src = CSRC / "tests" / "core_tests.cpp"
    exe = LIB.parent.parent / "bin" / "falcata_core_tests"
    exe.parent.mkdir(parents=True, exist_ok=True)
    if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, LIB.stat().st_mtime, _newest_header()):
        return exe
    cmd = [CXX, *COMMON, "-ffp-contract=off", str(src), "-o", str(exe), f"-L{LIB.parent}", "-lfalcata_core", "-Wl,-rpath,$ORIGIN/../lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"native test build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return exe


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_sanitized()); sys.exit(0)
    p = build(force="--force" in sys.argv, ptxas="--ptxas" in sys.argv, verbose=True)
    print(p)
