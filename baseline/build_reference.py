"""Build the reference framework (unmodified sources) offline into ``baseline/_ref``.

The reference's Python package is a scikit-build-core project that is staged from
several directories of its tree (the recipe of its ``build-python.sh``) and that
expects four third-party trees under ``external_libs/`` which are empty in an
offline checkout. This script

1. stages the package under a scratch directory (default ``/tmp/falcata_ref_stage``):
   ``python-package/*`` at the root plus ``CMakeLists.txt``, ``cmake/``, ``include/``,
   ``src/``, ``swig/``, ``external_libs/nccl`` and the licence / version files, every
   reference file byte for byte;
2. fills ``external_libs/{fmt,fast_double_parser,eigen,nanoarrow}`` with stand-ins:
   the ``fmt`` headers that ship inside the installed ``torch`` wheel (compiled
   header-only) and the small files under ``baseline/standins`` for the other three;
3. runs ``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref``
   on the staged tree, CUDA + NCCL on, device code for sm_100 only.

Nothing of this repository's own package is involved; ``bench.py --impl reference``
imports ``falcata`` from ``baseline/_ref`` in a process that never imports
``falcata_b200``.

Usage: ``python baseline/build_reference.py [--stage DIR] [--jobs N] [--keep-stage]``
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
REF = Path(os.environ.get("FALCATA_REFERENCE_DIR", "/root/reference"))
TARGET = HERE / "_ref"


def _copy(src: Path, dst: Path) -> None:
    if src.is_dir():
        shutil.copytree(src, dst, dirs_exist_ok=True, symlinks=False)
    else:
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copy2(src, dst)


def stage(stage_dir: Path) -> None:
    if stage_dir.exists():
        shutil.rmtree(stage_dir)
    stage_dir.mkdir(parents=True)
    _copy(REF / "python-package", stage_dir)
    for name in ("CMakeLists.txt", "cmake", "include", "src", "swig", "LICENSE", "NOTICE"):
        if (REF / name).exists():
            _copy(REF / name, stage_dir / name)
    _copy(REF / "VERSION.txt", stage_dir / "falcata" / "VERSION.txt")
    ext = stage_dir / "external_libs"
    _copy(REF / "external_libs" / "nccl", ext / "nccl")
    # stand-ins for the empty third-party trees
    import torch  # only to locate the fmt headers bundled with the wheel

    fmt_src = Path(torch.__file__).resolve().parent / "include" / "fmt"
    if not fmt_src.is_dir():
        raise SystemExit(f"fmt headers not found at {fmt_src}")
    _copy(fmt_src, ext / "fmt" / "include" / "fmt")
    _copy(HERE / "standins" / "fast_double_parser", ext / "fast_double_parser")
    _copy(HERE / "standins" / "eigen", ext / "eigen")
    _copy(HERE / "standins" / "nanoarrow", ext / "nanoarrow")
    (ext / "compute").mkdir(exist_ok=True)


def install(stage_dir: Path, jobs: int) -> int:
    if TARGET.exists():
        shutil.rmtree(TARGET)
    env = dict(os.environ)
    env.setdefault("CMAKE_BUILD_PARALLEL_LEVEL", str(jobs))
    env.setdefault("CUDACXX", "/usr/local/cuda/bin/nvcc")
    # the system GCC ships libgomp; a wrapper compiler that CC/CXX may point at need not
    if Path("/usr/bin/gcc").exists() and Path("/usr/bin/g++").exists():
        env["CC"], env["CXX"], env["CUDAHOSTCXX"] = "/usr/bin/gcc", "/usr/bin/g++", "/usr/bin/g++"
    defines = {
        "CMAKE_CUDA_ARCHITECTURES": "100-real",
        "USE_CUDA": "ON",
        "USE_NCCL": "ON",
        "BUILD_CLI": "OFF",
        "INSTALL_HEADERS": "OFF",
        # the stand-in fmt is used header-only; warnings raised by a newer compiler
        # than the reference's CI must not stop the build
        "CMAKE_CXX_FLAGS": "-DFMT_HEADER_ONLY=1",
        "CMAKE_CUDA_FLAGS": "-DFMT_HEADER_ONLY=1",
        "USE_WERROR": "OFF",
    }
    cmd = [
        sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
        "--find-links", "/opt/wheelhouse", "--target", str(TARGET), "-v",
    ]
    for k, v in defines.items():
        cmd.append(f"--config-settings=cmake.define.{k}={v}")
    cmd.append(str(stage_dir))
    print(" ".join(cmd), flush=True)
    return subprocess.call(cmd, env=env)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--stage", default="/tmp/falcata_ref_stage")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--keep-stage", action="store_true")
    args = ap.parse_args()
    stage_dir = Path(args.stage)
    stage(stage_dir)
    rc = install(stage_dir, args.jobs)
    if rc == 0:
        libs = list(TARGET.rglob("lib_falcata.so"))
        print("installed:", [str(p) for p in libs])
        if not libs:
            rc = 1
    if not args.keep_stage and rc == 0:
        shutil.rmtree(stage_dir, ignore_errors=True)
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
