#!/usr/bin/env python
"""Builds the reference implementation, unmodified, into ``baseline/_ref``.

The reference is a C++/CUDA project (no Python package), so it is built with its
own CMake files from a scratch copy of its CUDA library (the source tree itself
is never written to):

    python baseline/install_reference.py [--source /path/to/HyLink]

Result: ``baseline/_ref/libpccl.so``, ``baseline/_ref/libpccl_kernels.so`` and
its schedule files under ``baseline/_ref/ir``. ``bench.py --impl reference``
loads exactly these files.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("HYLINK_REFERENCE_SOURCE", "/root/reference"))
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    a = ap.parse_args()
    src = Path(a.source) / "pcie-ccl-cuda"
    if not src.is_dir():
        print(f"no reference source at {src}", file=sys.stderr)
        return 1
    dst = HERE / "_ref"
    with tempfile.TemporaryDirectory(prefix="hylink_ref_") as tmp:
        work = Path(tmp) / "pcie-ccl-cuda"
        shutil.copytree(src, work)
        build = work / "build"
        build.mkdir()
        env = dict(os.environ, CUDACXX=os.environ.get("CUDACXX", "/usr/local/cuda/bin/nvcc"))
        subprocess.check_call(["cmake", "-DCMAKE_BUILD_TYPE=Release", "-DPCCL_USE_CUDA=ON", "-DPCCL_CUDA_ARCHITECTURES=100", ".."],
                              cwd=build, env=env)
        subprocess.check_call(["make", f"-j{a.jobs}", "pccl"], cwd=build, env=env)
        dst.mkdir(parents=True, exist_ok=True)
        for name in ("libpccl.so", "libpccl_kernels.so"):
            found = list(build.rglob(name))
            if not found:
                print(f"{name} was not built", file=sys.stderr)
                return 1
            shutil.copy2(found[0], dst / name)
        if (dst / "ir").exists():
            shutil.rmtree(dst / "ir")
        shutil.copytree(work / "ir", dst / "ir")
    print("installed", dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
