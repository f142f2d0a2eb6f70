"""In-tree build of the native libraries.

Produces, under ``hylink_b200/lib/``:

* ``libhylink_b200.so`` — the whole collective stack (core, control plane,
  schedule IR, host SIMD, PCIe executor, sm_100a kernels, orchestrator, C API).
  Host code is compiled with g++, device code with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``; the CUDA runtime is linked
  statically and the driver is resolved at run time, so the library also loads
  on a machine without a GPU.
* ``libhylink_nccl.so`` — the drop-in ``nccl*`` symbol layer; ``libhylink_cudashim.so`` — opt-in
  interposers of host-blocking CUDA runtime calls.
* ``_hylink_c10d.so`` — the ``torch.distributed`` backend extension.

and ``hylink_b200/bin/hl_perf``, the stand-alone test executable.

Objects are rebuilt only when a source or any header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shlex
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build" / "obj"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

CORE_DIRS = ["core", "ctrl", "hal", "ir", "host", "pcie", "nvl", "orch", "api"]
SEPARATE = {"nccl_shim.cpp", "cuda_block_shim.cpp"}  # built into libhylink_nccl.so


def _run(cmd: list[str]) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(shlex.quote(c) for c in cmd), p.stdout))


def _newest_header() -> float:
    t = 0.0
    for ext in ("*.h", "*.cuh", "*.hpp"):
        for f in CSRC.rglob(ext):
            t = max(t, f.stat().st_mtime)
    return t


def _compile(src: Path, obj: Path, hdr_time: float, extra: list[str]) -> bool:
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_time):
        return False
    obj.parent.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(CSRC), "-I", str(CSRC / "include"), "-I", str(CUDA_HOME / "include")]
    if src.suffix == ".cu":
        cmd = [NVCC, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
               *inc, *extra, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", "-O2", "-g1", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function",
               "-pthread", *inc, *extra, "-c", str(src), "-o", str(obj)]
    _run(cmd)
    return True


def core_sources() -> list[Path]:
    out: list[Path] = []
    for d in CORE_DIRS:
        p = CSRC / d
        if not p.is_dir():
            continue
        for f in sorted(p.iterdir()):
            if f.suffix in (".cpp", ".cu") and f.name not in SEPARATE:
                out.append(f)
    return out


def build_core(verbose: bool = False) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    srcs = core_sources()
    objs = [OBJ / (s.relative_to(CSRC).as_posix().replace("/", "_") + ".o") for s in srcs]
    vis = ["-DHL_BUILDING=1"]
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        changed = list(ex.map(lambda so: _compile(so[0], so[1], hdr, vis), zip(srcs, objs)))
    target = LIB / "libhylink_b200.so"
    if any(changed) or not target.exists():
        cmd = [NVCC, *ARCH_FLAGS, "-shared", "-o", str(target), *map(str, objs), "-cudart", "static",
               "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        _run(cmd)
        if verbose:
            print("linked", target)
    return target


def build_nccl_shim(verbose: bool = False) -> Path | None:
    """libhylink_nccl.so (drop-in nccl* symbols) and libhylink_cudashim.so (opt-in interposers of blocking CUDA calls)."""
    hdr = _newest_header()
    out = None
    plan = [("nccl_shim.cpp", "libhylink_nccl.so", ["-L", str(CUDA_HOME / "lib64"), "-lcudart_static"]),
            ("cuda_block_shim.cpp", "libhylink_cudashim.so", []),
            ("../tools/nccl_trace.cpp", "libhylink_nccltrace.so", ["-L", str(CUDA_HOME / "lib64"), "-lcudart_static"])]
    for src_name, lib_name, extra in plan:
        src = (CSRC / "api" / src_name).resolve()
        if not src.exists():
            continue
        obj = OBJ / ("shim_" + Path(src_name).name + ".o")
        changed = _compile(src, obj, hdr, [])
        target = LIB / lib_name
        if changed or not target.exists():
            core = [] if "nccltrace" in lib_name else ["-L", str(LIB), "-lhylink_b200", "-Wl,-rpath,$ORIGIN"]
            # -Bsymbolic-functions: calls between this library's own nccl* entry points stay inside it even when the
            # process has another library with the same names loaded (the real NCCL)
            _run(["g++", "-shared", "-Wl,-Bsymbolic-functions", "-o", str(target), str(obj), *core, *extra, "-lpthread", "-ldl", "-lrt"])
            if verbose:
                print("linked", target)
        out = out or target
    return out


def build_torch_ext(verbose: bool = False) -> Path | None:
    src = CSRC / "torch" / "backend.cpp"
    if not src.exists():
        return None
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    target = LIB / "_hylink_c10d.so"
    hdr = _newest_header()
    if target.exists() and target.stat().st_mtime > max(src.stat().st_mtime, hdr):
        return target
    tlib = Path(torch.__file__).parent / "lib"
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}",
                                                     f"-I{CSRC}", f"-I{CSRC / 'include'}", f"-I{CUDA_HOME / 'include'}"]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-DTORCH_EXTENSION_NAME=_hylink_c10d",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-Wno-interference-size", *inc, str(src), "-o", str(target), f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-ltorch_python", "-ltorch_cuda", "-lc10_cuda", f"-L{LIB}", "-lhylink_b200",
           f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN", f"-L{CUDA_HOME / 'lib64'}", "-lcudart"]
    _run(cmd)
    if verbose:
        print("built", target)
    return target


def build_tools(verbose: bool = False) -> Path:
    """hylink_b200/bin/hl_perf: stand-alone correctness + bandwidth test executable."""
    bindir = ROOT / "bin"
    bindir.mkdir(parents=True, exist_ok=True)
    src = CSRC / "tools" / "hl_perf.cpp"
    obj = OBJ / "tools_hl_perf.cpp.o"
    changed = _compile(src, obj, _newest_header(), [])
    target = bindir / "hl_perf"
    if changed or not target.exists():
        _run(["g++", "-o", str(target), str(obj), "-L", str(LIB), "-lhylink_b200", "-Wl,-rpath,$ORIGIN/../lib",
              "-L", str(CUDA_HOME / "lib64"), "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
        if verbose:
            print("linked", target)
    return target


def build_sanitized(kind: str = "thread", verbose: bool = False) -> Path:
    """Host code under ``-fsanitize=thread`` or ``address``: a second copy of the library and of ``hl_perf`` in
    ``hylink_b200/build/san_<kind>/`` (device objects are reused unchanged). Run the tool there with
    ``--device host`` to check the control plane, the executor and the worker pool for races or bad accesses."""
    assert kind in ("thread", "address")
    build_core(verbose)  # device objects come from the regular build
    out = ROOT / "build" / f"san_{kind}"
    out.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    flags = [f"-fsanitize={kind}", "-O1", "-g", "-fno-omit-frame-pointer", "-DHL_BUILDING=1"]
    srcs = [s for s in core_sources() if s.suffix == ".cpp"]
    objs = [out / (s.relative_to(CSRC).as_posix().replace("/", "_") + ".o") for s in srcs]
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        list(ex.map(lambda so: _compile(so[0], so[1], hdr, flags), zip(srcs, objs)))
    dev_objs = [OBJ / (s.relative_to(CSRC).as_posix().replace("/", "_") + ".o") for s in core_sources() if s.suffix == ".cu"]
    lib = out / "libhylink_b200.so"
    _run([NVCC, *ARCH_FLAGS, "-shared", "-o", str(lib), *map(str, objs), *map(str, dev_objs), "-cudart", "static",
          "-Xcompiler", f"-fsanitize={kind}", "-lpthread", "-ldl", "-lrt"])
    tool_obj = out / "hl_perf.o"
    _compile(CSRC / "tools" / "hl_perf.cpp", tool_obj, hdr, flags)
    tool = out / "hl_perf"
    _run(["g++", f"-fsanitize={kind}", "-o", str(tool), str(tool_obj), "-L", str(out), "-lhylink_b200", "-Wl,-rpath,$ORIGIN",
          "-L", str(CUDA_HOME / "lib64"), "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    if verbose:
        print("built", tool)
    return tool


def build_all(verbose: bool = False) -> None:
    build_core(verbose)
    build_nccl_shim(verbose)
    build_torch_ext(verbose)
    build_tools(verbose)


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[1] == "--sanitize":
        print(build_sanitized(sys.argv[2], verbose=True))
        sys.exit(0)
    build_all(verbose=True)
    print("ok")
