"""ctypes binding of ``libhylink_b200.so``.

The library is built in-tree by :mod:`hylink_b200._build`; if it is missing it
is built on first import. There is no pure-Python fallback for the device
paths: on a machine with a GPU a missing library is an error, never a silent
detour through eager PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_LIB_PATH = _LIB_DIR / "libhylink_b200.so"


class HylinkError(RuntimeError):
    def __init__(self, code: int, where: str = ""):
        self.code = code
        msg = lib.hlGetErrorString(code).decode()
        detail = lib.hlGetLastError().decode()
        super().__init__(f"{where}: {msg}" + (f" ({detail})" if detail else ""))


def _load() -> C.CDLL:
    if not _LIB_PATH.exists() or os.environ.get("HYLINK_REBUILD") == "1":
        from . import _build

        _build.build_core()
    return C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

# hlDataType_t / hlRedOp_t numbering (identical to NCCL's)
DTYPES = {"int8": 0, "uint8": 1, "int32": 2, "uint32": 3, "int64": 4, "uint64": 5, "float16": 6, "float32": 7,
          "float64": 8, "bfloat16": 9}
OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
RESULTS = ["success", "invalid argument", "system error", "internal error", "device error", "network error",
           "timeout", "unsupported", "remote rank error"]


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


class CallOpts(C.Structure):
    _fields_ = [("path", C.c_int), ("algo", C.c_int), ("out_type", C.c_int), ("has_out_type", C.c_int),
                ("wire_type", C.c_int), ("has_wire_type", C.c_int), ("scale", C.c_float), ("max_blocks", C.c_int),
                ("deterministic", C.c_int)]


class CommStats(C.Structure):
    _fields_ = [("calls", C.c_uint64), ("bytes", C.c_uint64), ("nvl_bytes", C.c_uint64), ("pcie_bytes", C.c_uint64),
                ("kernel_launches", C.c_uint64), ("copy_engine_ops", C.c_uint64), ("last_alpha", C.c_double),
                ("last_fast_ms", C.c_double), ("last_pcie_ms", C.c_double), ("nvls", C.c_int), ("symm_mode", C.c_int),
                ("fused_landing_slices", C.c_uint64), ("folded_sources", C.c_uint64), ("registered_bytes", C.c_uint64), ("small_path_calls", C.c_uint64),
                ("h2h_range_jobs", C.c_uint64), ("composed_allreduces", C.c_uint64)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name, None)
    if fn is None:
        return
    fn.restype = restype
    fn.argtypes = list(argtypes)


_vp, _sz, _i, _f, _u64p = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.POINTER(C.c_uint64)
_sig("hlGetErrorString", C.c_char_p, _i)
_sig("hlGetLastError", C.c_char_p)
_sig("hlVersion", _i)
_sig("hlTypeSize", _sz, _i)
_sig("hlGetUniqueId", _i, C.POINTER(UniqueId))
_sig("hlCommInitRank", _i, C.POINTER(_vp), _i, UniqueId, _i)
_sig("hlCommInitRankDevice", _i, C.POINTER(_vp), _i, UniqueId, _i, _i)
_sig("hlCommDestroy", _i, _vp)
_sig("hlCommAbort", _i, _vp)
_sig("hlCommRank", _i, _vp, C.POINTER(_i))
_sig("hlCommSize", _i, _vp, C.POINTER(_i))
_sig("hlCommGetAsyncError", _i, _vp, C.POINTER(_i))
_sig("hlAllReduce", _i, _vp, _vp, _sz, _i, _i, _vp, _vp)
_sig("hlAllReduceEx", _i, _vp, _vp, _sz, _i, _i, C.POINTER(CallOpts), _vp, _vp)
_sig("hlReduceScatter", _i, _vp, _vp, _sz, _i, _i, _vp, _vp)
_sig("hlReduceScatterEx", _i, _vp, _vp, _sz, _i, _i, C.POINTER(CallOpts), _vp, _vp)
_sig("hlAllGather", _i, _vp, _vp, _sz, _i, _vp, _vp)
_sig("hlAllGatherEx", _i, _vp, _vp, _sz, _i, C.POINTER(CallOpts), _vp, _vp)
_sig("hlBroadcast", _i, _vp, _vp, _sz, _i, _i, _vp, _vp)
_sig("hlBroadcastEx", _i, _vp, _vp, _sz, _i, _i, C.POINTER(CallOpts), _vp, _vp)
_sig("hlAllToAll", _i, _vp, _vp, _sz, _i, _vp, _vp)
_sig("hlAllToAllEx", _i, _vp, _vp, _sz, _i, C.POINTER(CallOpts), _vp, _vp)
_sig("hlBarrier", _i, _vp, _vp)
_sig("hlCommGetStats", _i, _vp, C.POINTER(CommStats))
_sig("hlCommDumpTuning", _i, _vp, C.c_char_p, C.POINTER(_sz))
_sig("hlCommLoadTuning", _i, _vp, C.c_char_p)
_sig("hlEmuCreate", _i, _i, _i, _sz, _i, C.POINTER(_vp))
_sig("hlEmuDestroy", _i, _vp)
_sig("hlEmuCollective", _i, _vp, _i, C.POINTER(_vp), C.POINTER(_vp), _sz, _sz, _sz, _i, _i, _i, _i, _f, _i, _i, _i, _vp)
_sig("hlEmuSetActiveRanks", _i, _vp, _i)
_sig("hlEmuHeapAlloc", _i, _vp, _sz, C.POINTER(_vp))
_sig("hlEmuHeapFree", _i, _vp, _vp)
_sig("hlMemAlloc", _i, _vp, _sz, C.POINTER(_vp))
_sig("hlMemFree", _i, _vp, _vp)
_sig("hlMemIsRegistered", _i, _vp, _vp, _sz)
_sig("hlEmuStatus", _i, _vp, _i, _u64p, _u64p, _u64p)
_sig("hlEmuReset", _i, _vp)
_sig("hlEmuLaunches", _i, _vp, _u64p)
class IrInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("nranks", "instructions", "dependency_edges", "input_chunks", "output_chunks",
                                        "internal_chunks", "host_chunks", "numa_nodes", "uses_remote_device",
                                        "uses_host_reduce")]


_sig("hlIrGenerate", _i, C.c_char_p, C.c_char_p, C.c_char_p, _i, C.c_char_p, C.POINTER(_sz))
_sig("hlIrInspect", _i, C.c_char_p, C.c_char_p, _i, _i, _i, C.POINTER(IrInfo))
_sig("hlIrRoundTrip", _i, C.c_char_p, C.c_char_p, C.POINTER(_sz))
_sig("hlSubmitIr", _i, _vp, C.c_char_p, _vp, _vp, _sz, _sz, _i, _i, _i, _i, _vp)
_sig("hlCommNumaPattern", _i, _vp, C.c_char_p, C.POINTER(_sz))
_sig("hlCommDrain", _i, _vp)
_sig("hlHostReduce", _i, _vp, _vp, _vp, _sz, _i, _i, _i)
_sig("hlHostCopy", None, _vp, _vp, _sz, _i)
_sig("hlHostSimdLevel", _i)
_sig("hlCommKernelTimeline", _i, _vp, _u64p, C.POINTER(_sz))
_sig("hlEmuKernelTimeline", _i, _vp, _i, _u64p, C.POINTER(_sz))
_sig("hlNvlStageAccess", _i, _vp, _i, _sz, _vp, _sz)
_sig("hlNvlStageBytes", _sz, _vp)
_sig("hlNvlLinkProbe", _i, _vp, _i, _i, _i, _i, _i, _sz, _vp)
_sig("hlHostBench", _i, _i, _sz, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_double), C.POINTER(C.c_double))
_sig("hlHostNumaNodes", _i)
_sig("hlTraceOpen", None, C.c_char_p, _i)
_sig("hlTraceFlush", None)
_sig("hlConfigReload", None)
_sig("pcclReduceScatterStridedTyped", _i, _vp, _vp, _sz, _sz, _i, _i, _vp, _vp)
_sig("pcclAllGatherStridedTyped", _i, _vp, _vp, _sz, _sz, _i, _vp, _vp)
_sig("pcclAllToAllStridedTyped", _i, _vp, _vp, _sz, _sz, _i, _vp, _vp)
_sig("hlCtrlSelfTest", _i, UniqueId, _i, _i, _i)
_sig("hlReduceLanding", _i, _vp, C.POINTER(_vp), _i, _i, _sz, _i, _i, _f, _i, _vp)


def check(code: int, where: str = "hylink") -> None:
    if code != 0:
        raise HylinkError(code, where)


def torch_dtype_code(dtype) -> int:
    import torch

    table = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
             torch.float64: 8, torch.bfloat16: 9}
    if hasattr(torch, "uint32"):
        table[torch.uint32] = 3
    if hasattr(torch, "uint64"):
        table[torch.uint64] = 5
    try:
        return table[dtype]
    except KeyError:
        raise TypeError(f"hylink: unsupported dtype {dtype}") from None
