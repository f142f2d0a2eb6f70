"""N emulated ranks on ONE GPU.

Every NVLink-path kernel takes its peers as plain pointers, so the whole
cross-rank protocol (staging, per-block flag barriers, pull/push phases) can
run with all "ranks" resident on a single device. The ranks wait on one
another, so they are launched as one cooperative grid with one row per rank —
never as separate launches. This is how a one-GPU machine tests the multi-GPU
kernels; multicast (NVLS) variants need real peers and are not emulated.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .._native import OPS, check, lib, torch_dtype_code

KINDS = {"all_reduce": 0, "reduce_scatter": 1, "all_gather": 2, "broadcast": 3, "all_to_all": 4, "barrier": 5}
ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "pipelined": 4, "push": 5, "zerocopy": 6, "zerocopy_nvls": 7,
         "zerocopy_p2p": 8, "ll": 9}


class EmuGroup:
    def __init__(self, nranks: int, stage_bytes: int = 64 << 20, timeout_ms: int = 2000, device: int = 0):
        self.nranks = nranks
        self._h = C.c_void_p()
        check(lib.hlEmuCreate(nranks, device, stage_bytes, timeout_ms, C.byref(self._h)), "hlEmuCreate")

    def close(self):
        if self._h:
            lib.hlEmuDestroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ptrs(self, ts: Sequence[torch.Tensor] | None):
        arr = (C.c_void_p * self.nranks)()
        if ts is not None:
            for i, t in enumerate(ts):
                arr[i] = t.data_ptr() if t is not None else None
        return arr

    def run(self, kind: str, ins, outs, count: int, *, in_seg_stride: int = 0, out_seg_stride: int = 0,
            wire_dtype=None, op: str = "sum", scale: float = 1.0, root: int = 0, algo: str = "auto",
            max_blocks: int = 0):
        in_dt = torch_dtype_code(ins[0].dtype) if ins is not None else 7
        out_dt = torch_dtype_code(outs[0].dtype) if outs is not None else in_dt
        wire_dt = torch_dtype_code(wire_dtype) if wire_dtype is not None else in_dt
        stream = torch.cuda.current_stream().cuda_stream
        check(lib.hlEmuCollective(self._h, KINDS[kind], self._ptrs(ins), self._ptrs(outs), count, in_seg_stride,
                                  out_seg_stride, in_dt, out_dt, wire_dt, OPS[op], scale, root, ALGOS[algo],
                                  max_blocks, C.c_void_p(stream)), f"emu {kind}")

    def alloc_registered(self, numel: int, dtype=torch.float32):
        """One tensor per emulated rank in registered memory (the same heap offset on every rank)."""
        es = torch.empty((), dtype=dtype).element_size()
        ptrs = (C.c_void_p * self.nranks)()
        check(lib.hlEmuHeapAlloc(self._h, numel * es, ptrs), "hlEmuHeapAlloc")
        holder = _HeapBlock(self, ptrs[0])
        return [_tensor_at(ptrs[i], numel, dtype, holder) for i in range(self.nranks)]

    def kernel_timeline(self, i: int = 0):
        """Decoded kernel timeline of emulated rank ``i`` (needs ``HYLINK_KERNEL_TIMELINE=1`` when the group is made)."""
        from ..utils.kernel_timeline import decode

        n = C.c_size_t(0)
        check(lib.hlEmuKernelTimeline(self._h, i, None, C.byref(n)), "hlEmuKernelTimeline")
        buf = (C.c_uint64 * n.value)()
        check(lib.hlEmuKernelTimeline(self._h, i, buf, C.byref(n)), "hlEmuKernelTimeline")
        return decode(list(buf))

    def set_active_ranks(self, k: int):
        check(lib.hlEmuSetActiveRanks(self._h, k), "hlEmuSetActiveRanks")

    def status(self, i: int = 0):
        code, detail, block = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(lib.hlEmuStatus(self._h, i, C.byref(code), C.byref(detail), C.byref(block)), "hlEmuStatus")
        return code.value, detail.value >> 32, detail.value & 0xFFFFFFFF, block.value

    def reset(self):
        check(lib.hlEmuReset(self._h), "hlEmuReset")

    @property
    def launches(self) -> int:
        n = C.c_uint64()
        check(lib.hlEmuLaunches(self._h, C.byref(n)), "hlEmuLaunches")
        return n.value


class _HeapBlock:
    """Releases a registered allocation of the emulated group when its last tensor goes away."""

    def __init__(self, group: EmuGroup, ptr0):
        self.group, self.ptr0 = group, ptr0

    def __del__(self):
        try:
            if self.group._h:
                lib.hlEmuHeapFree(self.group._h, C.c_void_p(self.ptr0))
        except Exception:
            pass


class _Raw:
    """Just enough of the CUDA array interface for torch.as_tensor to wrap device memory it does not own."""

    def __init__(self, ptr, nbytes, holder):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
        self._holder = holder


def _tensor_at(ptr, numel, dtype, holder):
    es = torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_Raw(ptr, numel * es, holder), device="cuda")
    t = raw.view(dtype)
    if holder is not None:
        t._hl_holder = holder   # the view keeps the allocation alive
    return t
