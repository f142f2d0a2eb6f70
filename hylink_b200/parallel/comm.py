"""A communicator for callers that do not use ``torch.distributed``.

Wraps the ``hl*`` C API through ctypes. The unique id is exchanged by whatever
the caller has: pass ``store`` (any object with ``set``/``get`` — e.g. a
``torch.distributed.TCPStore``) or ``uid`` bytes directly.
"""
from __future__ import annotations

import ctypes as C

from .._native import CallOpts, CommStats, OPS, UniqueId, check, lib, torch_dtype_code

PATHS = {"auto": 0, "nvlink": 1, "pcie": 2, "split": 3}
ALGOS = {"auto": 0, "oneshot": 1, "twoshot": 2, "nvls": 3, "pipelined": 4, "push": 5, "zerocopy": 6, "zerocopy_nvls": 7,
         "zerocopy_p2p": 8, "ll": 9}


def unique_id() -> bytes:
    uid = UniqueId()
    check(lib.hlGetUniqueId(C.byref(uid)), "hlGetUniqueId")
    return bytes(uid.internal)


class Communicator:
    def __init__(self, rank: int, nranks: int, *, uid: bytes | None = None, store=None, device: int = -1,
                 key: str = "hylink/comm/uid"):
        if uid is None:
            if store is None:
                raise ValueError("need uid bytes or a store")
            if rank == 0:
                uid = unique_id()
                store.set(key, uid)
            else:
                uid = bytes(store.get(key))
        u = UniqueId()
        C.memmove(C.byref(u), uid.ljust(128, b"\0"), 128)
        self._h = C.c_void_p()
        self.rank, self.nranks = rank, nranks
        check(lib.hlCommInitRankDevice(C.byref(self._h), nranks, u, rank, device), "hlCommInitRankDevice")

    def close(self):
        if self._h:
            lib.hlCommDestroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------
    @staticmethod
    def _stream(t):
        if t.is_cuda:
            import torch

            return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
        return C.c_void_p(0)

    @staticmethod
    def _opts(path="auto", algo="auto", out_dtype=None, wire_dtype=None, scale=0.0, max_blocks=0, deterministic=False):
        o = CallOpts()
        o.path, o.algo = PATHS[path], ALGOS[algo]
        if out_dtype is not None:
            o.out_type, o.has_out_type = torch_dtype_code(out_dtype), 1
        if wire_dtype is not None:
            o.wire_type, o.has_wire_type = torch_dtype_code(wire_dtype), 1
        o.scale, o.max_blocks, o.deterministic = scale, max_blocks, int(deterministic)
        return o

    def all_reduce(self, send, recv=None, op="sum", **kw):
        recv = send if recv is None else recv
        o = self._opts(out_dtype=recv.dtype if recv.dtype != send.dtype else None, **kw)
        check(lib.hlAllReduceEx(send.data_ptr(), recv.data_ptr(), send.numel(), torch_dtype_code(send.dtype), OPS[op],
                                C.byref(o), self._h, self._stream(send)), "hlAllReduceEx")
        return recv

    def reduce_scatter(self, send, recv, op="sum", **kw):
        o = self._opts(**kw)
        check(lib.hlReduceScatterEx(send.data_ptr(), recv.data_ptr(), recv.numel(), torch_dtype_code(send.dtype),
                                    OPS[op], C.byref(o), self._h, self._stream(send)), "hlReduceScatterEx")
        return recv

    def all_gather(self, send, recv, **kw):
        o = self._opts(**kw)
        check(lib.hlAllGatherEx(send.data_ptr(), recv.data_ptr(), send.numel(), torch_dtype_code(send.dtype),
                                C.byref(o), self._h, self._stream(send)), "hlAllGatherEx")
        return recv

    def broadcast(self, buf, root=0, **kw):
        o = self._opts(**kw)
        check(lib.hlBroadcastEx(buf.data_ptr(), buf.data_ptr(), buf.numel(), torch_dtype_code(buf.dtype), root,
                                C.byref(o), self._h, self._stream(buf)), "hlBroadcastEx")
        return buf

    def all_to_all(self, send, recv, **kw):
        o = self._opts(**kw)
        check(lib.hlAllToAllEx(send.data_ptr(), recv.data_ptr(), send.numel() // self.nranks,
                               torch_dtype_code(send.dtype), C.byref(o), self._h, self._stream(send)), "hlAllToAllEx")
        return recv

    def alloc_registered(self, numel: int, dtype=None):
        """A tensor in the communicator's registered memory (see ``hlMemAlloc``): collectives on it run zero-copy.
        Collective in effect: every rank calls it in the same order with the same sizes."""
        import torch

        from ..ops.emu import _tensor_at

        dtype = dtype or torch.float32
        es = torch.empty((), dtype=dtype).element_size()
        p = C.c_void_p()
        check(lib.hlMemAlloc(self._h, numel * es, C.byref(p)), "hlMemAlloc")
        return _tensor_at(p.value, numel, dtype, _CommBlock(self, p.value))

    def is_registered(self, t) -> bool:
        lib.hlMemIsRegistered.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        return bool(lib.hlMemIsRegistered(self._h, C.c_void_p(t.data_ptr()), t.numel() * t.element_size()))

    def barrier(self, stream=None):
        import torch

        s = C.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else C.c_void_p(0)
        check(lib.hlBarrier(self._h, s), "hlBarrier")

    def drain(self):
        check(lib.hlCommDrain(self._h), "hlCommDrain")

    def stats(self) -> dict:
        st = CommStats()
        check(lib.hlCommGetStats(self._h, C.byref(st)), "hlCommGetStats")
        return {f[0]: getattr(st, f[0]) for f in CommStats._fields_}

    def async_error(self) -> int:
        e = C.c_int()
        check(lib.hlCommGetAsyncError(self._h, C.byref(e)), "hlCommGetAsyncError")
        return e.value

    def kernel_timeline(self):
        """Decoded kernel timeline (needs ``HYLINK_KERNEL_TIMELINE=1`` when the communicator is made)."""
        from ..utils.kernel_timeline import decode

        n = C.c_size_t(0)
        check(lib.hlCommKernelTimeline(self._h, None, C.byref(n)), "hlCommKernelTimeline")
        buf = (C.c_uint64 * n.value)()
        check(lib.hlCommKernelTimeline(self._h, buf, C.byref(n)), "hlCommKernelTimeline")
        return decode(list(buf))

    def dump_tuning(self) -> str:
        n = C.c_size_t(0)
        check(lib.hlCommDumpTuning(self._h, None, C.byref(n)), "hlCommDumpTuning")
        buf = C.create_string_buffer(n.value)
        check(lib.hlCommDumpTuning(self._h, buf, C.byref(n)), "hlCommDumpTuning")
        return buf.value.decode()

    def load_tuning(self, text: str):
        check(lib.hlCommLoadTuning(self._h, text.encode()), "hlCommLoadTuning")


class _CommBlock:
    def __init__(self, comm: Communicator, ptr):
        self.comm, self.ptr = comm, ptr

    def __del__(self):
        try:
            if self.comm._h:
                lib.hlMemFree(self.comm._h, C.c_void_p(self.ptr))
        except Exception:
            pass
