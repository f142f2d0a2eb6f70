"""The allocation-free all-reduce entry point (collected last on purpose).

Some callers may not allocate device memory when they need a reduction: their
memory is budgeted to the byte, their allocator is closed after start-up, or an
allocation would stall the device. ``hlAllReduceLocalNoAlloc`` serves them from
a fixed scratch array inside the library. Here it is called through its
exported C symbol, twice in a row, and compared with the regular emulated
group, which allocates its scratch with cudaMalloc.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, ins, outs, count, dtype_code, op=0):
    n = len(ins)
    a = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
    b = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    fn = lib.hlAllReduceLocalNoAlloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    return fn(n, a, b, count, dtype_code, op, C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_matches_the_allocating_entry_point_twice_in_a_row():
    from hylink_b200._native import lib, torch_dtype_code
    from hylink_b200.ops import EmuGroup

    torch.cuda.set_device(0)
    n = 4
    group = EmuGroup(n, stage_bytes=4 << 20)
    for round_, (dtype, count) in enumerate([(torch.bfloat16, 100003), (torch.float32, 65536)]):
        g = torch.Generator(device="cuda").manual_seed(17 + round_)
        ins = [(torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype) for _ in range(n)]
        want = [torch.empty_like(t) for t in ins]
        group.run("all_reduce", ins, want, count, algo="twoshot")
        got = [torch.full_like(t, 7) for t in ins]
        rc = _call(lib, ins, got, count, torch_dtype_code(dtype))
        assert rc == 0, lib.hlGetLastError().decode()
        torch.cuda.synchronize()
        for w, o in zip(want, got):
            torch.testing.assert_close(o, w, rtol=0, atol=0)
    group.close()


def test_rejects_what_does_not_fit():
    from hylink_b200._native import lib

    torch.cuda.set_device(0)
    big = [torch.zeros((256 << 10) // 4 + 1, device="cuda") for _ in range(2)]
    rc = _call(lib, big, big, big[0].numel(), 7)
    assert rc == 1 and b"exceed the fixed scratch" in lib.hlGetLastError()
    small = [torch.zeros(16, device="cuda") for _ in range(9)]
    rc = _call(lib, small, small, 16, 7)
    assert rc == 1 and b"supported range" in lib.hlGetLastError()
