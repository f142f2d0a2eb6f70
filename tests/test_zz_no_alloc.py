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

LIMIT = 256 << 10   # bytes per buffer (HL_NOALLOC_MAX_BYTES)
OPS = {"sum": 0, "avg": 4}


def _fn(lib):
    fn = lib.hlAllReduceLocalNoAlloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    return fn


def _call(lib, ins, outs, count, dtype_code, op=0):
    n = len(ins)
    a = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
    b = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    return _fn(lib)(n, a, b, count, dtype_code, op, C.c_void_p(torch.cuda.current_stream().cuda_stream))


def _status(lib):
    fn = lib.hlAllReduceLocalNoAllocStatus
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    code = C.c_int(-1)
    rc = fn(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(code))
    return rc, code.value


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
        assert _status(lib) == (0, 0)
    group.close()


@pytest.mark.parametrize("nbytes", [16, LIMIT - 2, LIMIT])
def test_rank_counts_and_the_size_limit(nbytes):
    """2, 3 and 8 buffers one after the other (another pointer-table row each time), up to the last byte that fits.
    With three buffers the shards do not divide evenly: the last one is short or empty."""
    from hylink_b200._native import lib, torch_dtype_code

    torch.cuda.set_device(0)
    count = nbytes // 2
    for n in (2, 3, 8, 3):
        g = torch.Generator(device="cuda").manual_seed(n * 1000 + nbytes)
        ins = [(torch.rand(count, generator=g, device="cuda") * 2 - 1).to(torch.bfloat16) for _ in range(n)]
        # guard bands: the outputs sit inside larger poison-filled buffers
        raw = [torch.full((count + 64,), 3.0, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
        outs = [t[32:32 + count] for t in raw]
        assert _call(lib, ins, outs, count, torch_dtype_code(torch.bfloat16)) == 0, lib.hlGetLastError().decode()
        torch.cuda.synchronize()
        acc = ins[0].float()
        for t in ins[1:]:
            acc = acc + t.float()   # ascending rank order, fp32, one rounding: what the kernel does
        want = acc.to(torch.bfloat16)
        for t, o in zip(raw, outs):
            torch.testing.assert_close(o, want, rtol=0, atol=0)
            assert bool((t[:32] == 3.0).all()) and bool((t[32 + count:] == 3.0).all())
        assert _status(lib) == (0, 0)


def test_in_place_average():
    from hylink_b200._native import lib, torch_dtype_code

    torch.cuda.set_device(0)
    n, count = 4, 4099
    bufs = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    assert _call(lib, bufs, bufs, count, torch_dtype_code(torch.float32), OPS["avg"]) == 0, lib.hlGetLastError().decode()
    torch.cuda.synchronize()
    for b in bufs:
        assert bool((b == 2.5).all())
    ints = [torch.full((count,), 4 * (r + 1), device="cuda", dtype=torch.int32) for r in range(n)]
    assert _call(lib, ints, ints, count, torch_dtype_code(torch.int32), OPS["avg"]) == 0, lib.hlGetLastError().decode()
    torch.cuda.synchronize()
    for b in ints:
        assert bool((b == 10).all())


def test_rejects_what_does_not_fit():
    from hylink_b200._native import lib

    torch.cuda.set_device(0)
    big = [torch.zeros((256 << 10) // 4 + 1, device="cuda") for _ in range(2)]
    rc = _call(lib, big, big, big[0].numel(), 7)
    assert rc == 1 and b"exceed the fixed scratch" in lib.hlGetLastError()
    # a count whose byte size wraps around in 64 bits must be refused too (nothing is launched)
    rc = _call(lib, big, big, 1 << 62, 7)
    assert rc == 1 and b"exceed the fixed scratch" in lib.hlGetLastError()
    small = [torch.zeros(16, device="cuda") for _ in range(9)]
    rc = _call(lib, small, small, 16, 7)
    assert rc == 1 and b"supported range" in lib.hlGetLastError()


def test_a_wait_that_runs_out_is_reported():
    """Only one of two grid rows is launched: its peer never signals, the bounded wait (2 s) runs out, the kernel
    returns by itself and the status call says so. The next call clears the state and works."""
    from hylink_b200._native import lib, torch_dtype_code

    torch.cuda.set_device(0)
    ins = [torch.ones(1024, device="cuda") for _ in range(2)]
    outs = [torch.zeros(1024, device="cuda") for _ in range(2)]
    lib.hlNoAllocSetActiveRowsForTest.argtypes = [C.c_int]
    lib.hlNoAllocSetActiveRowsForTest(1)
    try:
        assert _call(lib, ins, outs, 1024, torch_dtype_code(torch.float32)) == 0
        rc, code = _status(lib)
    finally:
        lib.hlNoAllocSetActiveRowsForTest(0)
    assert rc == 6 and code == 1 and b"gave up waiting" in lib.hlGetLastError()   # hlTimeout, HL_DEV_TIMEOUT
    assert _call(lib, ins, outs, 1024, torch_dtype_code(torch.float32)) == 0
    torch.cuda.synchronize()
    assert _status(lib) == (0, 0)
    assert bool((outs[0] == 2).all()) and bool((outs[1] == 2).all())
