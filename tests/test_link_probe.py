"""The link probe's copy kernels on one GPU (a one-rank communicator copies inside its own staging region): the
thread-driven loop in both address layouts and the bulk-copy-engine ring must move exactly the bytes asked for."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comm():
    import os

    os.environ["HYLINK_SYMM_STAGE_BYTES"] = str(64 << 20)
    from hylink_b200._native import lib
    from hylink_b200.parallel.comm import Communicator, unique_id

    lib.hlConfigReload()
    torch.cuda.set_device(0)
    c = Communicator(0, 1, uid=unique_id(), device=0)
    yield c
    c.close()
    os.environ.pop("HYLINK_SYMM_STAGE_BYTES", None)
    lib.hlConfigReload()


def _roundtrip(comm, mode, blocks, threads_or_tile, unroll, layout, nbytes):
    from hylink_b200._native import check, lib

    half = lib.hlNvlStageBytes(comm._h) // 2 // 16 * 16
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8)
    guard = 4096
    zeros = torch.zeros(nbytes + guard, dtype=torch.uint8)
    check(lib.hlNvlStageAccess(comm._h, 1, 0, C.c_void_p(src.data_ptr()), nbytes), "write source")
    check(lib.hlNvlStageAccess(comm._h, 1, half, C.c_void_p(zeros.data_ptr()), nbytes + guard), "clear destination")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib.hlNvlLinkProbe(comm._h, mode, blocks, threads_or_tile, unroll, layout, nbytes, stream), "probe")
    torch.cuda.synchronize()
    got = torch.empty(nbytes + guard, dtype=torch.uint8)
    check(lib.hlNvlStageAccess(comm._h, 0, half, C.c_void_p(got.data_ptr()), nbytes + guard), "read destination")
    assert torch.equal(got[:nbytes], src), "copied bytes differ"
    assert int(got[nbytes:].sum()) == 0, "bytes behind the end were written"
    assert comm.async_error() == 0


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("threads,unroll", [(256, 4), (512, 8), (1024, 8), (512, 16)])
def test_thread_copy_moves_exactly_the_bytes(comm, layout, threads, unroll):
    _roundtrip(comm, 2, 37, threads, unroll, layout, (8 << 20) + 48)


@pytest.mark.parametrize("tile", [1024, 8192, 16384, 24576])
@pytest.mark.parametrize("blocks,nbytes", [(1, 64 << 10), (148, (8 << 20) + 4096 + 16), (300, 1 << 20), (8, 16)])
def test_bulk_engine_ring_moves_exactly_the_bytes(comm, tile, blocks, nbytes):
    _roundtrip(comm, 6, blocks, tile, 0, 0, nbytes)
