"""The CPU-driven schedule executor on the host-memory device: real processes,
shared pinned-pool stand-ins, per-node progress counters in shared memory, the
NUMA worker pool and the host SIMD reduce — everything except the GPU."""
import ctypes as C

import pytest
import torch

from mp_util import run_ranks

SMALL_POOLS = {"HYLINK_HOST_BUFFER_SIZE": "64M", "HYLINK_INTERNAL_BUFFER_BYTES": "32M", "HYLINK_EXECUTOR_TIMEOUT_MS": "30000"}


def _comm(rank, n, uid):
    from hylink_b200.parallel.comm import Communicator

    return Communicator(rank, n, uid=uid, device=-2)


def _data(r, count, dtype, seed=0):
    g = torch.Generator().manual_seed(1000 * seed + r)
    return (torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1).to(dtype)


def _allreduce_worker(rank, n, uid, count, dtype_name, inplace):
    dtype = getattr(torch, dtype_name)
    c = _comm(rank, n, uid)
    x = _data(rank, count, dtype)
    out = x.clone() if inplace else torch.zeros(count, dtype=dtype)
    c.all_reduce(out if inplace else x, out)
    c.drain()
    ref = sum(_data(r, count, dtype).double() for r in range(n))
    tol = 1e-6 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.double(), ref, rtol=tol, atol=tol * n), (out[:4], ref[:4])
    st = c.stats()
    c.close()
    return st["pcie_bytes"]


@pytest.mark.parametrize("n", [2, 4])
def test_allreduce_4mib_fp32_against_fp64_oracle(n):
    """The CPU-only plumbing configuration: 4 MiB fp32 per rank, ring-free mesh schedule from the generator."""
    res = run_ranks(_allreduce_worker, n, 1 << 20, "float32", False, env=SMALL_POOLS)
    assert all(b == 4 << 20 for b in res)


def test_allreduce_bf16_in_place_odd_count():
    run_ranks(_allreduce_worker, 2, 100003, "bfloat16", True, env=SMALL_POOLS)


def test_allreduce_two_numa_nodes_host_reduce_variant():
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP="0011", HYLINK_IR_VARIANT="host_reduce")
    run_ranks(_allreduce_worker, 4, 50000, "float32", False, env=env)


def test_allreduce_rounds_when_message_exceeds_pools():
    env = dict(SMALL_POOLS, HYLINK_HOST_BUFFER_SIZE="4M", HYLINK_INTERNAL_BUFFER_BYTES="2M")
    run_ranks(_allreduce_worker, 2, 3 << 20, "float32", False, env=env)  # 12 MiB through 4 MiB pools


def _strided_worker(rank, n, uid):
    """Reduce-scatter / all-gather / all-to-all on the suffix of every segment (the multipath split)."""
    import hylink_b200._native as N

    c = _comm(rank, n, uid)
    seg, stride = 6000, 2500
    lib = N.lib
    f32, SUM = 7, 0
    # reduce-scatter: n input segments, output one segment; only [stride, seg) is touched
    x = torch.cat([_data(rank, seg, torch.float32, seed=q) for q in range(n)])
    out = torch.full((seg,), -7.0)
    from hylink_b200._native import check

    pccl = C.CDLL(None)
    check(lib.pcclReduceScatterStridedTyped(x.data_ptr(), out.data_ptr(), seg * n, stride, f32, SUM, c._h, None), "rs strided")
    c.drain()
    ref = sum(_data(r, seg, torch.float32, seed=rank).double() for r in range(n))
    assert torch.all(out[:stride] == -7.0)
    assert torch.allclose(out[stride:].double(), ref[stride:], atol=1e-5)
    # all-gather
    mine = _data(rank, seg, torch.float32, seed=50)
    full = torch.full((seg * n,), -3.0)
    check(lib.pcclAllGatherStridedTyped(mine.data_ptr(), full.data_ptr(), seg, stride, f32, c._h, None), "ag strided")
    c.drain()
    for q in range(n):
        assert torch.all(full[q * seg:q * seg + stride] == -3.0)
        assert torch.equal(full[q * seg + stride:(q + 1) * seg], _data(q, seg, torch.float32, seed=50)[stride:])
    # all-to-all
    a = torch.cat([_data(rank, seg, torch.float32, seed=70 + q) for q in range(n)])
    b = torch.full((seg * n,), -1.0)
    check(lib.pcclAllToAllStridedTyped(a.data_ptr(), b.data_ptr(), seg * n, stride, f32, c._h, None), "a2a strided")
    c.drain()
    for q in range(n):
        assert torch.all(b[q * seg:q * seg + stride] == -1.0)
        assert torch.equal(b[q * seg + stride:(q + 1) * seg], _data(q, seg, torch.float32, seed=70 + rank)[stride:])
    c.close()
    return True


@pytest.mark.parametrize("n", [2, 4])
def test_strided_collectives(n):
    run_ranks(_strided_worker, n, env=SMALL_POOLS)


def _misc_worker(rank, n, uid):
    c = _comm(rank, n, uid)
    # broadcast from the last rank
    t = _data(rank, 33333, torch.float32, seed=3)
    c.broadcast(t, root=n - 1)
    c.drain()
    assert torch.equal(t, _data(n - 1, 33333, torch.float32, seed=3))
    # in-place all-gather (send is the caller's slot of recv) and in-place reduce-scatter
    seg = 4097
    full = torch.zeros(seg * n)
    full[rank * seg:(rank + 1) * seg] = _data(rank, seg, torch.float32, seed=9)
    c.all_gather(full[rank * seg:(rank + 1) * seg], full)
    c.drain()
    for q in range(n):
        assert torch.equal(full[q * seg:(q + 1) * seg], _data(q, seg, torch.float32, seed=9))
    x = torch.cat([_data(rank, seg, torch.float32, seed=20 + q) for q in range(n)])
    ref = sum(_data(r, seg, torch.float32, seed=20 + rank).double() for r in range(n))
    c.reduce_scatter(x, x[rank * seg:(rank + 1) * seg])
    c.drain()
    assert torch.allclose(x[rank * seg:(rank + 1) * seg].double(), ref, atol=1e-5)
    # max / avg and integer types
    v = torch.full((1000,), float(rank + 1))
    c.all_reduce(v, op="max")
    c.drain()
    assert torch.all(v == n)
    v = torch.full((1000,), float(rank + 1))
    c.all_reduce(v, op="avg")
    c.drain()
    assert torch.allclose(v, torch.full((1000,), (n + 1) / 2))
    iv = torch.arange(777, dtype=torch.int64) + rank
    c.all_reduce(iv)
    c.drain()
    assert torch.equal(iv, torch.arange(777, dtype=torch.int64) * n + sum(range(n)))
    assert c.async_error() == 0
    c.close()
    return True


def test_broadcast_inplace_ops_and_integers():
    run_ranks(_misc_worker, 4, env=SMALL_POOLS)


def _custom_ir_worker(rank, n, uid, xml):
    import hylink_b200._native as N

    c = _comm(rank, n, uid)
    count = 20000
    x = _data(rank, count, torch.float32, seed=5)
    out = torch.zeros(count)
    N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), out.data_ptr(), count, 0, 1, 1, 7, 0, None), "hlSubmitIr")
    c.drain()
    ref = sum(_data(r, count, torch.float32, seed=5) for r in range(n))
    assert torch.allclose(out, ref, atol=1e-5)
    c.close()
    return True


def test_hand_written_schedule_runs():
    from test_ir import RELAY_AR

    run_ranks(_custom_ir_worker, 2, RELAY_AR, env=SMALL_POOLS)


def _dead_peer_worker(rank, n, uid):
    """Rank 1 leaves between collectives; rank 0's next collective must end with an error, not hang."""
    import time

    c = _comm(rank, n, uid)
    x = torch.ones(1000)
    c.all_reduce(x)
    c.drain()
    if rank == 1:
        import os

        os._exit(0)  # no goodbye: the peer has to notice on its own
    time.sleep(0.5)
    from hylink_b200 import HylinkError

    t0 = time.time()
    try:
        c.all_reduce(x)
        c.drain()
    except HylinkError as e:
        assert e.code in (6, 8), e  # timeout or remote error
        assert time.time() - t0 < 20
        return "detected"
    raise AssertionError("collective with a dead peer completed")


def test_dead_peer_is_detected():
    import multiprocessing as mp

    from hylink_b200.parallel.comm import unique_id
    from mp_util import _entry

    uid = unique_id().ljust(128, b"\0")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    env = dict(SMALL_POOLS, HYLINK_EXECUTOR_TIMEOUT_MS="3000", HYLINK_BARRIER_TIMEOUT_MS="3000", HYLINK_LOG_LEVEL="OFF")
    ps = [ctx.Process(target=_entry, args=(_dead_peer_worker, r, 2, uid, (), q, env)) for r in range(2)]
    for p in ps:
        p.start()
    r, status, val = q.get(timeout=60)
    for p in ps:
        p.join(20)
    assert (r, status, val) == (0, "ok", "detected"), val


def test_single_process_mode_threads_as_ranks_and_peer_device_reads():
    """Zeroed unique id: the ranks are threads of one process (the reference's SP mode). A schedule may then read a
    peer's device buffer directly (`src_rank`), which multi-process mode refuses."""
    import threading

    from hylink_b200._native import UniqueId, check, lib
    from hylink_b200.utils import schedule as S

    lib.hlConfigReload()
    n, count = 2, 30000
    # all-gather where every rank copies the peer's input straight out of the peer's buffer
    s = S.Schedule("allgather", n, topology="direct test", variant="direct")
    for r in range(n):
        s.d2d(r, 0, r)
        s.d2d(r, 0, 1 - r, src_rank=1 - r)
    xml = s.to_xml().encode()
    errors, outs = [], {}

    def run(rank):
        try:
            h = C.c_void_p()
            lib.pcclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
            check(lib.pcclCommInitRank(C.byref(h), n, UniqueId(), rank), "pcclCommInitRank")
            x = torch.full((count,), float(rank + 1))
            out = torch.zeros(count)
            lib.pcclAllReduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
            check(lib.pcclAllReduce(x.data_ptr(), out.data_ptr(), count, h, None), "pcclAllReduce")
            check(lib.hlCommDrain(h), "drain")
            assert torch.all(out == 3.0)
            g = torch.zeros(count * n)
            check(lib.hlSubmitIr(h, xml, x.data_ptr(), g.data_ptr(), count, 0, 1, n, 7, 0, None), "hlSubmitIr")
            check(lib.hlCommDrain(h), "drain")
            outs[rank] = g
            lib.pcclCommDestroy.argtypes = [C.c_void_p]
            check(lib.pcclCommDestroy(h), "destroy")
        except BaseException as e:  # noqa: BLE001
            errors.append((rank, repr(e)))

    import os

    os.environ.update(SMALL_POOLS)
    lib.hlConfigReload()
    ts = [threading.Thread(target=run, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(120)
    for k in SMALL_POOLS:
        os.environ.pop(k, None)
    lib.hlConfigReload()
    assert not errors, errors
    for r in range(n):
        assert torch.all(outs[r][:count] == 1.0) and torch.all(outs[r][count:] == 2.0)


def _refuse_peer_reads_worker(rank, n, uid):
    import hylink_b200._native as N
    from hylink_b200.utils import schedule as S

    c = _comm(rank, n, uid)
    s = S.Schedule("allgather", n)
    for r in range(n):
        s.d2d(r, 0, r)
        s.d2d(r, 0, 1 - r, src_rank=1 - r)
    x, g = torch.ones(100), torch.zeros(200)
    rc = N.lib.hlSubmitIr(c._h, s.to_xml().encode(), x.data_ptr(), g.data_ptr(), 100, 0, 1, n, 7, 0, None)
    msg = N.lib.hlGetLastError().decode()
    c.close()
    return rc, msg


def test_peer_device_reads_are_refused_between_processes():
    res = run_ranks(_refuse_peer_reads_worker, 2, env=SMALL_POOLS)
    for rc, msg in res:
        assert rc == 7 and "threads of one process" in msg, (rc, msg)  # hlUnsupported


def _eight_rank_worker(rank, n, uid):
    c = _comm(rank, n, uid)
    count = 80008
    x = _data(rank, count, torch.float32, seed=2)
    out = torch.zeros(count)
    c.all_reduce(x, out)
    c.drain()
    ref = sum(_data(r, count, torch.float32, seed=2).double() for r in range(n))
    assert torch.allclose(out.double(), ref, atol=1e-4)
    seg = 5000
    full = torch.zeros(seg * n)
    mine = _data(rank, seg, torch.float32, seed=4)  # the call is asynchronous: inputs must outlive it
    c.all_gather(mine, full)
    c.drain()
    for q in range(n):
        assert torch.equal(full[q * seg:(q + 1) * seg], _data(q, seg, torch.float32, seed=4))
    rs = torch.zeros(seg)
    parts = torch.cat([_data(rank, seg, torch.float32, seed=30 + q) for q in range(n)])
    c.reduce_scatter(parts, rs)
    c.drain()
    want = sum(_data(r, seg, torch.float32, seed=30 + rank).double() for r in range(n))
    assert torch.allclose(rs.double(), want, atol=1e-4)
    c.close()
    return True


def test_eight_ranks_two_numa_nodes():
    """The 8-GPU board layout (pattern 00001111): 72 host chunks per all-reduce, generated schedules."""
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP="00001111", HYLINK_HOST_BUFFER_SIZE="32M", HYLINK_H2H_WORKERS="1")
    run_ranks(_eight_rank_worker, 8, env=env, timeout=300)


def _many_rounds_worker(rank, n, uid):
    """Every collective through pools far smaller than the message: the rounds follow one another without a barrier,
    ordered only by the guards on the chunks they reuse."""
    c = _comm(rank, n, uid)
    count = 3 << 18                                   # 3 MiB of fp32 per segment
    for rep in range(2):
        x = _data(rank, count, torch.float32, seed=40 + rep)
        out = torch.zeros(count)
        c.all_reduce(x, out)
        seg = count // n
        part = torch.zeros(seg)
        c.reduce_scatter(x, part)
        full = torch.zeros(count)
        c.all_gather(x[:seg], full)
        a2a = torch.zeros(count)
        c.all_to_all(x, a2a)
        c.drain()
        ref = sum(_data(r, count, torch.float32, seed=40 + rep).double() for r in range(n))
        assert torch.allclose(out.double(), ref, atol=1e-5)
        assert torch.allclose(part.double(), ref[rank * seg:(rank + 1) * seg], atol=1e-5)
        assert torch.equal(full, torch.cat([_data(r, count, torch.float32, seed=40 + rep)[:seg] for r in range(n)]))
        assert torch.equal(a2a, torch.cat([_data(r, count, torch.float32, seed=40 + rep)[rank * seg:(rank + 1) * seg] for r in range(n)]))
    c.close()
    return True


@pytest.mark.parametrize("n,numa", [(2, "00"), (4, "0011")])
def test_rounds_without_a_barrier_between_them(n, numa):
    env = dict(SMALL_POOLS, HYLINK_HOST_BUFFER_SIZE="2M", HYLINK_INTERNAL_BUFFER_BYTES="1M", HYLINK_GPU_NUMA_MAP=numa)
    run_ranks(_many_rounds_worker, n, env=env, timeout=300)


def _range_job_worker(rank, n, uid, variant):
    c = _comm(rank, n, uid)
    count = 1 << 20                                      # 4 MiB of fp32: several slices per chunk
    x = _data(rank, count, torch.float32, seed=7)
    out = torch.zeros(count)
    c.all_reduce(x, out)
    seg = count // n
    full = torch.zeros(count)
    c.all_gather(x[:seg], full)
    c.drain()
    ref = sum(_data(r, count, torch.float32, seed=7).double() for r in range(n))
    assert torch.allclose(out.double(), ref, atol=1e-5)
    assert torch.equal(full, torch.cat([_data(r, count, torch.float32, seed=7)[:seg] for r in range(n)]))
    st = c.stats()
    c.close()
    return st["h2h_range_jobs"]


@pytest.mark.parametrize("workers", ["1", "3"])
def test_h2h_nodes_run_as_worker_owned_ranges(workers):
    """The host_reduce schedules fold on the CPU (H2HReduce chains): those nodes are handed to worker teams as whole
    nodes that follow their inputs slice by slice. One worker per pool is the hard case: the same worker must also
    run the plain copies the range waits for."""
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP="0011", HYLINK_H2H_WORKERS=workers, HYLINK_IR_VARIANT="host_reduce")
    jobs = run_ranks(_range_job_worker, 4, "host_reduce", env=env, timeout=300)
    assert all(j > 0 for j in (jobs.values() if isinstance(jobs, dict) else jobs))
    env["HYLINK_H2H_RANGE_JOBS"] = "0"
    jobs = run_ranks(_range_job_worker, 4, "host_reduce", env=env, timeout=300)
    assert all(j == 0 for j in (jobs.values() if isinstance(jobs, dict) else jobs))


def _composed_worker(rank, n, uid):
    c = _comm(rank, n, uid)
    count = n * 30001                                    # divisible by the rank count, odd segment length
    x = _data(rank, count, torch.float32, seed=11)
    out = torch.zeros(count)
    c.all_reduce(x, out, op="avg")
    inplace = x.clone()
    c.all_reduce(inplace, inplace)                       # in place: never composed
    odd = torch.zeros(count + 1)
    longer = torch.cat([x, x[:1]])                       # the call is asynchronous: inputs must outlive it
    c.all_reduce(longer, odd)                            # count not divisible: never composed
    c.drain()
    ref = sum(_data(r, count, torch.float32, seed=11).double() for r in range(n))
    assert torch.allclose(out.double(), ref / n, atol=1e-5)
    assert torch.allclose(inplace.double(), ref, atol=1e-5)
    assert torch.allclose(odd[:count].double(), ref, atol=1e-5)
    st = c.stats()
    c.close()
    return st["composed_allreduces"]


@pytest.mark.parametrize("n,numa", [(2, "00"), (4, "0011")])
def test_allreduce_composed_of_reduce_scatter_and_all_gather(n, numa):
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP=numa, HYLINK_PCIE_AR_COMPOSE="1")
    res = run_ranks(_composed_worker, n, env=env, timeout=300)
    assert all(v == 1 for v in (res.values() if isinstance(res, dict) else res))


@pytest.mark.parametrize("n,numa", [(2, "00"), (4, "0011")])
def test_allreduce_fp16(n, numa):
    """fp16 through every node type (the reference carries an unresolved fp16 hang repro, tests/dev/repro_fp16_allreduce.cpp)."""
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP=numa)
    run_ranks(_allreduce_worker, n, 3 << 18, "float16", False, env=env)
    run_ranks(_allreduce_worker, n, 100003, "float16", True, env=dict(env, HYLINK_IR_VARIANT="host_reduce"))


def _ring_worker(rank, n, uid):
    c = _comm(rank, n, uid)
    count = n * 400003                                   # several slices per chunk, odd segment length
    x = _data(rank, count, torch.float32, seed=21)
    out = torch.zeros(count)
    c.all_reduce(x, out)
    seg = count // n
    part = torch.zeros(seg)
    c.reduce_scatter(x, part)
    inplace = x.clone()
    c.all_reduce(inplace, inplace)
    c.drain()
    ref = sum(_data(r, count, torch.float32, seed=21).double() for r in range(n))
    assert torch.allclose(out.double(), ref, atol=1e-5)
    assert torch.allclose(part.double(), ref[rank * seg:(rank + 1) * seg], atol=1e-5)
    assert torch.allclose(inplace.double(), ref, atol=1e-5)
    st = c.stats()
    c.close()
    return st["h2h_range_jobs"]


@pytest.mark.parametrize("n,numa", [(2, "00"), (3, "001"), (4, "0011"), (8, "00112233")])
def test_ring_schedules_through_host_memory(n, numa):
    """The ring variant of the generator: a segment's partial sum travels around the ring through host memory and
    every rank folds its own contribution on the CPU (the plumbing configuration: fp32 sum, host-memory device)."""
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP=numa, HYLINK_IR_VARIANT="ring", HYLINK_H2H_WORKERS="2")
    jobs = run_ranks(_ring_worker, n, env=env, timeout=300)
    if n <= 4:   # with 8 ranks the 64 MiB test pools cut the message into rounds of single-slice chunks
        assert all(j > 0 for j in (jobs.values() if isinstance(jobs, dict) else jobs))  # the folds ran as worker-owned ranges
