"""Pair topology: NVML answers through a fake library, and the rule that selects the `_direct` schedule files (no GPU)."""
import ctypes as C
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE_NVML = r"""
#include <string.h>
#include <stdlib.h>
/* devices are their bus-id strings; "0000:0a:00.0" and "0000:0b:00.0" share a switch, "0000:c0:00.0" is elsewhere and
   has NVLink to everybody */
int nvmlInit_v2(void) { return 0; }
int nvmlShutdown(void) { return 0; }
int nvmlDeviceGetHandleByPciBusId_v2(const char* bus, void** dev) {
  if (strncmp(bus, "0000:", 5) != 0) return 2;
  *dev = strdup(bus);
  return 0;
}
int nvmlDeviceGetTopologyCommonAncestor(void* a, void* b, int* level) {
  const char *x = (const char*)a, *y = (const char*)b;
  *level = (x[5] == '0' && y[5] == '0') ? 10 : 50;   /* SINGLE under the first switch, SYSTEM otherwise */
  return 0;
}
int nvmlDeviceGetP2PStatus(void* a, void* b, int index, int* status) {
  const char *x = (const char*)a, *y = (const char*)b;
  *status = (index == 2 && (x[5] == 'c' || y[5] == 'c')) ? 0 : 5;
  return 0;
}
"""


def test_nvml_by_dlopen_and_the_direct_rule(tmp_path):
    src = tmp_path / "fake_nvml.c"
    src.write_text(FAKE_NVML)
    lib = tmp_path / "libfake_nvml.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-o", str(lib), str(src)])
    code = textwrap.dedent("""
        import ctypes as C
        from hylink_b200._native import lib
        q = lib.hlTopoPairQuery
        q.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        pix, nvl = C.c_int(-1), C.c_int(-1)
        assert q(b"0000:0a:00.0", b"0000:0b:00.0", C.byref(pix), C.byref(nvl)) == 1 and (pix.value, nvl.value) == (1, 0)
        assert q(b"0000:0a:00.0", b"0000:c0:00.0", C.byref(pix), C.byref(nvl)) == 1 and (pix.value, nvl.value) == (0, 1)
        assert q(b"bogus", b"0000:0b:00.0", C.byref(pix), C.byref(nvl)) == 0
        print("NVML_OK")
    """)
    env = dict(os.environ, PYTHONPATH=ROOT, HYLINK_NVML_LIB=str(lib))
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "NVML_OK" in p.stdout, p.stdout + p.stderr


def _allowed(coll, pattern, pix_pairs=(), nvlink_pairs=(), peer_pairs=()):
    from hylink_b200._native import lib

    n = len(pattern)

    def mat(pairs):
        m = (C.c_ubyte * (n * n))()
        for i, j in pairs:
            m[i * n + j] = m[j * n + i] = 1
        return m

    f = lib.hlTopoDirectAllowed
    f.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_ubyte), C.POINTER(C.c_ubyte), C.POINTER(C.c_ubyte), C.c_int]
    return bool(f(coll.encode(), pattern.encode(), mat(pix_pairs), mat(nvlink_pairs), mat(peer_pairs), n))


def test_direct_schedules_need_a_shared_switch_peer_access_and_no_nvlink():
    pairs = [(0, 1), (2, 3)]
    assert _allowed("allgather", "0011", pairs, (), pairs)
    assert _allowed("reducescatter", "0000", pairs, (), pairs)
    assert _allowed("allreduce", "00", [(0, 1)], (), [(0, 1)])
    assert not _allowed("allreduce", "0011", pairs, (), pairs)            # no direct all-reduce across two NUMA nodes
    assert not _allowed("allgather", "0011", pairs, [(0, 2)], pairs)       # NVLink anywhere: the other path's job
    assert not _allowed("allgather", "0011", [(0, 1)], (), pairs)          # second pair not under one switch
    assert not _allowed("allgather", "0011", pairs, (), [(0, 1)])          # second pair without peer access
    assert not _allowed("allgather", "00112233", pairs, (), pairs)         # no pair schedule for eight ranks
    assert not _allowed("alltoall", "0011", pairs, (), pairs)
    # broadcasts copy from the root: peer access inside the pairs (2, 4 ranks) or everywhere (8 ranks)
    assert _allowed("broadcast_root1", "0011", (), (), pairs)
    assert not _allowed("broadcast_root0", "00112233", (), (), pairs)
    assert _allowed("broadcast_root0", "00112233", (), (), [(i, j) for i in range(8) for j in range(i + 1, 8)])


def _scope_rank(comm_hash, n, rank, device, wait_ms, hold_s, q):
    import ctypes as C
    import time

    from hylink_b200._native import lib

    lib.hlNodeScopeDetect.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
    lib.hlNodeScopeLeave.argtypes = [C.c_uint64, C.c_int, C.c_int]
    flags = C.c_int(0)
    seen = lib.hlNodeScopeDetect(comm_hash, n, rank, device, wait_ms, C.byref(flags))
    q.put((rank, seen, flags.value))
    time.sleep(hold_s)          # the entry stays while the "communicator" lives
    lib.hlNodeScopeLeave(comm_hash, n, rank)


def _run_scope(n_present, n, devices, wait_ms=3000):
    import multiprocessing as mp
    import os

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    comm_hash = int.from_bytes(os.urandom(8), "little")
    ps = [ctx.Process(target=_scope_rank, args=(comm_hash, n, r, devices[r], wait_ms, 1.0, q)) for r in range(n_present)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=60) for _ in range(n_present))
    for p in ps:
        p.join(30)
    return res


def test_node_scope_sees_every_local_rank_and_misses_absent_ones():
    res = _run_scope(4, 4, [0, 1, 2, 3])
    assert all(seen == 4 and flags == 7 for _, seen, flags in res), res           # all here, distinct devices, in rank order
    res = _run_scope(4, 4, [3, 1, 2, 0])
    assert all(seen == 4 and flags == 3 for _, seen, flags in res), res           # all here and distinct, not in rank order
    res = _run_scope(2, 2, [0, 0])
    assert all(seen == 2 and flags & 1 and not flags & 2 for _, seen, flags in res), res   # two ranks on one device
    res = _run_scope(3, 4, [0, 1, 2, 3], wait_ms=400)                                 # the fourth rank lives on another machine
    assert all(seen == 3 and flags == 0 for _, seen, flags in res), res
