"""Orchestrator decision logic (no GPU): buckets, planner, the three feedback
algorithms, per-key isolation, tuning-table round trip, overlap metrics."""
import ctypes as C
import json

import pytest

from hylink_b200._native import lib

lib.hlSizeBucket.restype = C.c_int
lib.hlSizeBucket.argtypes = [C.c_size_t]
lib.hlPlanCreate.argtypes = [C.c_size_t, C.c_double, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t,
                             C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_int)]
lib.hlCtlCreate.restype = C.c_void_p
lib.hlCtlCreate.argtypes = [C.c_char_p, C.c_int]
lib.hlCtlDestroy.argtypes = [C.c_void_p]
lib.hlCtlSuggest.restype = C.c_double
lib.hlCtlSuggest.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int]
lib.hlCtlUpdate.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_double, C.c_double, C.c_size_t, C.c_size_t,
                            C.c_int, C.c_int]
lib.hlCtlUsePcie.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int]
lib.hlCtlDump.restype = C.c_size_t
lib.hlCtlDump.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
lib.hlCtlLoad.argtypes = [C.c_void_p, C.c_char_p]
lib.hlPathTiming.argtypes = [C.c_double] * 4 + [C.POINTER(C.c_double)]

MB = 1 << 20
AR, AG = 0, 1
BF16, F32 = 9, 7


def plan(total, alpha, allowed=1, elem=2, min_msg=0, min_part=0):
    f, p, u = C.c_size_t(), C.c_size_t(), C.c_int()
    lib.hlPlanCreate(total, alpha, allowed, elem, min_msg, min_part, C.byref(f), C.byref(p), C.byref(u))
    return f.value, p.value, bool(u.value)


class Ctl:
    def __init__(self, algo, n=8):
        self.h = lib.hlCtlCreate(algo.encode(), n)
        self.n = n

    def suggest(self, op=AR, nbytes=256 * MB, dt=BF16):
        return lib.hlCtlSuggest(self.h, op, nbytes, dt, self.n)

    def run(self, alpha, bf, bp, op=AR, nbytes=256 * MB, dt=BF16, fast_ok=1, pcie_ok=1):
        """One forked call on links of bf / bp bytes per second."""
        fb, pb, use = plan(nbytes, alpha, elem=2)
        lib.hlCtlUpdate(self.h, op, nbytes, dt, self.n, fb / bf, pb / bp if pb else 0.0, fb, pb, fast_ok, pcie_ok)

    def dump(self):
        n = lib.hlCtlDump(self.h, None, 0)
        b = C.create_string_buffer(n)
        lib.hlCtlDump(self.h, b, n)
        return b.value.decode()

    def __del__(self):
        lib.hlCtlDestroy(self.h)


def test_size_buckets_two_per_octave_from_4mib():
    assert lib.hlSizeBucket(4 * MB - 1) == -1
    assert lib.hlSizeBucket(4 * MB) == 0
    assert lib.hlSizeBucket(int(4 * MB * 2 ** 0.5) + 1) == 1
    assert lib.hlSizeBucket(8 * MB) == 2
    assert lib.hlSizeBucket(1 << 30) == 16


def test_planner_gates_and_alignment():
    assert plan(2 * MB, 0.3) == (2 * MB, 0, False)                 # below the minimum message
    assert plan(64 * MB, 0.0) == (64 * MB, 0, False)
    assert plan(64 * MB, 0.3, allowed=0) == (64 * MB, 0, False)
    f, p, use = plan(64 * MB + 6, 0.1, elem=2)
    assert use and f + p == 64 * MB + 6 and f % 128 == 0 and p % 2 == 0
    assert abs(p / (f + p) - 0.1) < 1e-3
    f, p, use = plan(64 * MB, 0.1, elem=12)                        # odd element size: the cut keeps elements whole
    assert use and f % 12 == 0 and f % 128 == 0
    assert plan(64 * MB, 1e-6) == (64 * MB, 0, False)              # PCIe part below the minimum part
    assert plan(64 * MB, 1.0) == (0, 64 * MB, True)


def test_split_ratio_finds_the_balance_point_and_follows_interference():
    c = Ctl("split_ratio")
    bf, bp = 700e9, 50e9
    for _ in range(40):
        c.run(c.suggest(), bf, bp)
    a = c.suggest()
    assert abs(a - bp / (bp + bf)) < 0.01, a
    for _ in range(40):                                            # PCIe interference: 75 % of the link is taken
        c.run(c.suggest(), bf, bp / 4)
    a2 = c.suggest()
    assert a2 < a / 2 and abs(a2 - (bp / 4) / (bp / 4 + bf)) < 0.01, a2
    for _ in range(40):                                            # and back
        c.run(c.suggest(), bf, bp)
    assert abs(c.suggest() - a) < 0.01


def test_tcp_hold_band_grow_and_halve():
    c = Ctl("tcp")
    a0 = c.suggest()
    assert abs(a0 - 0.01) < 1e-9
    bf, bp = 700e9, 50e9
    for _ in range(2):                                             # the first two samples are ignored
        c.run(a0, bf, bp)
    assert c.suggest() == a0
    c.run(a0, bf, bp)                                              # PCIe far too fast (rate >> 1.10): grow
    a1 = c.suggest()
    assert a1 > a0
    for _ in range(60):
        c.run(c.suggest(), bf, bp)
    a = c.suggest()
    fb, pb, _ = plan(256 * MB, a)
    rate = (fb / bf) / (pb / bp)
    assert 0.9 < rate < 1.15 and a <= 0.39                         # settled inside (or next to) the hold band
    c.run(a, bf, bp / 10)                                          # PCIe now much slower: halve
    assert abs(c.suggest() - a / 2) < 1e-6


def test_failure_shrinks_and_pcie_failure_latches_off():
    c = Ctl("split_ratio")
    a = c.suggest()
    c.run(a, 700e9, 50e9, fast_ok=0)
    assert abs(c.suggest() - a / 2) < 1e-9
    assert lib.hlCtlUsePcie(c.h, AR, 256 * MB, BF16, 8) == 1
    c.run(a, 700e9, 50e9, pcie_ok=0)
    assert lib.hlCtlUsePcie(c.h, AR, 256 * MB, BF16, 8) == 0
    assert c.suggest() == 0.0
    # other keys are untouched
    assert lib.hlCtlUsePcie(c.h, AG, 256 * MB, BF16, 8) == 1
    assert c.suggest(op=AG) > 0


def test_keys_are_isolated_by_op_bucket_and_dtype():
    c = Ctl("split_ratio")
    for _ in range(30):
        c.run(c.suggest(), 700e9, 50e9)
    tuned = c.suggest()
    fresh = Ctl("split_ratio").suggest()
    assert abs(tuned - fresh) > 0.005
    assert c.suggest(op=AG) == fresh
    assert c.suggest(nbytes=16 * MB) == fresh
    assert c.suggest(dt=F32) == fresh
    assert c.suggest(nbytes=300 * MB) == tuned                     # same bucket as 256 MiB


def test_static_keeps_alpha():
    c = Ctl("static")
    a = c.suggest()
    for _ in range(5):
        c.run(a, 700e9, 10e9)
    assert c.suggest() == a


def test_tuning_table_round_trip():
    c = Ctl("split_ratio")
    for _ in range(25):
        c.run(c.suggest(), 700e9, 50e9)
        c.run(c.suggest(op=AG, nbytes=32 * MB), 600e9, 40e9, op=AG, nbytes=32 * MB)
    text = c.dump()
    table = json.loads(text)
    assert len(table["entries"]) == 2
    d = Ctl("split_ratio")
    assert lib.hlCtlLoad(d.h, text.encode()) == 0
    assert abs(d.suggest() - c.suggest()) < 1e-6
    assert abs(d.suggest(op=AG, nbytes=32 * MB) - c.suggest(op=AG, nbytes=32 * MB)) < 1e-6
    assert lib.hlCtlLoad(d.h, b"not json") != 0


def test_path_timing_overlap():
    out = (C.c_double * 5)()
    lib.hlPathTiming(0.0, 1.0, 0.25, 1.5, out)
    fast, pcie, overlap, span, eff = list(out)
    assert (fast, pcie, overlap, span) == (1.0, 1.25, 0.75, 1.5)
    assert abs(eff - 2.25 / 3.0) < 1e-12
    lib.hlPathTiming(0.0, 1.0, 2.0, 3.0, out)                      # disjoint: no overlap
    assert out[2] == 0.0


def test_no_gain_guard_pauses_a_split_that_keeps_losing():
    c = Ctl("split_ratio")
    a = c.suggest()
    assert a > 0
    nbytes = 256 * MB
    for _ in range(16):  # PCIe half takes 3x as long as the whole message would take on the link alone
        fb, pb, _ = plan(nbytes, a)
        lib.hlCtlUpdate(c.h, AR, nbytes, BF16, 8, fb / 700e9, 3 * nbytes / 700e9, fb, pb, 1, 1)
    assert c.suggest() == 0.0 and lib.hlCtlUsePcie(c.h, AR, nbytes, BF16, 8) == 1   # paused, not latched off
    for _ in range(198):
        assert c.suggest() == 0.0
    c.suggest()
    assert c.suggest() > 0.0                                                       # probes again after the cool-down


def test_dma_lane_policy_table():
    """Lanes per direction by collective and size: many for bursts of short transfers, two for long messages,
    one for broadcast; the forced value and the lane limit win over the table."""
    import ctypes as C

    from hylink_b200._native import lib

    f = lib.hlDmaLaneCount
    f.restype = C.c_int
    f.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.c_int, C.c_int]
    mib = 1 << 20
    assert f(b"allreduce", 1 * mib, 8, 8, 0) == 4 and f(b"allreduce", 32 * mib, 8, 8, 0) == 3 and f(b"allreduce", 1024 * mib, 8, 8, 0) == 2
    assert f(b"allgather", 16 * mib, 4, 8, 0) == 4 and f(b"allgather", 17 * mib, 4, 8, 0) == 2
    assert f(b"reducescatter", 64 * mib, 4, 8, 0) == 3
    assert f(b"alltoall", 2 * mib, 8, 8, 0) == 8 and f(b"alltoall", 2 * mib, 4, 8, 0) == 4
    assert f(b"broadcast", 64 * mib, 8, 8, 0) == 1 and f(b"allreduce", 0, 8, 8, 0) == 1
    assert f(b"allreduce", 1 * mib, 8, 8, 6) == 6 and f(b"allreduce", 1 * mib, 8, 2, 0) == 2 and f(b"allreduce", 1 * mib, 8, 8, 99) == 8
