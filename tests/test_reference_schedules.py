"""The reference's own schedule files: every one must compile, and whole sets must run (no GPU).

The files are read where the reference keeps them (its two ``ir`` folders) or where its build was installed
(``baseline/_ref/ir``); without any of them the tests are skipped. Execution uses the host-memory device: real
processes, shared pools, the same executor and compiler as on a GPU, checked against an fp64 sum.
"""
import os
import re
from pathlib import Path

import pytest
import torch

from mp_util import run_ranks

ROOT = Path(__file__).resolve().parent.parent
DIRS = [d for d in (ROOT / "baseline" / "_ref" / "ir", Path("/root/reference/pcie-ccl-cuda/ir"), Path("/root/reference/pcie-ccl-ascend/ir"))
        if d.is_dir()]
FILES = sorted({d.parent.name + "/" + f.name: f for d in DIRS for f in d.glob("*.xml")}.items())
NAME = re.compile(r"^(allreduce|allgather|reducescatter|alltoall|broadcast_root(\d+))_(\d+)(?:_(\w+))?\.xml$")
SMALL_POOLS = {"HYLINK_HOST_BUFFER_SIZE": "96M", "HYLINK_INTERNAL_BUFFER_BYTES": "48M", "HYLINK_EXECUTOR_TIMEOUT_MS": "60000"}

pytestmark = pytest.mark.skipif(not FILES, reason="the reference's schedule files are not on this machine")


def _split(name):
    m = NAME.match(name)
    assert m, name
    coll = "broadcast" if m.group(1).startswith("broadcast") else m.group(1)
    return coll, int(m.group(2) or 0), m.group(3), m.group(4) or ""


@pytest.mark.parametrize("label,path", FILES, ids=[k for k, _ in FILES])
def test_every_reference_file_compiles(label, path):
    from hylink_b200.utils import schedule as S

    coll, _root, pattern, _variant = _split(path.name)
    ss, rs = S.segments(coll, len(pattern))
    info = S.inspect(path.read_text(), pattern, ss, rs)
    assert info["nranks"] == len(pattern) and info["instructions"] > 0
    if coll in ("allreduce", "alltoall") and _variant != "direct":
        # (a peer-read schedule run in place may be refused: a peer could read an input chunk that was overwritten)
        S.inspect(path.read_text(), pattern, ss, rs, in_place="same")


def _data(r, count, seed):
    g = torch.Generator().manual_seed(1000 * seed + r)
    return (torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1).float()


def _run_set_worker(rank, n, uid, files, seg):
    """Runs the reference's files for one pattern through hlSubmitIr (so exactly those files execute)."""
    import hylink_b200._native as N
    from hylink_b200.parallel.comm import Communicator

    c = Communicator(rank, n, uid=uid, device=-2)
    f32, SUM = 7, 0
    done = []
    for name, xml in files:
        coll, root, _pattern, _variant = _split(name)
        if coll == "allreduce":
            count = seg * n
            x, out = _data(rank, count, 1), torch.zeros(seg * n)
            N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), out.data_ptr(), count, 0, 1, 1, f32, SUM, None), name)
            c.drain()
            ref = sum(_data(r, count, 1).double() for r in range(n))
            assert torch.allclose(out.double(), ref, atol=1e-5), name
        elif coll == "reducescatter":
            x, out = _data(rank, seg * n, 2), torch.zeros(seg)
            N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), out.data_ptr(), seg, 0, n, 1, f32, SUM, None), name)
            c.drain()
            ref = sum(_data(r, seg * n, 2).double() for r in range(n))[rank * seg:(rank + 1) * seg]
            assert torch.allclose(out.double(), ref, atol=1e-5), name
        elif coll == "allgather":
            x, out = _data(rank, seg, 3), torch.zeros(seg * n)
            N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), out.data_ptr(), seg, 0, 1, n, f32, SUM, None), name)
            c.drain()
            assert torch.equal(out, torch.cat([_data(r, seg, 3) for r in range(n)])), name
        elif coll == "alltoall":
            x, out = _data(rank, seg * n, 4), torch.zeros(seg * n)
            N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), out.data_ptr(), seg, 0, n, n, f32, SUM, None), name)
            c.drain()
            assert torch.equal(out, torch.cat([_data(r, seg * n, 4)[rank * seg:(rank + 1) * seg] for r in range(n)])), name
        else:
            x = _data(rank, seg * n, 5)
            N.check(N.lib.hlSubmitIr(c._h, xml.encode(), x.data_ptr(), x.data_ptr(), seg * n, 0, 1, 1, f32, SUM, None), name)
            c.drain()
            assert torch.equal(x, _data(root, seg * n, 5)), name
        done.append(name)
    c.close()
    return len(done)


@pytest.mark.parametrize("pattern", ["00", "01", "0000", "0011", "00112233"])
def test_reference_sets_execute_on_the_host_device(pattern):
    """All host-relay files of one NUMA pattern (the `_direct` ones read peers' device memory, which the
    host-memory device serves only between threads of one process)."""
    seen, files = set(), []
    for _label, path in FILES:
        coll, _root, pat, variant = _split(path.name)
        text = path.read_text()
        if pat != pattern or variant == "direct" or (path.name, text) in seen:
            continue   # (the installed copy repeats the CUDA tree's files)
        seen.add((path.name, text))
        files.append((path.name, text))
    if not files:
        pytest.skip(f"no files for pattern {pattern}")
    n = len(pattern)
    env = dict(SMALL_POOLS, HYLINK_GPU_NUMA_MAP=",".join(pattern))
    res = run_ranks(_run_set_worker, n, files, 30011, env=env, timeout=300)
    assert res == [len(files)] * n
