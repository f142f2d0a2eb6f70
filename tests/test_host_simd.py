"""Host SIMD kernels of the PCIe path against PyTorch references (no GPU)."""
import ctypes as C
import os

import pytest
import torch

from hylink_b200._native import DTYPES, OPS, lib

TORCH = {"float32": torch.float32, "float64": torch.float64, "bfloat16": torch.bfloat16, "float16": torch.float16,
         "int32": torch.int32, "int64": torch.int64, "int8": torch.int8, "uint8": torch.uint8}


def _rand(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, dtype=torch.float64) * 4 - 2).to(dtype)
    lo, hi = (0, 100) if dtype == torch.uint8 else (-100, 100)
    return torch.randint(lo, hi, (n,), generator=g).to(dtype)


def _ref(a, b, op):
    wide = torch.float32 if a.dtype in (torch.bfloat16, torch.float16) else a.dtype
    x, y = a.to(wide), b.to(wide)
    r = {"sum": x + y, "prod": x * y, "max": torch.maximum(x, y), "min": torch.minimum(x, y)}[op]
    return r.to(a.dtype)


@pytest.mark.parametrize("dtype", list(TORCH))
@pytest.mark.parametrize("op", ["sum", "prod", "max", "min"])
def test_three_address_reduce_matches_reference_at_every_simd_level(dtype, op):
    best = lib.hlHostSimdLevel()
    for count in (1, 15, 16, 17, 63, 64, 1000, 65537):
        a, b = _rand(count, TORCH[dtype], 3), _rand(count, TORCH[dtype], 4)
        want = _ref(a, b, op)
        for level in range(best + 1):  # scalar, avx2, avx512 as far as this CPU goes
            out = torch.zeros_like(a)
            rc = lib.hlHostReduce(out.data_ptr(), a.data_ptr(), b.data_ptr(), count, DTYPES[dtype], OPS[op], level)
            assert rc == 0
            assert torch.equal(out.view(torch.uint8), want.view(torch.uint8)), (dtype, op, count, level)


def test_in_place_accumulate_and_unknown_type():
    a, b = _rand(4099, torch.float32, 1), _rand(4099, torch.float32, 2)
    want = a + b
    assert lib.hlHostReduce(a.data_ptr(), a.data_ptr(), b.data_ptr(), 4099, DTYPES["float32"], OPS["sum"], -1) == 0
    assert torch.equal(a, want)
    assert lib.hlHostReduce(a.data_ptr(), a.data_ptr(), b.data_ptr(), 4, 99, 0, -1) != 0


@pytest.mark.parametrize("nt", [0, 1])
def test_copy_any_alignment(nt):
    src = torch.arange(1 << 20, dtype=torch.uint8)
    for off_s, off_d, n in [(0, 0, 1 << 20), (1, 3, 70001), (7, 0, 4096), (0, 63, 999983)]:
        dst = torch.zeros((1 << 20) + 128, dtype=torch.uint8)
        lib.hlHostCopy(dst.data_ptr() + off_d, src.data_ptr() + off_s, n, nt)
        assert torch.equal(dst[off_d:off_d + n], src[off_s:off_s + n])
        assert dst[off_d + n:].sum() == 0 and dst[:off_d].sum() == 0


def test_host_micro_benchmark_runs_through_the_worker_pool():
    """`microbench h2h`: copy and reduce through the NUMA worker pool, one JSON line per configuration."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "hylink_b200.utils.microbench", "h2h", "--bytes", "4M", "--threads", "1,2",
                        "--iters", "2", "--dtype", "bf16"], cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, timeout=120, env=dict(os.environ, PYTHONPATH=root))
    assert p.returncode == 0, p.stdout[-2000:]
    rows = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert {(r["op"], r["threads"]) for r in rows} >= {("copy", 1), ("copy", 2), ("reduce", 1), ("reduce", 2)}
    assert all(r["GBs"] > 0 for r in rows)
