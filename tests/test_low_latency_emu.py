"""Barrier-free small-message kernels (every 16-byte store carries its arrival flag), all ranks emulated on one GPU.

Reference: plain PyTorch, fp32 accumulation in ascending rank order, one rounding. The kernels promise that very
order, so results are compared bit for bit.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _group(n, **kw):
    from hylink_b200.ops import EmuGroup

    return EmuGroup(n, **kw)


def _inputs(n, count, dtype, seed):
    out = []
    for r in range(n):
        g = torch.Generator(device="cuda").manual_seed(seed * 131 + r)
        if dtype.is_floating_point:
            out.append((torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype))
        else:
            out.append(torch.randint(-50, 50, (count,), generator=g, device="cuda").to(dtype))
    return out


def _ordered_sum(ts, dtype, scale=1.0):
    acc_t = torch.float32 if dtype.is_floating_point and dtype != torch.float64 else dtype
    acc = ts[0].to(acc_t).clone()
    for t in ts[1:]:
        acc = acc + t.to(acc_t)
    if scale != 1.0:
        acc = acc * scale
    return acc.to(dtype)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int32])
def test_allreduce(n, dtype):
    g = _group(n, stage_bytes=1 << 20)
    es = torch.empty((), dtype=dtype).element_size()
    epp = 16 // es
    seed = 0
    # one packet, fewer packets than ranks, a ragged last shard, several sweeps of the grid
    for count in [epp, (n - 1) * epp, 4099 * epp, (1 << 20) // es]:
        for rep in range(3):                             # consecutive calls alternate the two halves of the region
            seed += 1
            ins = _inputs(n, count, dtype, seed)
            outs = [torch.full((count + 2 * epp,), 7, dtype=dtype, device="cuda") for _ in range(n)]
            before = g.launches
            g.run("all_reduce", ins, [o[epp:epp + count] for o in outs], count, algo="ll")
            torch.cuda.synchronize()
            assert g.launches == before + 1
            ref = _ordered_sum(ins, dtype)
            for o in outs:
                assert torch.equal(o[epp:epp + count], ref), (n, dtype, count, rep)
                assert bool((o[:epp] == 7).all()) and bool((o[epp + count:] == 7).all()), "wrote outside the buffer"
            assert g.status(0)[0] == 0
        if dtype.is_floating_point:                      # in place, with the average folded in
            ins = _inputs(n, count, dtype, seed + 1000)
            want = _ordered_sum(ins, dtype, 1.0 / n)
            g.run("all_reduce", ins, ins, count, op="avg", algo="ll")
            torch.cuda.synchronize()
            for t in ins:
                assert torch.equal(t, want)
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_reduce_scatter_and_all_gather(n, dtype):
    g = _group(n, stage_bytes=1 << 20)
    es = torch.empty((), dtype=dtype).element_size()
    epp = 16 // es
    for seg in [epp, 777 * epp, (256 << 10) // es]:
        full = _inputs(n, seg * n, dtype, seg)
        want = _ordered_sum(full, dtype)
        # reduce-scatter, out of place
        outs = [torch.zeros(seg, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("reduce_scatter", full, outs, seg, in_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r, o in enumerate(outs):
            assert torch.equal(o, want[r * seg:(r + 1) * seg]), (n, seg, r)
        # reduce-scatter into the own slot of the input
        work = [t.clone() for t in full]
        g.run("reduce_scatter", work, [t[r * seg:(r + 1) * seg] for r, t in enumerate(work)], seg, in_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r, t in enumerate(work):
            assert torch.equal(t[r * seg:(r + 1) * seg], want[r * seg:(r + 1) * seg])
        # all-gather, out of place and from the own slot of the output
        mine = [t[:seg].contiguous() for t in full]
        gathered = [torch.zeros(seg * n, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_gather", mine, gathered, seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        ref = torch.cat(mine)
        for t in gathered:
            assert torch.equal(t, ref)
        for r, t in enumerate(gathered):
            t.zero_()
            t[r * seg:(r + 1) * seg].copy_(mine[r])
        g.run("all_gather", [t[r * seg:(r + 1) * seg] for r, t in enumerate(gathered)], gathered, seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for t in gathered:
            assert torch.equal(t, ref)
        assert g.status(0)[0] == 0
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_all_to_all(n):
    g = _group(n, stage_bytes=1 << 20)
    dtype = torch.float32
    for seg in [4, 777 * 4, (128 << 10) // 4]:
        ins = _inputs(n, seg * n, dtype, seg + 5)
        outs = [torch.zeros(seg * n, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_to_all", ins, outs, seg, in_seg_stride=seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r in range(n):
            want = torch.cat([ins[s][r * seg:(r + 1) * seg] for s in range(n)])
            assert torch.equal(outs[r], want), (n, seg, r)
        work = [t.clone() for t in ins]                  # in place
        g.run("all_to_all", work, work, seg, in_seg_stride=seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r in range(n):
            assert torch.equal(work[r], torch.cat([ins[s][r * seg:(r + 1) * seg] for s in range(n)]))
        assert g.status(0)[0] == 0
    g.close()


def test_auto_takes_the_low_latency_kernels_for_small_messages_and_mixes_with_the_others(monkeypatch):
    """Small calls, large calls (barrier kernels) and small calls again: the region's halves stay consistent."""
    monkeypatch.setenv("HYLINK_KERNEL_TIMELINE", "1")
    n, dtype = 4, torch.bfloat16
    g = _group(n, stage_bytes=8 << 20)
    small, large = 64 << 10, 6 << 20                      # elements: 128 KiB and 12 MiB
    for rep in range(4):
        for count in (small, large, small, small):
            ins = _inputs(n, count, dtype, rep * 10 + count % 7)
            outs = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(n)]
            g.run("all_reduce", ins, outs, count)
            torch.cuda.synchronize()
            if count == small:
                assert g.kernel_timeline()[-1]["kind"] == "lowlatency_allreduce"
                ref = _ordered_sum(ins, dtype)
                for o in outs:
                    assert torch.equal(o, ref)
            else:
                assert g.kernel_timeline()[-1]["kind"] != "lowlatency_allreduce"
                ref = torch.stack([t.float() for t in ins]).sum(0)
                for o in outs:
                    assert torch.allclose(o.float(), ref, rtol=2e-2, atol=2e-2)
    assert g.status(0)[0] == 0
    g.close()


def test_named_request_is_refused_when_the_call_does_not_qualify():
    g = _group(2, stage_bytes=1 << 20)
    big = [torch.ones(8 << 20, dtype=torch.float32, device="cuda") for _ in range(2)]  # 32 MiB: no slot holds it
    with pytest.raises(RuntimeError):
        g.run("all_reduce", big, [torch.empty_like(t) for t in big], 8 << 20, algo="ll")
    with pytest.raises(RuntimeError):                                                  # no type conversion
        g.run("all_reduce", [t[:4096] for t in big], [torch.empty(4096, dtype=torch.bfloat16, device="cuda") for _ in range(2)], 4096, algo="ll")
    g.close()


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_any_alignment_and_any_count(n, dtype):
    """Which kernel a call takes must not depend on a pointer (ranks need not agree on those): views that start in
    the middle of a packet and counts that end in one go through the same kernels."""
    g = _group(n, stage_bytes=1 << 20)
    es = torch.empty((), dtype=dtype).element_size()
    epp = 16 // es
    for count, off_in, off_out in [(1, 0, 0), (epp + 1, 1, 0), (1001, 0, 3), (4099 * epp + 5, 1, 1)]:
        base = _inputs(n, count + off_in, dtype, count)
        ins = [t[off_in:] for t in base]
        outs = [torch.full((count + off_out + epp,), 7, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_reduce", ins, [o[off_out:off_out + count] for o in outs], count, algo="ll")
        torch.cuda.synchronize()
        ref = _ordered_sum(ins, dtype)
        for o in outs:
            assert torch.equal(o[off_out:off_out + count], ref), (n, dtype, count, off_in, off_out)
            assert bool((o[:off_out] == 7).all()) and bool((o[off_out + count:] == 7).all()), "wrote outside the buffer"
        # reduce-scatter and all-gather with segments that are neither aligned nor whole packets
        seg = count
        full = _inputs(n, seg * n + off_in, dtype, count + 1)
        fin = [t[off_in:] for t in full]
        want = _ordered_sum(fin, dtype)
        parts = [torch.full((seg + off_out + epp,), 7, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("reduce_scatter", fin, [p[off_out:off_out + seg] for p in parts], seg, in_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r, p in enumerate(parts):
            assert torch.equal(p[off_out:off_out + seg], want[r * seg:(r + 1) * seg]), (n, dtype, seg, r)
            assert bool((p[off_out + seg:] == 7).all())
        gathered = [torch.full((seg * n + off_out + epp,), 7, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_gather", [t[:seg] for t in fin], [t[off_out:off_out + seg * n] for t in gathered], seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        refg = torch.cat([t[:seg] for t in fin])
        for t in gathered:
            assert torch.equal(t[off_out:off_out + seg * n], refg)
            assert bool((t[off_out + seg * n:] == 7).all())
        a2a = [torch.full((seg * n + off_out + epp,), 7, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_to_all", fin, [t[off_out:off_out + seg * n] for t in a2a], seg, in_seg_stride=seg, out_seg_stride=seg, algo="ll")
        torch.cuda.synchronize()
        for r, t in enumerate(a2a):
            assert torch.equal(t[off_out:off_out + seg * n], torch.cat([fin[s][r * seg:(r + 1) * seg] for s in range(n)]))
        assert g.status(0)[0] == 0
    g.close()


def test_missing_rank_runs_into_the_bounded_wait():
    """One row of the launch is left out: its packets never arrive, the others give up after the limit and report it."""
    n = 4
    g = _group(n, stage_bytes=1 << 20, timeout_ms=200)
    count = 4096
    ins = _inputs(n, count, torch.float32, 3)
    outs = [torch.empty_like(t) for t in ins]
    g.set_active_ranks(n - 1)
    g.run("all_reduce", ins, outs, count, algo="ll")
    torch.cuda.synchronize()                                           # returns: the wait was bounded
    code, step, peer, _ = g.status(0)
    assert code == 1 and step == 8 and peer == n - 1, (code, step, peer)   # a low-latency packet that never arrived
    g.set_active_ranks(n)
    g.reset()
    g.run("all_reduce", ins, outs, count, algo="ll")
    torch.cuda.synchronize()
    assert torch.equal(outs[0], _ordered_sum(ins, torch.float32))
    g.close()
