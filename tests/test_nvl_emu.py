"""Cross-rank NVLink-path kernels, all ranks emulated on one GPU.

Each case compares the sm_100a kernel against a plain PyTorch reference
computed in fp32/fp64 with the same (ascending-rank) summation order.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _group(n, **kw):
    from hylink_b200.ops import EmuGroup

    return EmuGroup(n, **kw)


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(dtype)
    return torch.randint(-50, 50, (n,), generator=g, device="cuda", dtype=torch.int64).to(dtype)


def _ordered_sum(ts, acc_dtype):
    acc = ts[0].to(acc_dtype).clone()
    for t in ts[1:]:
        acc = acc + t.to(acc_dtype)
    return acc


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
def test_allreduce_sum_bitwise(n, dtype, algo):
    g = _group(n, stage_bytes=8 << 20)
    for count in [1, 3, 15, 16, 17, 4095, 65536 + 5, 300000]:
        ins = [_rand(count, dtype, 100 * r + count % 97) for r in range(n)]
        outs = [torch.full((count + 8,), 7, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_reduce", ins, [o[:count] for o in outs], count, algo=algo)
        torch.cuda.synchronize()
        acc = torch.float64 if dtype == torch.float64 else (torch.float32 if dtype.is_floating_point else dtype)
        ref = _ordered_sum(ins, acc).to(dtype)
        for r in range(n):
            assert torch.equal(outs[r][:count], ref), (n, dtype, algo, count, r)
            assert torch.all(outs[r][count:] == 7), "wrote past the end"
        assert g.status(0)[0] == 0
    g.close()


@pytest.mark.parametrize("op", ["max", "min", "prod", "avg"])
def test_allreduce_ops(op):
    n, count = 4, 10007
    g = _group(n)
    ins = [_rand(count, torch.float32, 7 + r) for r in range(n)]
    outs = [torch.empty(count, device="cuda") for _ in range(n)]
    g.run("all_reduce", ins, outs, count, op=op, algo="twoshot")
    torch.cuda.synchronize()
    st = torch.stack(ins)
    ref = {"max": st.max(0).values, "min": st.min(0).values, "prod": st.prod(0), "avg": st.sum(0) / n}[op]
    for o in outs:
        torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-6)
    g.close()


def test_allreduce_inplace_unaligned_and_scale():
    n, count = 4, 33333
    g = _group(n)
    bufs = [_rand(count + 3, torch.bfloat16, r) for r in range(n)]
    views = [b[1:1 + count] for b in bufs]  # 2-byte offset: element-wise path
    ref = (_ordered_sum([v.clone() for v in views], torch.float32) * 0.25).to(torch.bfloat16)
    g.run("all_reduce", views, views, count, scale=0.25, algo="twoshot")
    torch.cuda.synchronize()
    for v in views:
        assert torch.equal(v, ref)
    g.close()


def test_allreduce_fused_cast():
    """fp32 gradients, bf16 on the wire, fp32 result: the cast rides inside the kernel."""
    n, count = 8, 70001
    g = _group(n)
    ins = [_rand(count, torch.float32, 31 + r) for r in range(n)]
    outs = [torch.empty(count, device="cuda") for _ in range(n)]
    g.run("all_reduce", ins, outs, count, wire_dtype=torch.bfloat16, algo="twoshot")
    torch.cuda.synchronize()
    ref = _ordered_sum([t.to(torch.bfloat16) for t in ins], torch.float32).to(torch.bfloat16).float()
    for o in outs:
        assert torch.equal(o, ref)
    # and the other direction: bf16 in, fp32 wire and result
    ins16 = [t.to(torch.bfloat16) for t in ins]
    g.run("all_reduce", ins16, outs, count, wire_dtype=torch.float32, algo="oneshot")
    torch.cuda.synchronize()
    ref = _ordered_sum(ins16, torch.float32)
    for o in outs:
        assert torch.equal(o, ref)
    g.close()


def test_allreduce_sliced_over_small_staging():
    """A message larger than the staging region is cut into several launches."""
    n, count = 4, (1 << 20) + 77
    g = _group(n, stage_bytes=1 << 20)
    ins = [_rand(count, torch.float32, r) for r in range(n)]
    outs = [torch.empty(count, device="cuda") for _ in range(n)]
    before = g.launches
    g.run("all_reduce", ins, outs, count, algo="twoshot")
    torch.cuda.synchronize()
    assert g.launches - before >= 4
    ref = _ordered_sum(ins, torch.float32)
    for o in outs:
        assert torch.equal(o, ref)
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter_strided_prefix(n, dtype):
    g = _group(n)
    seg, prefix = 5000, 3001  # only the first `prefix` elements of each segment are handled
    ins = [_rand(seg * n, dtype, 3 + r) for r in range(n)]
    outs = [torch.full((seg,), 9, dtype=dtype, device="cuda") for _ in range(n)]
    g.run("reduce_scatter", ins, outs, prefix, in_seg_stride=seg)
    torch.cuda.synchronize()
    for r in range(n):
        ref = _ordered_sum([t[r * seg:r * seg + prefix] for t in ins], torch.float32).to(dtype)
        assert torch.equal(outs[r][:prefix], ref)
        assert torch.all(outs[r][prefix:] == 9)
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_all_gather_strided_prefix(n):
    g = _group(n)
    seg, prefix = 4099, 2050
    ins = [_rand(seg, torch.float16, 11 + r) for r in range(n)]
    outs = [torch.full((seg * n,), 5, dtype=torch.float16, device="cuda") for _ in range(n)]
    g.run("all_gather", ins, outs, prefix, out_seg_stride=seg)
    torch.cuda.synchronize()
    for r in range(n):
        for q in range(n):
            assert torch.equal(outs[r][q * seg:q * seg + prefix], ins[q][:prefix])
            assert torch.all(outs[r][q * seg + prefix:(q + 1) * seg] == 5)
    g.close()


@pytest.mark.parametrize("n", [2, 4])
def test_all_to_all(n):
    g = _group(n)
    seg = 1237
    ins = [_rand(seg * n, torch.int32, 17 + r) for r in range(n)]
    outs = [torch.zeros(seg * n, dtype=torch.int32, device="cuda") for _ in range(n)]
    g.run("all_to_all", ins, outs, seg, in_seg_stride=seg, out_seg_stride=seg)
    torch.cuda.synchronize()
    for r in range(n):
        for q in range(n):
            assert torch.equal(outs[r][q * seg:(q + 1) * seg], ins[q][r * seg:(r + 1) * seg])
    g.close()


@pytest.mark.parametrize("root", [0, 3])
def test_broadcast(root):
    n, count = 4, 99991
    g = _group(n)
    bufs = [_rand(count, torch.float32, 23 + r) for r in range(n)]
    want = bufs[root].clone()
    g.run("broadcast", bufs, bufs, count, root=root)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b, want)
    g.close()


def test_back_to_back_calls_reuse_staging():
    """Mixed algorithms in sequence on one stream: the staging-reuse rules hold."""
    n, count = 4, 50000
    g = _group(n, stage_bytes=4 << 20)
    for it in range(6):
        ins = [_rand(count, torch.float32, it * 10 + r) for r in range(n)]
        outs = [torch.empty(count, device="cuda") for _ in range(n)]
        g.run("all_reduce", ins, outs, count, algo="oneshot" if it % 2 else "twoshot")
        outs2 = [torch.empty(count * n, device="cuda") for _ in range(n)]
        g.run("all_gather", outs, outs2, count, out_seg_stride=count)
        torch.cuda.synchronize()
        ref = _ordered_sum(ins, torch.float32)
        for o in outs2:
            assert torch.equal(o, ref.repeat(n))
    g.close()


def test_bounded_wait_reports_timeout_and_recovers():
    """A flag that nothing sets: the wait runs out, the kernel records a status
    and returns; the context stays usable and the group can be reset."""
    n, count = 2, 4096
    g = _group(n, timeout_ms=200)
    ins = [_rand(count, torch.float32, r) for r in range(n)]
    outs = [torch.zeros(count, device="cuda") for _ in range(n)]
    g.set_active_ranks(1)  # rank 1 never launches, so rank 0's barrier cannot complete
    g.run("all_reduce", ins, outs, count, algo="twoshot")
    torch.cuda.synchronize()  # returns: the wait was bounded
    code, step, peer, _ = g.status(0)
    assert code == 1 and step == 1 and peer == 1
    # a poisoned group turns later launches into no-ops instead of new waits
    g.run("all_reduce", ins, outs, count, algo="twoshot")
    torch.cuda.synchronize()
    g.set_active_ranks(n)
    g.reset()
    g.run("all_reduce", ins, outs, count, algo="twoshot")
    torch.cuda.synchronize()
    assert g.status(0)[0] == 0
    assert torch.equal(outs[0], ins[0] + ins[1]) and torch.equal(outs[1], outs[0])
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pipelined_allreduce_bitwise(n, dtype):
    """Warp-specialised tiles (copy-in / exchange / copy-out overlapped): same fixed-order sum."""
    g = _group(n, stage_bytes=64 << 20)
    for count in [5, 4097, 300001, (1 << 21) + 13]:
        ins = [_rand(count, dtype, 7 * r + count % 89) for r in range(n)]
        outs = [torch.full((count + 8,), 3, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_reduce", ins, [o[:count] for o in outs], count, algo="pipelined", scale=0.5)
        torch.cuda.synchronize()
        ref = (_ordered_sum(ins, torch.float32) * 0.5).to(dtype)
        for r in range(n):
            assert torch.equal(outs[r][:count], ref), (n, dtype, count, r)
            assert torch.all(outs[r][count:] == 3)
        assert g.status(0)[0] == 0
    g.close()


def test_pipelined_allreduce_in_place_sliced_and_mixed_with_classic_kernels():
    n, count = 4, (3 << 20) + 5
    g = _group(n, stage_bytes=8 << 20)  # forces several launches per call
    for it in range(3):
        bufs = [_rand(count, torch.float32, 31 * it + r) for r in range(n)]
        ref = _ordered_sum([b.clone() for b in bufs], torch.float32)
        g.run("all_reduce", bufs, bufs, count, algo="pipelined")
        small = [b[:1000].clone() for b in bufs]
        g.run("all_reduce", small, small, 1000, algo="oneshot")
        torch.cuda.synchronize()
        for b, s in zip(bufs, small):
            assert torch.equal(b, ref)
            assert torch.equal(s, ref[:1000] * n)
    g.close()


@pytest.mark.parametrize("n", [2, 8])
def test_pipelined_reduce_scatter_strided(n):
    g = _group(n, stage_bytes=64 << 20)
    seg, prefix = 400000, 333337
    ins = [_rand(seg * n, torch.bfloat16, 5 + r) for r in range(n)]
    outs = [torch.full((seg,), 9, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    g.run("reduce_scatter", ins, outs, prefix, in_seg_stride=seg, algo="pipelined")
    torch.cuda.synchronize()
    for r in range(n):
        ref = _ordered_sum([t[r * seg:r * seg + prefix] for t in ins], torch.float32).to(torch.bfloat16)
        assert torch.equal(outs[r][:prefix], ref)
        assert torch.all(outs[r][prefix:] == 9)
    g.close()


def test_pipelined_wait_is_bounded():
    n, count = 2, 1 << 20
    g = _group(n, timeout_ms=200)
    ins = [_rand(count, torch.float32, r) for r in range(n)]
    outs = [torch.zeros(count, device="cuda") for _ in range(n)]
    g.set_active_ranks(1)
    g.run("all_reduce", ins, outs, count, algo="pipelined")
    torch.cuda.synchronize()
    assert g.status(0)[0] == 1
    g.set_active_ranks(n)
    g.reset()
    g.run("all_reduce", ins, outs, count, algo="pipelined")
    torch.cuda.synchronize()
    assert torch.equal(outs[0], ins[0] + ins[1])
    g.close()


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_push_allreduce_bitwise(n, dtype):
    """Stores-only peer kernel: shards pushed to their owner, folded locally, results pushed back."""
    g = _group(n, stage_bytes=32 << 20)
    for count in [1, 17, 4099, 300001, (1 << 20) + 7]:
        ins = [_rand(count, dtype, 11 * r + count % 83) for r in range(n)]
        outs = [torch.full((count + 8,), 3, dtype=dtype, device="cuda") for _ in range(n)]
        g.run("all_reduce", ins, [o[:count] for o in outs], count, algo="push")
        torch.cuda.synchronize()
        acc = torch.float32 if dtype.is_floating_point else dtype
        ref = _ordered_sum(ins, acc).to(dtype)
        for r in range(n):
            assert torch.equal(outs[r][:count], ref), (n, dtype, count, r)
            assert torch.all(outs[r][count:] == 3)
    # in place, back to back, sliced over a small staging region
    g2 = _group(n, stage_bytes=2 << 20)
    for it in range(3):
        bufs = [_rand(700001, torch.float32, 5 * it + r) for r in range(n)]
        ref = _ordered_sum([b.clone() for b in bufs], torch.float32)
        g2.run("all_reduce", bufs, bufs, 700001, algo="push")
        torch.cuda.synchronize()
        for b in bufs:
            assert torch.equal(b, ref)
    g.close()
    g2.close()


def test_collectives_replay_from_a_cuda_graph():
    """The kernels keep their flag sequence in device memory, so a captured launch can be replayed."""
    n, count = 4, 200003
    g = _group(n, stage_bytes=16 << 20)
    ins = [_rand(count, torch.float32, r) for r in range(n)]
    outs = [torch.zeros(count, device="cuda") for _ in range(n)]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g.run("all_reduce", ins, outs, count, algo="push")  # first use outside the capture
        g.run("all_reduce", ins, outs, count, algo="pipelined")
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        g.run("all_reduce", ins, outs, count, algo="push")
        g.run("all_reduce", outs, outs, count, algo="pipelined", scale=1.0 / n)
    for it in range(3):
        for r in range(n):
            ins[r].copy_(_rand(count, torch.float32, 100 * it + r))
        ref = _ordered_sum(ins, torch.float32)
        ref = _ordered_sum([ref] * n, torch.float32) * (1.0 / n)
        graph.replay()
        torch.cuda.synchronize()
        for o in outs:
            assert torch.equal(o, ref), it
    # and eager calls still line up with the replays
    g.run("all_reduce", ins, outs, count, algo="twoshot")
    torch.cuda.synchronize()
    assert torch.equal(outs[0], _ordered_sum(ins, torch.float32))
    assert g.status(0)[0] == 0
    g.close()


def test_kernel_timeline_records_phases_in_order(monkeypatch):
    """With the timeline on, every CTA's stamps of a launch are monotonic: entry, barrier arrivals and releases, exit."""
    from hylink_b200.utils.kernel_timeline import summarise

    monkeypatch.setenv("HYLINK_KERNEL_TIMELINE", "1")
    g = _group(2, stage_bytes=16 << 20)
    try:
        n = 1 << 20
        ins = [torch.full((n,), float(r + 1), device="cuda", dtype=torch.bfloat16) for r in range(2)]
        outs = [torch.empty_like(t) for t in ins]
        for algo in ("push", "twoshot"):
            g.run("all_reduce", ins, outs, n, algo=algo)
        torch.cuda.synchronize()
        assert float(outs[1][-1]) == 3.0
        launches = g.kernel_timeline(0)
        assert [l["kind"] for l in launches[-2:]] == ["allreduce_push", "allreduce_twoshot"]
        for l in launches[-2:]:
            assert l["count"] == n and l["blocks"] >= 1
            for s in l["stamps"]:
                taken = [v for v in (s[0], s[1], s[2], s[3], s[4], s[7]) if v]
                assert len(taken) == 6 and taken == sorted(taken), s
            summary = summarise(l)
            assert summary["total_us"] > 0 and "entry->arrive1" in summary["phases"]
    finally:
        g.close()


@pytest.mark.parametrize("algo", ["auto", "twoshot", "pipelined"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_all_gather_kernels_agree(n, algo):
    """Stores-only (auto), staged pull (twoshot) and lane (pipelined) all-gather: odd prefix inside a wider segment,
    out of place and in place, several launches back to back, guard values behind every prefix."""
    g = _group(n, stage_bytes=32 << 20)
    seg, prefix = 300007, 262147
    ins = [_rand(seg, torch.bfloat16, 31 + r) for r in range(n)]
    outs = [torch.full((seg * n,), 7, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    for _ in range(3):
        g.run("all_gather", ins, outs, prefix, out_seg_stride=seg, algo=algo)
    torch.cuda.synchronize()
    for r in range(n):
        for q in range(n):
            assert torch.equal(outs[r][q * seg:q * seg + prefix], ins[q][:prefix]), (r, q)
            assert torch.all(outs[r][q * seg + prefix:(q + 1) * seg] == 7)
    # in place: every rank's input already sits in its own segment of its output
    bufs = [torch.full((seg * n,), 3, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    for r in range(n):
        bufs[r][r * seg:r * seg + prefix] = ins[r][:prefix]
    g.run("all_gather", [bufs[r][r * seg:] for r in range(n)], bufs, prefix, out_seg_stride=seg, algo=algo)
    torch.cuda.synchronize()
    for r in range(n):
        for q in range(n):
            assert torch.equal(bufs[r][q * seg:q * seg + prefix], ins[q][:prefix]), (r, q)
            assert torch.all(bufs[r][q * seg + prefix:(q + 1) * seg] == 3)
    assert g.status(0)[0] == 0
    g.close()
