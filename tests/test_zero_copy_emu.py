"""Zero-copy kernels on registered memory, all ranks emulated on one GPU (peer-pointer flavour; the NVSwitch
flavour needs real peers and is covered by the multi-GPU tests).

Every rank's buffers come from the group's symmetric heap, so the kernels read the peers' inputs and write the
peers' outputs in place. Reference: plain PyTorch, fp32 accumulation in ascending rank order, one rounding.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _group(n, **kw):
    from hylink_b200.ops import EmuGroup

    return EmuGroup(n, **kw)


def _fill(ts, dtype, seed):
    for r, t in enumerate(ts):
        g = torch.Generator(device="cuda").manual_seed(seed * 977 + r)
        if dtype.is_floating_point:
            t.copy_((torch.rand(t.numel(), generator=g, device="cuda") * 2 - 1).to(dtype))
        else:
            t.copy_(torch.randint(-50, 50, (t.numel(),), generator=g, device="cuda").to(dtype))


def _ordered_sum(ts, dtype):
    acc_t = torch.float32 if dtype.is_floating_point and dtype != torch.float64 else dtype
    acc = ts[0].to(acc_t).clone()
    for t in ts[1:]:
        acc = acc + t.to(acc_t)
    return acc.to(dtype)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int32])
def test_allreduce_reads_and_writes_peers_in_place(n, dtype):
    g = _group(n, stage_bytes=1 << 20)
    es = torch.empty((), dtype=dtype).element_size()
    epp = 16 // es
    for count in [epp, 5 * epp, 4096 * epp + epp, (3 << 20) // es]:
        ins = g.alloc_registered(count, dtype)
        outs = g.alloc_registered(count + 2 * epp, dtype)     # guard packets on both sides
        _fill(ins, dtype, count)
        for o in outs:
            o.fill_(7)
        before = g.launches
        g.run("all_reduce", ins, [o[epp:epp + count] for o in outs], count, algo="zerocopy")
        torch.cuda.synchronize()
        assert g.launches == before + 1     # one launch whatever the size: nothing is staged
        ref = _ordered_sum(ins, dtype)
        for o in outs:
            assert torch.equal(o[epp:epp + count], ref), (n, dtype, count)
            assert bool((o[:epp] == 7).all()) and bool((o[epp + count:] == 7).all()), "wrote outside the buffer"
        assert g.status(0)[0] == 0
        # in place, with the average folded in
        if dtype.is_floating_point:
            want = (_ordered_sum(ins, torch.float32).float() if dtype == torch.float32 else None)
            acc = ins[0].float().clone()
            for t in ins[1:]:
                acc = acc + t.float()
            want = (acc * (1.0 / n)).to(dtype)
            g.run("all_reduce", ins, ins, count, op="avg", algo="zerocopy_p2p")
            torch.cuda.synchronize()
            for t in ins:
                assert torch.equal(t, want)
        del ins, outs
    g.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_reduce_scatter_all_gather_broadcast(n):
    g = _group(n)
    dtype = torch.bfloat16
    seg = 8 * 1031
    full = g.alloc_registered(seg * n, dtype)
    _fill(full, dtype, 3)
    outs = [torch.full((seg,), 5.0, device="cuda", dtype=dtype) for _ in range(n)]   # the output need not be registered
    g.run("reduce_scatter", full, outs, seg, in_seg_stride=seg, algo="zerocopy")
    torch.cuda.synchronize()
    ref = _ordered_sum(full, dtype)
    for r in range(n):
        assert torch.equal(outs[r], ref[r * seg:(r + 1) * seg])
    # all-gather: ordinary inputs, registered output, each rank's segment lands in every peer's buffer
    mine = [(torch.arange(seg, device="cuda") % 251 + r).to(dtype) for r in range(n)]
    gathered = g.alloc_registered(seg * n, dtype)
    for t in gathered:
        t.fill_(-1)
    g.run("all_gather", mine, gathered, seg, out_seg_stride=seg, algo="zerocopy")
    torch.cuda.synchronize()
    want = torch.cat(mine)
    for t in gathered:
        assert torch.equal(t, want)
    # in place: the input already sits in its segment of the output
    for r, t in enumerate(gathered):
        t.fill_(-1)
        t[r * seg:(r + 1) * seg] = mine[r]
    g.run("all_gather", [t[r * seg:(r + 1) * seg] for r, t in enumerate(gathered)], gathered, seg, out_seg_stride=seg, algo="zerocopy")
    torch.cuda.synchronize()
    for t in gathered:
        assert torch.equal(t, want)
    # broadcast from the last rank
    for r, t in enumerate(gathered):
        t.fill_(float(r))
    g.run("broadcast", gathered, gathered, seg * n, root=n - 1, algo="zerocopy")
    torch.cuda.synchronize()
    for t in gathered:
        assert bool((t == float(n - 1)).all())
    assert g.status(0)[0] == 0
    g.close()


def test_auto_uses_zero_copy_only_when_every_condition_holds():
    """Registered, aligned, whole packets: one launch and no staging. Anything else takes the staged kernels and
    still gives the same bits; asking for zero-copy by name is refused then."""
    from hylink_b200 import HylinkError

    n = 4
    g = _group(n, stage_bytes=256 << 10)        # staging far smaller than the message: staged calls need several launches
    dtype = torch.float32
    count = (8 << 20) // 4                      # above the sizes the barrier-free small-message kernels take
    ins = g.alloc_registered(count, dtype)
    outs = g.alloc_registered(count, dtype)
    _fill(ins, dtype, 11)
    ref = _ordered_sum(ins, dtype)
    before = g.launches
    g.run("all_reduce", ins, outs, count)      # auto
    torch.cuda.synchronize()
    assert g.launches == before + 1
    for o in outs:
        assert torch.equal(o, ref)
    # odd element count: not whole packets -> staged (sliced into several launches), same result
    before = g.launches
    g.run("all_reduce", [t[:count - 1] for t in ins], [o[:count - 1] for o in outs], count - 1)
    torch.cuda.synchronize()
    assert g.launches > before + 1
    for o in outs:
        assert torch.equal(o[:count - 1], ref[:count - 1])
    # unregistered output -> staged
    plain = [torch.empty(count, device="cuda") for _ in range(n)]
    before = g.launches
    g.run("all_reduce", ins, plain, count)
    torch.cuda.synchronize()
    assert g.launches > before + 1
    for o in plain:
        assert torch.equal(o, ref)
    with pytest.raises(HylinkError):
        g.run("all_reduce", ins, plain, count, algo="zerocopy")
    with pytest.raises(HylinkError):
        g.run("all_reduce", [t[1:] for t in ins], [o[1:] for o in outs], count - 1, algo="zerocopy")   # 4-byte offset
    g.close()


def test_heap_allocator_reuses_and_merges():
    g = _group(2)
    a = g.alloc_registered(1000)
    b = g.alloc_registered(1000)
    pa, pb = a[0].data_ptr(), b[0].data_ptr()
    assert pb > pa and (pb - pa) % 512 == 0
    assert a[1].data_ptr() != pa                # another rank's heap
    del a
    c = g.alloc_registered(500)                 # first fit: the hole at the front
    assert c[0].data_ptr() == pa
    del b, c
    d = g.alloc_registered(1 << 20)             # both holes merged with the rest
    assert d[0].data_ptr() == pa
    g.close()
