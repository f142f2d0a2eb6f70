"""Landing-reduce kernel against PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
    return torch.randint(-100, 100, (n,), generator=g, device="cuda").to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32,
                                   torch.int64, torch.int8, torch.uint8])
@pytest.mark.parametrize("count", [1, 17, 4096, 100003])
def test_two_address_sum(dtype, count):
    from hylink_b200.ops import reduce_landing

    a, b = _rand(count, dtype, 1), _rand(count, dtype, 2)
    if dtype == torch.uint8:
        a, b = a.abs().to(dtype), b.abs().to(dtype)
    dst = a.clone()
    reduce_landing(dst, [b], accumulate=True)
    torch.cuda.synchronize()
    if dtype in (torch.bfloat16, torch.float16):
        ref = (a.float() + b.float()).to(dtype)
    else:
        ref = a + b
    assert torch.equal(dst, ref)


@pytest.mark.parametrize("op", ["sum", "max", "min"])
@pytest.mark.parametrize("k", [1, 3, 8])
def test_k_way_three_address(op, k):
    from hylink_b200.ops import reduce_landing

    count = 70001
    srcs = [_rand(count, torch.bfloat16, 10 + i) for i in range(k)]
    dst = torch.empty(count, dtype=torch.bfloat16, device="cuda")
    reduce_landing(dst, srcs, op=op, scale=0.5 if op == "sum" else 1.0)
    torch.cuda.synchronize()
    acc = srcs[0].float()
    for s in srcs[1:]:
        acc = {"sum": acc + s.float(), "max": torch.maximum(acc, s.float()), "min": torch.minimum(acc, s.float())}[op]
    if op == "sum":
        acc = acc * 0.5
    assert torch.equal(dst, acc.to(torch.bfloat16))


def test_pinned_host_source_and_unaligned():
    from hylink_b200.ops import reduce_landing

    count = 50001
    host = torch.randn(count + 1).pin_memory()
    dev = torch.randn(count + 1, device="cuda")
    dst = dev.clone()
    reduce_landing(dst[1:], [host[1:]], accumulate=True)  # 4-byte offset: element-wise path
    torch.cuda.synchronize()
    torch.testing.assert_close(dst[1:], dev[1:] + host[1:].cuda(), rtol=0, atol=0)
    dst2 = dev.clone()
    reduce_landing(dst2[:count], [host[:count]], accumulate=True)  # aligned: vector path over PCIe
    torch.cuda.synchronize()
    assert torch.equal(dst2[:count], dev[:count] + host[:count].cuda())
