"""A small single-GPU workload for profilers: each collective kernel once or twice.

    python -m hylink_b200.utils.profile_kernels [--ranks 4] [--mib 48]

Runs, on ONE device: the two-shot pull all-reduce, the push all-reduce, the
pipelined all-reduce, the push reduce-scatter, the all-gather, the zero-copy
kernels on registered memory (peer-pointer flavour) and the low-latency kernels with `--ranks`
emulated ranks (one cooperative launch each; `--mib` MiB of bf16 per rank, so
the working set is larger than the 126 MB L2 while staying within a few
hundred MB), and the landing-reduce kernel over four `--landing-mib` MiB sources. Prints the
CUDA-event time of every launch and the HBM traffic it implies. Meant to be run
plainly first and then under ``ncu -k regex:... -c N --clock-control none``.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--mib", type=int, default=48)
    ap.add_argument("--reps", type=int, default=2, help="timed launches after the warm-up launch (0: warm-up only)")
    ap.add_argument("--landing-mib", type=int, default=128)
    ap.add_argument("--no-zero-copy", action="store_true")
    a = ap.parse_args(argv)
    from hylink_b200.ops import EmuGroup, reduce_landing

    torch.cuda.set_device(0)
    n, count = a.ranks, a.mib * (1 << 20) // 2
    g = EmuGroup(n, stage_bytes=2 * a.mib << 20, timeout_ms=5000)
    ins = [torch.randn(count, device="cuda").to(torch.bfloat16) for _ in range(n)]
    outs = [torch.empty_like(t) for t in ins]
    seg = count // n
    gathered = [torch.empty(count, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    results = []

    def timed(name, fn, bytes_moved):
        fn()  # warm-up
        torch.cuda.synchronize()
        for _ in range(a.reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            results.append({"kernel": name, "ms": round(ms, 4), "hbm_GBs": round(bytes_moved / ms / 1e6, 1)})

    nb = count * 2
    # HBM bytes per launch, all emulated ranks together (reads + writes of every phase)
    timed("allreduce_twoshot_pull", lambda: g.run("all_reduce", ins, outs, count, algo="twoshot"), n * nb * (2 + 1 + 1.0 / n + 1 + 1))
    timed("allreduce_push", lambda: g.run("all_reduce", ins, outs, count, algo="push"), n * nb * (2.0 * (n - 1) / n + 1 + 2.0 / n + 2.0 * (n - 1) / n + 2.0 * (n - 1) / n))
    timed("allreduce_pipelined_push", lambda: g.run("all_reduce", ins, outs, count, algo="pipelined"), n * nb * (2.0 * (n - 1) / n + 1 + 2.0 / n + 2.0 * (n - 1) / n + 2.0 * (n - 1) / n))
    timed("reducescatter_push", lambda: g.run("reduce_scatter", ins, [o[:seg] for o in outs], seg, in_seg_stride=seg),
          n * nb * (2.0 * (n - 1) / n + 1 + 1.0 / n))
    timed("allgather_pull", lambda: g.run("all_gather", [t[:seg] for t in ins], gathered, seg, out_seg_stride=seg), n * (2 * seg * 2 + 2 * count * 2))
    # zero-copy kernels on registered memory (peer-pointer flavour; the switch flavour needs real peers)
    if not a.no_zero_copy:
        rin = g.alloc_registered(count, torch.bfloat16)
        rout = g.alloc_registered(count, torch.bfloat16)
        for t, src in zip(rin, ins):
            t.copy_(src)
        timed("allreduce_zerocopy_p2p", lambda: g.run("all_reduce", rin, rout, count, algo="zerocopy_p2p"), n * nb * (1 + 1))
        timed("reducescatter_zerocopy_p2p", lambda: g.run("reduce_scatter", rin, [o[:seg] for o in outs], seg, in_seg_stride=seg, algo="zerocopy_p2p"),
              n * nb * (1 + 1.0 / n))
        timed("allgather_zerocopy_p2p", lambda: g.run("all_gather", [t[:seg] for t in ins], rout, seg, out_seg_stride=seg, algo="zerocopy_p2p"),
              n * (seg * 2 + count * 2))
        del rin, rout
    # low-latency kernels (flag in every 16-byte store): small by design, 512 KiB per source
    lc = (512 << 10) // 2
    lins = [t[:lc * n] for t in ins]
    louts = [t[:lc * n] for t in outs]
    timed("allreduce_lowlatency", lambda: g.run("all_reduce", [t[:lc] for t in lins], [t[:lc] for t in louts], lc, algo="ll"), n * lc * 2 * (2 + 8.0 * (n - 1) / n))
    timed("reducescatter_lowlatency", lambda: g.run("reduce_scatter", lins, [t[:lc] for t in louts], lc, in_seg_stride=lc, algo="ll"),
          n * lc * 2 * (n + 4.0 * (n - 1) + 1))
    timed("allgather_lowlatency", lambda: g.run("all_gather", [t[:lc] for t in lins], louts, lc, out_seg_stride=lc, algo="ll"),
          n * lc * 2 * (1 + 4.0 * (n - 1) + n))
    srcs = [torch.randn(a.landing_mib << 19, device="cuda").to(torch.bfloat16) for _ in range(4)]
    dst = torch.empty_like(srcs[0])
    timed("reduce_landing_4way", lambda: reduce_landing(dst, srcs), 5 * srcs[0].numel() * 2)
    g.close()
    for r in results:
        print(json.dumps(r), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
