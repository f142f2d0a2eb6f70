"""Schedule DSL: build, generate, inspect and save PCIe-path schedules.

A schedule is the reference's XML "IR program": per rank, a list of copy /
reduce instructions over chunks of the user buffers, a device scratch buffer
and per-NUMA pinned host chunks. :class:`Schedule` builds one instruction by
instruction; :func:`generate` asks the library's generator for a complete
schedule for any GPU->NUMA pattern; :func:`inspect` compiles a schedule and
reports its size and dependency structure; ``python -m
hylink_b200.utils.schedule --emit DIR`` writes the standard set of files.

File naming follows the loader: ``<collective>_<pattern>[_<variant>].xml`` and
``broadcast_root<r>_<pattern>.xml``.
"""
from __future__ import annotations

import argparse
import ctypes as C
from pathlib import Path
from xml.sax.saxutils import escape

from .._native import IrInfo, check, lib

COLLECTIVES = ("allreduce", "allgather", "reducescatter", "alltoall", "broadcast")
STANDARD_PATTERNS = ("00", "01", "0000", "0011", "00112233", "00001111")
IN_PLACE = {"none": 0, "same": 1, "gather_slot": 2, "scatter_slot": 3}


class Schedule:
    """Instruction-by-instruction builder that serialises to the XML format."""

    def __init__(self, name: str, nranks: int, topology: str = "", variant: str = "", description: str = ""):
        self.name, self.nranks, self.topology, self.variant, self.description = name, nranks, topology, variant, description
        self.ranks: list[list[dict]] = [[] for _ in range(nranks)]

    def _add(self, rank: int, op: str, **attrs):
        self.ranks[rank].append({"op": op, **{k: v for k, v in attrs.items() if v is not None}})
        return self

    def d2h(self, rank, src_chunk, dst_chunk, dst_numa=None, src_buf=None, src_rank=None):
        return self._add(rank, "D2H", src_rank=src_rank, src_buf=src_buf, src_chunk=src_chunk, dst_chunk=dst_chunk, dst_numa=dst_numa)

    def h2d(self, rank, src_chunk, dst_chunk, src_numa=None, dst_buf=None):
        return self._add(rank, "H2D", src_chunk=src_chunk, src_numa=src_numa, dst_buf=dst_buf, dst_chunk=dst_chunk)

    def d2d(self, rank, src_chunk, dst_chunk, src_buf=None, dst_buf=None, src_rank=None):
        return self._add(rank, "D2D", src_rank=src_rank, src_buf=src_buf, dst_buf=dst_buf, src_chunk=src_chunk, dst_chunk=dst_chunk)

    def d2d_reduce(self, rank, src_chunk, dst_chunk, src_buf=None, dst_buf=None, src_rank=None):
        return self._add(rank, "D2DReduce", src_rank=src_rank, src_buf=src_buf, dst_buf=dst_buf, src_chunk=src_chunk, dst_chunk=dst_chunk)

    def h2h(self, rank, src_chunk, dst_chunk, src_numa=None, dst_numa=None):
        return self._add(rank, "H2H", src_chunk=src_chunk, src_numa=src_numa, dst_chunk=dst_chunk, dst_numa=dst_numa)

    def h2h_reduce(self, rank, src1_chunk, src2_chunk, dst_chunk, src1_numa=None, src2_numa=None, dst_numa=None):
        return self._add(rank, "H2HReduce", src1_chunk=src1_chunk, src1_numa=src1_numa, src2_chunk=src2_chunk,
                         src2_numa=src2_numa, dst_chunk=dst_chunk, dst_numa=dst_numa)

    def nop(self, rank):
        return self._add(rank, "NOP")

    def to_xml(self) -> str:
        head = f'<ir_program name="{self.name}" nranks="{self.nranks}" topology="{self.topology}"'
        if self.variant:
            head += f' variant="{self.variant}"'
        out = ['<?xml version="1.0" encoding="UTF-8"?>', head + ' nnodes="1">']
        if self.description:
            out.append(f"  <description>{escape(self.description)}</description>")
        for r, instrs in enumerate(self.ranks):
            out.append(f'  <rank id="{r}">')
            for ins in instrs:
                attrs = " ".join(f'{k}="{v}"' for k, v in ins.items())
                out.append(f"    <instruction {attrs}/>")
            out.append("  </rank>")
        out.append("</ir_program>")
        return "\n".join(out) + "\n"


def _sized(fn, *args) -> str:
    n = C.c_size_t(0)
    check(fn(*args, None, C.byref(n)), fn.__name__)
    buf = C.create_string_buffer(n.value)
    check(fn(*args, buf, C.byref(n)), fn.__name__)
    return buf.value.decode()


def generate(collective: str, pattern: str, variant: str = "", root: int = 0) -> str:
    """Schedule XML for ``collective`` on GPUs whose logical NUMA ids spell ``pattern``."""
    return _sized(lib.hlIrGenerate, collective.encode(), pattern.encode(), variant.encode(), root)


def round_trip(xml: str) -> str:
    return _sized(lib.hlIrRoundTrip, xml.encode())


def inspect(xml: str, pattern: str | None = None, send_segs: int = 1, recv_segs: int = 1, in_place: str = "none") -> dict:
    info = IrInfo()
    check(lib.hlIrInspect(xml.encode(), pattern.encode() if pattern else None, send_segs, recv_segs, IN_PLACE[in_place],
                          C.byref(info)), "hlIrInspect")
    return {f[0]: getattr(info, f[0]) for f in IrInfo._fields_}


def segments(collective: str, nranks: int) -> tuple[int, int]:
    """(send segments, receive segments) of a collective's buffers."""
    return {"allreduce": (1, 1), "broadcast": (1, 1), "allgather": (1, nranks), "reducescatter": (nranks, 1),
            "alltoall": (nranks, nranks)}[collective]


def emit_standard_set(directory: str | Path, patterns=STANDARD_PATTERNS) -> list[Path]:
    """Writes the standard schedule files (every collective, pattern and variant)."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    written = []
    for pat in patterns:
        n = len(pat)
        for coll in COLLECTIVES:
            if coll == "broadcast":
                for root in range(n):
                    p = d / f"broadcast_root{root}_{pat}.xml"
                    p.write_text(generate(coll, pat, "", root))
                    written.append(p)
                continue
            variants = [""]
            if coll in ("allgather", "alltoall") and len(set(pat)) > 1:
                variants.append("single_d2h")
            if coll in ("allreduce", "reducescatter"):
                variants += ["host_reduce", "ring"]
            for v in variants:
                p = d / (f"{coll}_{pat}" + (f"_{v}" if v else "") + ".xml")
                p.write_text(generate(coll, pat, v))
                written.append(p)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--emit", metavar="DIR", help="write the standard schedule set into DIR")
    ap.add_argument("--collective")
    ap.add_argument("--pattern")
    ap.add_argument("--variant", default="")
    ap.add_argument("--root", type=int, default=0)
    ap.add_argument("--inspect", metavar="FILE")
    a = ap.parse_args(argv)
    if a.emit:
        files = emit_standard_set(a.emit)
        print(f"wrote {len(files)} schedules to {a.emit}")
    if a.collective and a.pattern:
        print(generate(a.collective, a.pattern, a.variant, a.root))
    if a.inspect:
        xml = Path(a.inspect).read_text()
        print(inspect(xml))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
