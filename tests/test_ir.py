"""Schedule IR: XML format, generator coverage and the compiler's ordering rules (no GPU)."""
import pytest

from hylink_b200.utils import schedule as S

# A two-rank all-reduce written by hand in the schedule format: one-step
# reduce-scatter and one-step all-gather through NUMA node 0.
RELAY_AR = """<?xml version="1.0" encoding="UTF-8"?>
<ir_program name="allreduce" nranks="2" topology="1numa_2gpu_per_numa" variant="relay_ring" nnodes="1">
  <description>hand-written test schedule &amp; comment</description>
  <!-- rank 0 owns chunk 0 -->
  <rank id="0">
    <instruction op="D2H" src_buf="input" src_chunk="1" dst_chunk="0" dst_numa="0"/>
    <instruction op="D2D" src_buf="input" src_chunk="0" dst_buf="internal" dst_chunk="0"/>
    <instruction op="H2D" src_chunk="1" src_numa="0" dst_buf="internal" dst_chunk="1"/>
    <instruction op="D2DReduce" src_buf="internal" src_chunk="1" dst_buf="internal" dst_chunk="0"/>
    <instruction op="D2H" src_buf="internal" src_chunk="0" dst_chunk="2" dst_numa="0"/>
    <instruction op="D2D" src_buf="internal" src_chunk="0" dst_buf="output" dst_chunk="0"/>
    <instruction op="H2D" src_chunk="3" src_numa="0" dst_buf="output" dst_chunk="1"/>
  </rank>
  <rank id="1">
    <instruction op="D2H" src_buf="input" src_chunk="0" dst_chunk="1" dst_numa="0"/>
    <instruction op="D2D" src_buf="input" src_chunk="1" dst_buf="internal" dst_chunk="1"/>
    <instruction op="H2D" src_chunk="0" src_numa="0" dst_buf="internal" dst_chunk="0"/>
    <instruction op="D2DReduce" src_buf="internal" src_chunk="0" dst_buf="internal" dst_chunk="1"/>
    <instruction op="D2H" src_buf="internal" src_chunk="1" dst_chunk="3" dst_numa="0"/>
    <instruction op="D2D" src_buf="internal" src_chunk="1" dst_buf="output" dst_chunk="1"/>
    <instruction op="H2D" src_chunk="2" src_numa="0" dst_buf="output" dst_chunk="0"/>
  </rank>
</ir_program>
"""


def test_parse_hand_written_schedule():
    info = S.inspect(RELAY_AR, "00")
    assert info["nranks"] == 2 and info["instructions"] == 14
    assert info["input_chunks"] == 2 and info["output_chunks"] == 2
    assert info["internal_chunks"] == 2 and info["host_chunks"] == 4
    assert info["dependency_edges"] >= 12  # every H2D waits for a D2H, every reduce for its operands ...
    # in place: the final H2D into output chunk 1 must wait for the D2H that read input chunk 1
    assert S.inspect(RELAY_AR, "00", in_place="same")["dependency_edges"] > info["dependency_edges"]


def test_round_trip_is_stable():
    once = S.round_trip(RELAY_AR)
    assert S.round_trip(once) == once
    assert S.inspect(once, "00") == S.inspect(RELAY_AR, "00")


@pytest.mark.parametrize("pattern", ["00", "01", "0000", "0011", "00112233", "00001111", "012", "0"])
@pytest.mark.parametrize("coll", S.COLLECTIVES)
def test_generator_covers_every_pattern(pattern, coll):
    n = len(pattern)
    ss, rs = S.segments(coll, n)
    variants = [""]
    if coll in ("allreduce", "reducescatter"):
        variants += ["host_reduce", "ring"]
    if coll in ("allgather", "alltoall"):
        variants.append("single_d2h")
    for v in variants:
        xml = S.generate(coll, pattern, v, root=n - 1)
        info = S.inspect(xml, pattern, ss, rs)
        assert info["nranks"] == n
        assert info["numa_nodes"] <= len(set(pattern))
        assert info["uses_host_reduce"] == (1 if (v in ("host_reduce", "ring") and n > 1) else 0)
        if coll in ("allreduce", "alltoall"):
            S.inspect(xml, pattern, ss, rs, in_place="same")
        if coll == "allgather":
            S.inspect(xml, pattern, ss, rs, in_place="gather_slot")
        if coll == "reducescatter" and v in ("", "ring"):
            S.inspect(xml, pattern, ss, rs, in_place="scatter_slot")


def test_builder_matches_format():
    s = S.Schedule("allgather", 2, topology="test")
    for r in range(2):
        s.d2h(r, 0, r, dst_numa=0).d2d(r, 0, r).h2d(r, 1 - r, 1 - r, src_numa=0)
    info = S.inspect(s.to_xml(), "00", 1, 2)
    assert info["instructions"] == 6 and info["host_chunks"] == 2 and info["output_chunks"] == 2


@pytest.mark.parametrize("bad,needle", [
    (RELAY_AR.replace('op="D2H" src_buf="input" src_chunk="1"', 'op="D2X" src_chunk="1"'), "unknown op"),
    (RELAY_AR.replace("</ir_program>", ""), "missing"),
    (RELAY_AR.replace('nranks="2"', 'nranks="0"'), "nranks"),
    (RELAY_AR.replace('<rank id="1">', '<rank id="7">'), "rank id"),
    ("<ir_program name='x' nranks='1'><rank id='0'><instruction op='H2D' src_chunk='0' dst_chunk='0'/></rank></ir_program>",
     "nothing writes"),
])
def test_malformed_schedules_are_rejected_with_a_reason(bad, needle):
    from hylink_b200 import HylinkError

    with pytest.raises(HylinkError) as e:
        S.inspect(bad, "00")
    assert needle in str(e.value)


def test_cycle_is_detected():
    from hylink_b200 import HylinkError

    # each rank's download waits for the other's upload, which in turn waits for that download's target
    s = S.Schedule("custom", 2)
    s.h2d(0, 0, 0, src_numa=0, dst_buf="internal").d2h(0, 0, 1, dst_numa=0, src_buf="internal")
    s.h2d(1, 1, 0, src_numa=0, dst_buf="internal").d2h(1, 0, 0, dst_numa=0, src_buf="internal")
    with pytest.raises(HylinkError) as e:
        S.inspect(s.to_xml(), "00")
    assert "cycle" in str(e.value)
