// Schedule compiler: IR program -> address-free dependency graph.
//
// Every instruction becomes a node that runs as `nslices` pipelined slices.
// Slice k of a node may start once slice k of each node in `wait_for` is done.
// The dependencies come from a version walk over the whole program (all ranks,
// ascending rank id, program order inside a rank):
//   * a write creates the next version of its (space, owner, chunk) location;
//   * a read binds to the latest version at that point of the walk, or to the
//     FINAL version when nothing has been written yet (the writer is a rank
//     that appears later in the file);
//   * read-after-write: reader waits for the version's writer;
//   * write-after-read / write-after-write: the writer of version v+1 waits
//     for every reader of version v and for v's writer;
//   * D2DReduce reads its destination before writing it.
// In-place calls are handled by aliasing: output chunks are mapped onto the
// input chunks they share memory with before the walk, so the same rules order
// them; a schedule that would read user input after an aliased write is
// reported (the caller then stages the input).
//
// Parity: pcie-ccl-cuda/src/ir/compiler.cpp:124-619 keeps per-(space, owner,
// chunk, version) progress keys with reader ids, ring-buffer eligibility and
// overwrite guards. This design keeps the same ordering semantics with one
// progress counter per node, which is what the executor publishes across ranks.
#pragma once
#include <vector>

#include "ir/ir.h"

namespace hl {
namespace ir {

struct Loc {
  Buf space = Buf::Input;
  int owner = 0;  // rank for device spaces, NUMA node for Buf::Host
  int chunk = 0;
  bool operator<(const Loc& o) const {
    if (space != o.space) return space < o.space;
    if (owner != o.owner) return owner < o.owner;
    return chunk < o.chunk;
  }
  bool operator==(const Loc& o) const { return space == o.space && owner == o.owner && chunk == o.chunk; }
};

struct Node {
  int id = 0;
  int rank = 0;
  Op op = Op::NOP;
  Loc src, src2, dst;       // src2: second operand of H2HReduce
  bool skip = false;        // aliased self-copy: completes without work
  int line = 0;
  std::vector<int> wait_for;
  // Landing fusion (a property of the graph; an executor may ignore it). A D2DReduce whose source chunk was put
  // into device scratch by an H2D of the same rank, for that reduce alone, can read the pinned host chunk itself:
  // `fused_h2d` names that H2D node on the reduce, `fused_into` names the reduce on the H2D node.
  int fused_h2d = -1;
  int fused_into = -1;
  // Round guards. A message larger than the staging pools runs the same graph several times ("rounds") over the same
  // host, internal and scratch chunks. Before this node overwrites such a chunk in round w + 1, every node (of any
  // rank) that touched the chunk in round w must be through with it: these are those nodes. With them a round needs
  // no barrier at its end; only the chunks that are really reused wait for their last users.
  std::vector<int> round_guards;
};

enum class InPlace { None, Same, GatherSlot, ScatterSlot };

struct CompileOptions {
  int send_segs = 1;
  int recv_segs = 1;
  InPlace in_place = InPlace::None;  // Same: out==in; GatherSlot: in==out+rank*seg; ScatterSlot: out==in+rank*seg
  std::vector<int> gpu_numa;         // logical NUMA node of each rank (default NUMA of host chunks)
};

struct CompiledGraph {
  int nranks = 0;
  std::vector<Node> nodes;                 // global ids
  std::vector<std::vector<int>> by_rank;   // node ids of each rank, program order
  int input_chunks = 0, output_chunks = 0, internal_chunks = 0, scratch_chunks = 0, host_chunks = 0;
  int send_segs = 1, recv_segs = 1;
  int numa_nodes = 1;
  bool uses_remote_device = false;         // some node reads another rank's device buffer
  bool uses_host_reduce = false;
};

// hlUnsupported with "in-place conflict" in the message when staging is needed.
hlResult_t compile(const Program& p, const CompileOptions& opt, CompiledGraph* out);

// Per-call geometry shared by every rank (sizes only, no addresses).
struct Geometry {
  size_t elem = 4;
  size_t seg_count = 0;      // elements per segment (full, including the other path's prefix)
  size_t stride = 0;         // leading elements of every segment that are skipped
  size_t active = 0;         // elements of every segment handled by this call (after `stride`)
  size_t chunk_elems = 0;    // elements per device chunk (last chunk of a segment may be shorter)
  size_t chunk_bytes = 0;    // bytes of one internal / scratch / host chunk (256-byte multiple)
  size_t pitch_bytes = 0;    // distance between two such chunks in their pool (>= chunk_bytes; equal unless the caller sets it)
  size_t slice_bytes = 0;
  int nslices = 1;
  int cps_in = 1, cps_out = 1;
};
// `active` == 0 means "everything behind the stride".
hlResult_t makeGeometry(const CompiledGraph& g, size_t seg_count, size_t stride, size_t active, size_t elem, Geometry* out);
// Byte offset from the user buffer's base and byte length of device chunk c.
void deviceChunkSpan(const Geometry& geo, int cps, int c, size_t* offset, size_t* bytes);

}  // namespace ir
}  // namespace hl
