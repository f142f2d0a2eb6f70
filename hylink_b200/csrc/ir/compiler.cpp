#include "ir/compiler.h"

#include <algorithm>
#include <map>
#include <set>

namespace hl {
namespace ir {

namespace {

struct LocState {
  int version = 0;                              // latest version produced so far in the walk
  std::vector<int> writer;                      // writer[v] = node id (index 0 unused)
  std::vector<std::vector<int>> readers;        // readers[v] = node ids
  std::vector<int> pending;                     // nodes that read before any write: bind to the final version
};

struct Walker {
  const Program& p;
  const CompileOptions& opt;
  CompiledGraph& g;
  std::map<Loc, LocState> st;
  std::string conflict;
  int cps_in = 1, cps_out = 1;

  Walker(const Program& pp, const CompileOptions& o, CompiledGraph& gg) : p(pp), opt(o), g(gg) {}

  int numaOf(int rank) const { return rank < (int)opt.gpu_numa.size() ? opt.gpu_numa[(size_t)rank] : 0; }

  // Aliasing of an in-place call: an output chunk that shares memory with an
  // input chunk is renamed to it before the version walk.
  Loc canon(Loc l) const {
    if (l.space != Buf::Output || opt.in_place == InPlace::None) return l;
    switch (opt.in_place) {
      case InPlace::Same:
        if (l.chunk < g.input_chunks || g.input_chunks == 0) l.space = Buf::Input;
        break;
      case InPlace::GatherSlot:  // input chunk j lives at output chunk rank*cps_out + j
        if (l.chunk / cps_out == l.owner && (l.chunk % cps_out) < std::max(1, g.input_chunks)) {
          l.space = Buf::Input;
          l.chunk = l.chunk % cps_out;
        }
        break;
      case InPlace::ScatterSlot:  // output chunk j lives at input chunk rank*cps_in + j
        l.space = Buf::Input;
        l.chunk = l.owner * cps_in + l.chunk;
        break;
      default: break;
    }
    return l;
  }

  void read(Node& n, const Loc& raw, bool wants_user_input) {
    const Loc l = canon(raw);
    LocState& s = st[l];
    if (s.version == 0) {
      if (l.space == Buf::Input) {
        // version 0 of an input chunk is the caller's data
        if (s.readers.empty()) s.readers.resize(1);
        s.readers[0].push_back(n.id);
      } else {
        s.pending.push_back(n.id);
      }
      return;
    }
    if (wants_user_input && l.space == Buf::Input && conflict.empty())
      conflict = "line " + std::to_string(n.line) + " reads user input after an aliased output chunk was written";
    n.wait_for.push_back(s.writer[(size_t)s.version]);
    if ((int)s.readers.size() <= s.version) s.readers.resize((size_t)s.version + 1);
    s.readers[(size_t)s.version].push_back(n.id);
  }

  void write(Node& n, const Loc& raw) {
    const Loc l = canon(raw);
    LocState& s = st[l];
    const int v = s.version;
    if (v > 0) n.wait_for.push_back(s.writer[(size_t)v]);
    if ((int)s.readers.size() > v)
      for (int r : s.readers[(size_t)v])
        if (r != n.id) n.wait_for.push_back(r);
    s.version = v + 1;
    if ((int)s.writer.size() <= s.version) s.writer.resize((size_t)s.version + 1, -1);
    s.writer[(size_t)s.version] = n.id;
  }
};

}  // namespace

hlResult_t compile(const Program& p, const CompileOptions& opt, CompiledGraph* out) {
  CompiledGraph g;
  g.nranks = p.nranks;
  g.input_chunks = p.input_chunks;
  g.output_chunks = p.output_chunks;
  g.internal_chunks = p.internal_chunks;
  g.scratch_chunks = p.scratch_chunks;
  g.host_chunks = p.host_chunks;
  g.send_segs = std::max(1, opt.send_segs);
  g.recv_segs = std::max(1, opt.recv_segs);
  g.by_rank.resize((size_t)p.nranks);
  int numa_max = p.numa_nodes - 1;
  for (int v : opt.gpu_numa) numa_max = std::max(numa_max, v);
  g.numa_nodes = numa_max + 1 < 1 ? 1 : numa_max + 1;
  if (g.input_chunks && g.input_chunks % g.send_segs)
    return fail(hlInvalidArgument, "schedule reads %d input chunks, not a multiple of %d segments", g.input_chunks, g.send_segs);
  if (g.output_chunks && g.output_chunks % g.recv_segs)
    return fail(hlInvalidArgument, "schedule writes %d output chunks, not a multiple of %d segments", g.output_chunks, g.recv_segs);

  Walker w(p, opt, g);
  w.cps_in = g.input_chunks ? g.input_chunks / g.send_segs : 1;
  w.cps_out = g.output_chunks ? g.output_chunks / g.recv_segs : 1;

  for (int r = 0; r < p.nranks; ++r) {
    for (const Instr& x : p.ranks[(size_t)r]) {
      Node n;
      n.id = (int)g.nodes.size();
      n.rank = r;
      n.op = x.op;
      n.line = x.line;
      const int my_numa = w.numaOf(r);
      auto host = [&](int chunk, int numa) { return Loc{Buf::Host, numa >= 0 ? numa : my_numa, chunk}; };
      auto dev = [&](Buf b, int owner, int chunk) { return Loc{b, owner, chunk}; };
      const int src_owner = x.src_rank >= 0 ? x.src_rank : r;
      switch (x.op) {
        case Op::NOP: break;
        case Op::D2D:
          n.src = dev(x.src_buf, src_owner, x.src_chunk);
          n.dst = dev(x.dst_buf, r, x.dst_chunk);
          break;
        case Op::D2DReduce:
          n.src = dev(x.src_buf, src_owner, x.src_chunk);
          n.dst = dev(x.dst_buf, r, x.dst_chunk);
          break;
        case Op::D2H:
          n.src = dev(x.src_buf, src_owner, x.src_chunk);
          n.dst = host(x.dst_chunk, x.dst_numa);
          break;
        case Op::H2D:
          n.src = host(x.src_chunk, x.src_numa);
          n.dst = dev(x.dst_buf, r, x.dst_chunk);
          break;
        case Op::H2H:
          n.src = host(x.src_chunk, x.src_numa);
          n.dst = host(x.dst_chunk, x.dst_numa);
          break;
        case Op::H2HReduce:
          n.src = host(x.src1_chunk, x.src1_numa);
          n.src2 = host(x.src2_chunk, x.src2_numa);
          n.dst = host(x.dst_chunk, x.dst_numa);
          g.uses_host_reduce = true;
          break;
      }
      if (src_owner != r && (x.op == Op::D2D || x.op == Op::D2DReduce || x.op == Op::D2H)) g.uses_remote_device = true;
      if (n.dst.space == Buf::Input && x.op != Op::NOP)
        return fail(hlInvalidArgument, "schedule line %d writes the input buffer", x.line);
      if (n.dst.space == Buf::Host && n.dst.owner >= kMaxNuma) return fail(hlInvalidArgument, "schedule line %d: NUMA id out of range", x.line);
      g.nodes.push_back(n);
      Node& nn = g.nodes.back();
      if (x.op != Op::NOP) {
        if (x.op == Op::D2D && w.canon(nn.src) == w.canon(nn.dst)) {
          nn.skip = true;  // in-place call: the chunk is already where it belongs
        } else {
          w.read(nn, nn.src, x.src_buf == Buf::Input && nn.src.space == Buf::Input);
          if (x.op == Op::H2HReduce) w.read(nn, nn.src2, false);
          if (x.op == Op::D2DReduce) w.read(nn, nn.dst, false);
          w.write(nn, nn.dst);
        }
      }
      g.by_rank[(size_t)r].push_back(nn.id);
    }
  }
  // reads that came before any write bind to the final version
  for (auto& kv : w.st) {
    LocState& s = kv.second;
    if (s.pending.empty()) continue;
    if (s.version == 0)
      return fail(hlInvalidArgument, "schedule reads %s chunk %d (owner %d) that nothing writes", bufName(kv.first.space),
                  kv.first.chunk, kv.first.owner);
    for (int id : s.pending) g.nodes[(size_t)id].wait_for.push_back(s.writer[(size_t)s.version]);
  }
  if (!w.conflict.empty()) return fail(hlUnsupported, "in-place conflict: %s", w.conflict.c_str());
  // dedupe, drop self edges, and make sure the slice-level wait graph has no cycle
  for (Node& n : g.nodes) {
    std::sort(n.wait_for.begin(), n.wait_for.end());
    n.wait_for.erase(std::unique(n.wait_for.begin(), n.wait_for.end()), n.wait_for.end());
    n.wait_for.erase(std::remove(n.wait_for.begin(), n.wait_for.end(), n.id), n.wait_for.end());
  }
  {
    const size_t N = g.nodes.size();
    std::vector<int> indeg(N, 0);
    std::vector<std::vector<int>> fwd(N);
    for (const Node& n : g.nodes)
      for (int d : n.wait_for) {
        fwd[(size_t)d].push_back(n.id);
        indeg[(size_t)n.id]++;
      }
    std::vector<int> q;
    for (size_t i = 0; i < N; ++i)
      if (!indeg[i]) q.push_back((int)i);
    size_t seen = 0;
    while (!q.empty()) {
      int v = q.back();
      q.pop_back();
      ++seen;
      for (int t : fwd[(size_t)v])
        if (--indeg[(size_t)t] == 0) q.push_back(t);
    }
    if (seen != N) return fail(hlInvalidArgument, "schedule has a dependency cycle (%zu of %zu nodes orderable)", seen, N);
  }
  // Landing fusion: pair every D2DReduce with the H2D that produced its source chunk when nobody else reads it.
  {
    std::vector<int> readers(g.nodes.size(), 0);          // how many nodes wait for node i because they READ what it wrote
    for (const Node& n : g.nodes)
      for (int d : n.wait_for) {
        const Node& wtr = g.nodes[(size_t)d];
        const bool reads_it = (n.src == wtr.dst && n.op != Op::NOP) || (n.op == Op::H2HReduce && n.src2 == wtr.dst) ||
                              (n.op == Op::D2DReduce && n.dst == wtr.dst);
        if (reads_it) readers[(size_t)d]++;
      }
    for (Node& r : g.nodes) {
      if (r.op != Op::D2DReduce || r.skip) continue;
      if (r.src.space != Buf::Internal && r.src.space != Buf::Scratch) continue;
      if (r.src.owner != r.rank) continue;
      for (int d : r.wait_for) {
        Node& wtr = g.nodes[(size_t)d];
        if (wtr.op == Op::H2D && wtr.rank == r.rank && wtr.dst == r.src && readers[(size_t)d] == 1 && wtr.fused_into < 0) {
          r.fused_h2d = wtr.id;
          wtr.fused_into = r.id;
          break;
        }
      }
    }
  }
  // Round guards: for every node that writes a staging chunk, all other nodes that read or write that chunk.
  {
    std::map<Loc, std::vector<int>> users;
    auto staged = [](const Loc& l) { return l.space == Buf::Host || l.space == Buf::Internal || l.space == Buf::Scratch; };
    for (const Node& n : g.nodes) {
      if (n.op == Op::NOP || n.skip) continue;
      if (staged(n.src)) users[n.src].push_back(n.id);
      if (n.op == Op::H2HReduce && staged(n.src2)) users[n.src2].push_back(n.id);
      if (staged(n.dst)) users[n.dst].push_back(n.id);
    }
    for (Node& n : g.nodes) {
      if (n.op == Op::NOP || n.skip || !staged(n.dst)) continue;
      for (int u : users[n.dst])
        if (u != n.id) n.round_guards.push_back(u);
      std::sort(n.round_guards.begin(), n.round_guards.end());
      n.round_guards.erase(std::unique(n.round_guards.begin(), n.round_guards.end()), n.round_guards.end());
    }
  }
  *out = std::move(g);
  return hlSuccess;
}

hlResult_t makeGeometry(const CompiledGraph& g, size_t seg_count, size_t stride, size_t active_in, size_t elem, Geometry* out) {
  if (stride > seg_count) return fail(hlInvalidArgument, "stride %zu exceeds the segment length %zu", stride, seg_count);
  Geometry geo;
  geo.elem = elem;
  geo.seg_count = seg_count;
  geo.stride = stride;
  geo.cps_in = g.input_chunks ? g.input_chunks / g.send_segs : 1;
  geo.cps_out = g.output_chunks ? g.output_chunks / g.recv_segs : 1;
  if (active_in > seg_count - stride) return fail(hlInvalidArgument, "active range exceeds the segment");
  const size_t active = active_in ? active_in : seg_count - stride;
  geo.active = active;
  const size_t ce_in = (active + (size_t)geo.cps_in - 1) / (size_t)geo.cps_in;
  const size_t ce_out = (active + (size_t)geo.cps_out - 1) / (size_t)geo.cps_out;
  if (g.input_chunks && g.output_chunks && ce_in != ce_out)
    return fail(hlInvalidArgument, "schedule splits input and output into different chunk sizes (%zu vs %zu elements)", ce_in, ce_out);
  geo.chunk_elems = g.input_chunks ? ce_in : ce_out;
  if (geo.chunk_elems == 0) geo.chunk_elems = 1;
  geo.chunk_bytes = (geo.chunk_elems * elem + 255) & ~(size_t)255;
  geo.pitch_bytes = geo.chunk_bytes;
  geo.slice_bytes = subchunkSliceFor(geo.chunk_bytes);
  // slices must be element- and 16-byte aligned
  geo.slice_bytes = std::max<size_t>(256, geo.slice_bytes & ~(size_t)255);
  geo.nslices = (int)((geo.chunk_bytes + geo.slice_bytes - 1) / geo.slice_bytes);
  if (geo.nslices < 1) geo.nslices = 1;
  *out = geo;
  return hlSuccess;
}

void deviceChunkSpan(const Geometry& geo, int cps, int c, size_t* offset, size_t* bytes) {
  const size_t seg = (size_t)(c / cps), j = (size_t)(c % cps);
  const size_t active = geo.active;
  const size_t first = std::min(active, j * geo.chunk_elems);
  const size_t len = std::min(geo.chunk_elems, active - first);
  *offset = (seg * geo.seg_count + geo.stride + first) * geo.elem;
  *bytes = len * geo.elem;
}

}  // namespace ir
}  // namespace hl
