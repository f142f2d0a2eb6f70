#include "ir/ir.h"

#include <dlfcn.h>
#include <sys/stat.h>

#include <algorithm>
#include <fstream>
#include <set>
#include <sstream>

#include "ir/xml.h"

namespace hl {
namespace ir {

const char* opName(Op op) {
  switch (op) {
    case Op::NOP: return "NOP";
    case Op::D2D: return "D2D";
    case Op::D2H: return "D2H";
    case Op::H2D: return "H2D";
    case Op::H2H: return "H2H";
    case Op::H2HReduce: return "H2HReduce";
    case Op::D2DReduce: return "D2DReduce";
  }
  return "?";
}
const char* bufName(Buf b) {
  switch (b) {
    case Buf::Input: return "input";
    case Buf::Output: return "output";
    case Buf::Scratch: return "scratch";
    case Buf::Internal: return "internal";
    case Buf::Host: return "host";
  }
  return "?";
}

size_t Program::instructions() const {
  size_t n = 0;
  for (auto& r : ranks) n += r.size();
  return n;
}

static bool parseOp(const std::string& s, Op* op) {
  static const struct { const char* n; Op o; } t[] = {{"NOP", Op::NOP}, {"D2D", Op::D2D}, {"D2H", Op::D2H},
      {"H2D", Op::H2D}, {"H2H", Op::H2H}, {"H2HReduce", Op::H2HReduce}, {"D2DReduce", Op::D2DReduce},
      {"REDUCE", Op::H2HReduce}};
  for (auto& e : t)
    if (s == e.n) {
      *op = e.o;
      return true;
    }
  return false;
}
static bool parseBuf(const std::string& s, Buf* b) {
  if (s == "input") *b = Buf::Input;
  else if (s == "output") *b = Buf::Output;
  else if (s == "scratch") *b = Buf::Scratch;
  else if (s == "internal") *b = Buf::Internal;
  else return false;
  return true;
}
static bool parseInt(const std::string* s, int* out) {
  if (!s) return false;
  char* end = nullptr;
  long v = strtol(s->c_str(), &end, 10);
  if (end == s->c_str() || *end) return false;
  *out = (int)v;
  return true;
}

hlResult_t parseProgram(const std::string& text, Program* out) {
  std::string err;
  auto root = xml::parse(text, &err);
  if (!root) return fail(hlInvalidArgument, "schedule XML: %s", err.c_str());
  if (root->name != "ir_program") return fail(hlInvalidArgument, "schedule XML: root element is <%s>, expected <ir_program>", root->name.c_str());
  Program p;
  if (auto* a = root->attr("name")) p.name = *a;
  if (auto* a = root->attr("topology")) p.topology = *a;
  if (auto* a = root->attr("variant")) p.variant = *a;
  if (!parseInt(root->attr("nranks"), &p.nranks) || p.nranks < 1 || p.nranks > 64)
    return fail(hlInvalidArgument, "schedule XML: missing or bad nranks");
  if (!parseInt(root->attr("nnodes"), &p.nnodes)) p.nnodes = 1;
  p.ranks.resize((size_t)p.nranks);
  std::vector<bool> seen((size_t)p.nranks, false);
  for (auto& child : root->children) {
    if (child->name == "description") {
      p.description = child->text;
      continue;
    }
    if (child->name != "rank") continue;
    int id = -1;
    if (!parseInt(child->attr("id"), &id) || id < 0 || id >= p.nranks)
      return fail(hlInvalidArgument, "schedule XML line %d: bad rank id", child->line);
    if (seen[(size_t)id]) return fail(hlInvalidArgument, "schedule XML line %d: rank %d defined twice", child->line, id);
    seen[(size_t)id] = true;
    for (auto& in : child->children) {
      if (in->name != "instruction") continue;
      Instr x;
      x.rank = id;
      x.line = in->line;
      const std::string* op = in->attr("op");
      if (!op || !parseOp(*op, &x.op)) return fail(hlInvalidArgument, "schedule XML line %d: unknown op '%s'", in->line, op ? op->c_str() : "");
      if (auto* a = in->attr("src_buf"))
        if (!parseBuf(*a, &x.src_buf)) return fail(hlInvalidArgument, "schedule XML line %d: bad src_buf '%s'", in->line, a->c_str());
      if (auto* a = in->attr("dst_buf"))
        if (!parseBuf(*a, &x.dst_buf)) return fail(hlInvalidArgument, "schedule XML line %d: bad dst_buf '%s'", in->line, a->c_str());
      parseInt(in->attr("src_rank"), &x.src_rank);
      parseInt(in->attr("src_numa"), &x.src_numa);
      parseInt(in->attr("dst_numa"), &x.dst_numa);
      parseInt(in->attr("src1_numa"), &x.src1_numa);
      parseInt(in->attr("src2_numa"), &x.src2_numa);
      const bool need_src = x.op != Op::NOP && x.op != Op::H2HReduce;
      const bool need_dst = x.op != Op::NOP;
      if (need_src && !parseInt(in->attr("src_chunk"), &x.src_chunk))
        return fail(hlInvalidArgument, "schedule XML line %d: %s needs src_chunk", in->line, opName(x.op));
      if (need_dst && !parseInt(in->attr("dst_chunk"), &x.dst_chunk))
        return fail(hlInvalidArgument, "schedule XML line %d: %s needs dst_chunk", in->line, opName(x.op));
      if (x.op == Op::H2HReduce) {
        if (!parseInt(in->attr("src1_chunk"), &x.src1_chunk) || !parseInt(in->attr("src2_chunk"), &x.src2_chunk))
          return fail(hlInvalidArgument, "schedule XML line %d: H2HReduce needs src1_chunk and src2_chunk", in->line);
      }
      p.ranks[(size_t)id].push_back(x);
    }
  }
  HL_CHECK(finalize(&p));
  *out = std::move(p);
  return hlSuccess;
}

hlResult_t loadProgramFile(const std::string& path, Program* out) {
  std::ifstream f(path);
  if (!f) return fail(hlSystemError, "cannot open schedule file %s", path.c_str());
  std::stringstream ss;
  ss << f.rdbuf();
  return parseProgram(ss.str(), out);
}

hlResult_t finalize(Program* p) {
  int in_max = -1, out_max = -1, int_max = -1, scr_max = -1, host_max = -1, numa_max = -1;
  size_t total = 0;
  auto devTouch = [&](Buf b, int c, bool write) {
    if (b == Buf::Input && !write) in_max = std::max(in_max, c);
    if (b == Buf::Input && write) in_max = std::max(in_max, c);
    if (b == Buf::Output) out_max = std::max(out_max, c);
    if (b == Buf::Internal) int_max = std::max(int_max, c);
    if (b == Buf::Scratch) scr_max = std::max(scr_max, c);
  };
  for (auto& rk : p->ranks)
    for (auto& x : rk) {
      ++total;
      auto chk = [&](int c) { return c >= 0 && c < kMaxChunks; };
      auto numaOk = [&](int m) { return m >= -1 && m < kMaxNuma; };
      if (!numaOk(x.src_numa) || !numaOk(x.dst_numa) || !numaOk(x.src1_numa) || !numaOk(x.src2_numa))
        return fail(hlInvalidArgument, "schedule line %d: NUMA id out of range", x.line);
      numa_max = std::max({numa_max, x.src_numa, x.dst_numa, x.src1_numa, x.src2_numa});
      if (x.src_rank >= p->nranks) return fail(hlInvalidArgument, "schedule line %d: src_rank %d out of range", x.line, x.src_rank);
      switch (x.op) {
        case Op::NOP: break;
        case Op::D2D:
        case Op::D2DReduce:
          if (!chk(x.src_chunk) || !chk(x.dst_chunk)) return fail(hlInvalidArgument, "schedule line %d: chunk index out of range", x.line);
          devTouch(x.src_buf, x.src_chunk, false);
          devTouch(x.dst_buf, x.dst_chunk, true);
          break;
        case Op::D2H:
          if (!chk(x.src_chunk) || !chk(x.dst_chunk)) return fail(hlInvalidArgument, "schedule line %d: chunk index out of range", x.line);
          devTouch(x.src_buf, x.src_chunk, false);
          host_max = std::max(host_max, x.dst_chunk);
          break;
        case Op::H2D:
          if (!chk(x.src_chunk) || !chk(x.dst_chunk)) return fail(hlInvalidArgument, "schedule line %d: chunk index out of range", x.line);
          host_max = std::max(host_max, x.src_chunk);
          devTouch(x.dst_buf, x.dst_chunk, true);
          break;
        case Op::H2H:
          if (!chk(x.src_chunk) || !chk(x.dst_chunk)) return fail(hlInvalidArgument, "schedule line %d: chunk index out of range", x.line);
          host_max = std::max({host_max, x.src_chunk, x.dst_chunk});
          break;
        case Op::H2HReduce:
          if (!chk(x.src1_chunk) || !chk(x.src2_chunk) || !chk(x.dst_chunk))
            return fail(hlInvalidArgument, "schedule line %d: chunk index out of range", x.line);
          host_max = std::max({host_max, x.src1_chunk, x.src2_chunk, x.dst_chunk});
          break;
      }
    }
  if (total > (size_t)kMaxNodes) return fail(hlInvalidArgument, "schedule has %zu instructions, limit %d", total, kMaxNodes);
  p->input_chunks = in_max + 1;
  p->output_chunks = out_max + 1;
  p->internal_chunks = int_max + 1;
  p->scratch_chunks = scr_max + 1;
  p->host_chunks = host_max + 1;
  p->numa_nodes = numa_max + 1;
  return hlSuccess;
}

std::string toXml(const Program& p) {
  std::ostringstream o;
  o << "<?xml version=\"1.0\" encoding=\"UTF-8\"?>\n";
  o << "<ir_program name=\"" << p.name << "\" nranks=\"" << p.nranks << "\" topology=\"" << p.topology << "\"";
  if (!p.variant.empty()) o << " variant=\"" << p.variant << "\"";
  o << " nnodes=\"" << p.nnodes << "\">\n";
  if (!p.description.empty()) o << "  <description>" << p.description << "</description>\n";
  for (int r = 0; r < p.nranks; ++r) {
    o << "  <rank id=\"" << r << "\">\n";
    for (auto& x : p.ranks[(size_t)r]) {
      o << "    <instruction op=\"" << opName(x.op) << "\"";
      const bool dev_src = x.op == Op::D2D || x.op == Op::D2DReduce || x.op == Op::D2H;
      const bool dev_dst = x.op == Op::D2D || x.op == Op::D2DReduce || x.op == Op::H2D;
      if (dev_src && x.src_rank >= 0 && x.src_rank != r) o << " src_rank=\"" << x.src_rank << "\"";
      if (dev_src && x.src_buf != Buf::Input) o << " src_buf=\"" << bufName(x.src_buf) << "\"";
      if (dev_dst && x.dst_buf != Buf::Output) o << " dst_buf=\"" << bufName(x.dst_buf) << "\"";
      if (x.op == Op::H2HReduce) {
        o << " src1_chunk=\"" << x.src1_chunk << "\"";
        if (x.src1_numa >= 0) o << " src1_numa=\"" << x.src1_numa << "\"";
        o << " src2_chunk=\"" << x.src2_chunk << "\"";
        if (x.src2_numa >= 0) o << " src2_numa=\"" << x.src2_numa << "\"";
      } else if (x.op != Op::NOP) {
        o << " src_chunk=\"" << x.src_chunk << "\"";
        if (x.src_numa >= 0 && (x.op == Op::H2D || x.op == Op::H2H)) o << " src_numa=\"" << x.src_numa << "\"";
      }
      if (x.op != Op::NOP) {
        o << " dst_chunk=\"" << x.dst_chunk << "\"";
        if (x.dst_numa >= 0 && (x.op == Op::D2H || x.op == Op::H2H || x.op == Op::H2HReduce)) o << " dst_numa=\"" << x.dst_numa << "\"";
      }
      o << "/>\n";
    }
    o << "  </rank>\n";
  }
  o << "</ir_program>\n";
  return o.str();
}

std::string numaPattern(const std::vector<int>& gpu_numa) {
  std::string s;
  for (int v : gpu_numa) s.push_back((char)('0' + (v < 0 ? 0 : v % 10)));
  return s;
}
std::vector<int> parsePattern(const std::string& pattern) {
  std::vector<int> v;
  for (char c : pattern)
    if (c >= '0' && c <= '9') v.push_back(c - '0');
  return v;
}

static bool fileExists(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

static std::string libraryDir() {
  Dl_info info;
  if (dladdr((void*)&libraryDir, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    size_t k = p.rfind('/');
    if (k != std::string::npos) return p.substr(0, k);
  }
  return ".";
}

std::string findProgramFile(const std::string& collective, const std::string& pattern, const std::string& variant,
                            const std::string& extra_dir) {
  const std::string file = collective + "_" + pattern + (variant.empty() ? "" : "_" + variant) + ".xml";
  std::vector<std::string> dirs;
  if (!extra_dir.empty()) dirs.push_back(extra_dir);
  const std::string cfg = Config::get().ir_path;
  if (!cfg.empty()) {
    if (cfg.size() > 4 && cfg.compare(cfg.size() - 4, 4, ".xml") == 0) {
      if (fileExists(cfg)) return cfg;  // a single file forced by the user
    } else {
      dirs.push_back(cfg);
    }
  }
  const std::string lib = libraryDir();
  dirs.push_back(lib + "/ir");
  dirs.push_back(lib + "/../ir");
  dirs.push_back(lib + "/../share/hylink/ir");
  dirs.push_back("./ir");
  for (auto& d : dirs)
    if (fileExists(d + "/" + file)) return d + "/" + file;
  return "";
}

// ------------------------------------------------------------------ generator
namespace {
struct Gen {
  Program p;
  const std::vector<int>& numa;
  int n;
  explicit Gen(const std::vector<int>& nm) : numa(nm), n((int)nm.size()) {
    p.nranks = n;
    p.ranks.resize((size_t)n);
  }
  Instr& add(int r, Op op) {
    p.ranks[(size_t)r].emplace_back();
    Instr& x = p.ranks[(size_t)r].back();
    x.op = op;
    x.rank = r;
    return x;
  }
  void d2h(int r, Buf sb, int sc, int hc, int hn) {
    Instr& x = add(r, Op::D2H);
    x.src_buf = sb;
    x.src_chunk = sc;
    x.dst_chunk = hc;
    x.dst_numa = hn;
  }
  void h2d(int r, int hc, int hn, Buf db, int dc) {
    Instr& x = add(r, Op::H2D);
    x.src_chunk = hc;
    x.src_numa = hn;
    x.dst_buf = db;
    x.dst_chunk = dc;
  }
  void d2d(int r, Buf sb, int sc, Buf db, int dc, Op op = Op::D2D) {
    Instr& x = add(r, op);
    x.src_buf = sb;
    x.src_chunk = sc;
    x.dst_buf = db;
    x.dst_chunk = dc;
  }
  void h2hReduce(int r, int c1, int n1, int c2, int n2, int dc, int dn) {
    Instr& x = add(r, Op::H2HReduce);
    x.src1_chunk = c1;
    x.src1_numa = n1;
    x.src2_chunk = c2;
    x.src2_numa = n2;
    x.dst_chunk = dc;
    x.dst_numa = dn;
  }
  // NUMA nodes that host at least one rank other than `except`
  std::vector<int> readerNumas(int except) const {
    std::set<int> s;
    for (int q = 0; q < n; ++q)
      if (q != except) s.insert(numa[(size_t)q]);
    return std::vector<int>(s.begin(), s.end());
  }
};

std::string topologyName(const std::vector<int>& numa) {
  std::set<int> s(numa.begin(), numa.end());
  std::ostringstream o;
  o << s.size() << "numa_" << numa.size() << "gpu_" << numaPattern(numa);
  return o.str();
}
}  // namespace

hlResult_t generate(const std::string& collective, const std::vector<int>& gpu_numa, const std::string& variant,
                    int root, Program* out) {
  const int n = (int)gpu_numa.size();
  if (n < 1 || n > 16) return fail(hlInvalidArgument, "schedule generator: %d ranks unsupported", n);
  for (int v : gpu_numa)
    if (v < 0 || v >= kMaxNuma) return fail(hlInvalidArgument, "schedule generator: NUMA id %d out of range", v);
  Gen g(gpu_numa);
  g.p.name = collective;
  g.p.variant = variant;
  g.p.topology = topologyName(gpu_numa);
  const bool single = variant == "single_d2h";
  const bool host_reduce = variant == "host_reduce";
  const bool ring = variant == "ring";
  const int K = std::max(1, std::min(n - 1, 4));  // landing slots in the internal buffer
  auto numaOf = [&](int r) { return gpu_numa[(size_t)r]; };

  if (collective == "allgather") {
    g.p.description = "generated: each rank uploads its chunk to every NUMA node that has readers; all downloads are NUMA-local";
    for (int r = 0; r < n; ++r) {
      if (single) g.d2h(r, Buf::Input, 0, r, numaOf(r));
      else
        for (int m : g.readerNumas(r)) g.d2h(r, Buf::Input, 0, r, m);
      g.d2d(r, Buf::Input, 0, Buf::Output, r);
      for (int k = 1; k < n; ++k) {
        const int q = (r + k) % n;
        g.h2d(r, q, single ? numaOf(q) : numaOf(r), Buf::Output, q);
      }
    }
  } else if (collective == "alltoall") {
    g.p.description = "generated: sender uploads chunk q to the receiver's NUMA node; receiver downloads locally";
    for (int r = 0; r < n; ++r) {
      for (int k = 1; k < n; ++k) {
        const int q = (r + k) % n;
        g.d2h(r, Buf::Input, q, q * n + r, single ? numaOf(r) : numaOf(q));
      }
      g.d2d(r, Buf::Input, r, Buf::Output, r);
      for (int k = 1; k < n; ++k) {
        const int q = (r + k) % n;
        g.h2d(r, r * n + q, single ? numaOf(q) : numaOf(r), Buf::Output, q);
      }
    }
  } else if (collective == "broadcast") {
    if (root < 0 || root >= n) return fail(hlInvalidArgument, "schedule generator: broadcast root %d out of range", root);
    g.p.description = "generated: root uploads once per NUMA node with readers; everyone downloads locally";
    for (int r = 0; r < n; ++r) {
      if (r == root) {
        for (int m : g.readerNumas(root)) g.d2h(r, Buf::Input, 0, 0, m);
        g.d2d(r, Buf::Input, 0, Buf::Output, 0);
      } else {
        g.h2d(r, 0, numaOf(r), Buf::Output, 0);
      }
    }
  } else if (collective == "reducescatter" || collective == "allreduce") {
    const bool ar = collective == "allreduce";
    const int out_chunk_of_owner = 0;
    if (ring) {
      // Segment s travels once around the ring s+1, s+2, ..., s through host memory: the first rank uploads its
      // contribution, every later rank folds its own contribution into the travelling partial sum on the CPU
      // (H2HReduce), the owner s folds last and downloads the result. The CPU work of a segment is spread over n - 1
      // ranks instead of sitting on the owner (the host_reduce variant).
      g.p.description = "generated: ring through host memory, every rank folds its own contribution into the travelling partial sum on the CPU";
      auto pos = [&](int s, int r) { const int k = (r - s + n) % n; return k == 0 ? n : k; };   // 1-based place of r in the chain of segment s
      auto consumer = [&](int s, int r) { return pos(s, r) == 1 ? (r + 1) % n : r; };           // who reads contribution (s, r)
      auto acc = [&](int s, int k) { return n * n + s * n + k; };                              // partial sum of segment s after k contributions
      for (int r = 0; r < n; ++r) {
        const int own_out = ar ? r : out_chunk_of_owner;
        for (int k = 1; k <= n; ++k) {
          const int s = (r - k + n) % n;   // the segment in whose chain r has place k
          g.d2h(r, Buf::Input, s, s * n + r, numaOf(consumer(s, r)));
        }
        if (n == 1) {
          g.h2d(r, r * n + r, numaOf(r), Buf::Output, own_out);
          continue;
        }
        for (int k = 2; k <= n; ++k) {
          const int s = (r - k + n) % n;
          const int prev_rank = (r - 1 + n) % n;
          const int prev = k == 2 ? s * n + prev_rank : acc(s, k - 1);
          const int dst_numa = k == n ? numaOf(r) : numaOf((r + 1) % n);
          g.h2hReduce(r, prev, numaOf(r), s * n + r, numaOf(r), acc(s, k), dst_numa);
        }
        g.h2d(r, acc(r, n), numaOf(r), Buf::Output, own_out);
        if (ar)
          for (int k = 1; k < n; ++k) {
            const int q = (r + k) % n;
            g.h2d(r, acc(q, n), numaOf(q), Buf::Output, q);
          }
      }
    } else if (!host_reduce) {
      g.p.description = ar ? "generated: mesh reduce-scatter with device reduce on landing, then all-gather through NUMA-local host chunks"
                           : "generated: one-shot mesh, owner reduces every landed contribution on the device";
      for (int r = 0; r < n; ++r) {
        const int own_out = ar ? r : out_chunk_of_owner;
        for (int k = 1; k < n; ++k) {
          const int s = (r + k) % n;  // contribution for owner s lands on s's NUMA node
          g.d2h(r, Buf::Input, s, s * n + r, numaOf(s));
        }
        g.d2d(r, Buf::Input, r, Buf::Output, own_out);
        for (int k = 1; k < n; ++k) {
          const int s = (r + k) % n;
          const int slot = (k - 1) % K;
          g.h2d(r, r * n + s, numaOf(r), Buf::Internal, slot);
          g.d2d(r, Buf::Internal, slot, Buf::Output, own_out, Op::D2DReduce);
        }
        if (ar) {
          for (int m : g.readerNumas(r)) g.d2h(r, Buf::Output, r, n * n + r, m);
          for (int k = 1; k < n; ++k) {
            const int q = (r + k) % n;
            g.h2d(r, n * n + q, numaOf(r), Buf::Output, q);
          }
        }
      }
    } else {
      g.p.description = "generated: every contribution is uploaded to the owner's NUMA node and folded by the CPU (H2HReduce chain)";
      for (int r = 0; r < n; ++r) {
        const int own_out = ar ? r : out_chunk_of_owner;
        for (int k = 0; k < n; ++k) {
          const int s = (r + k) % n;
          g.d2h(r, Buf::Input, s, s * n + r, numaOf(s));
        }
        // temporaries of owner r: two alternating chunks behind the n*n landing area
        const int t0 = n * n + 2 * r, t1 = t0 + 1;
        const int m = numaOf(r);
        int cur = -1;
        if (n == 1) {
          cur = r * n;
        } else {
          g.h2hReduce(r, r * n + 0, m, r * n + 1, m, t0, m);
          cur = t0;
          for (int s = 2; s < n; ++s) {
            const int nxt = cur == t0 ? t1 : t0;
            g.h2hReduce(r, cur, m, r * n + s, m, nxt, m);
            cur = nxt;
          }
        }
        g.h2d(r, cur, m, Buf::Output, own_out);
        if (ar) {
          // the folded chunk of owner q is read straight from q's NUMA node
          for (int k = 1; k < n; ++k) {
            const int q = (r + k) % n;
            const int fin = (n == 1) ? q * n : ((n - 1) % 2 == 1 ? n * n + 2 * q : n * n + 2 * q + 1);
            g.h2d(r, fin, numaOf(q), Buf::Output, q);
          }
        }
      }
    }
  } else {
    return fail(hlInvalidArgument, "schedule generator: unknown collective '%s'", collective.c_str());
  }
  HL_CHECK(finalize(&g.p));
  *out = std::move(g.p);
  return hlSuccess;
}

}  // namespace ir
}  // namespace hl
