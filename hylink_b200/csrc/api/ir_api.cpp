// C entry points of the schedule tools: generate, validate/compile and run
// schedule XML. Used by the Python DSL and by tests.
#include <cstring>

#include "api/comm.h"
#include "hylink/hylink_ext.h"
#include "ir/compiler.h"
#include "host/topology.h"
#include "pcie/pcie_path.h"

using namespace hl;

static hlResult_t copyOut(const std::string& s, char* buf, size_t* len) {
  if (!len) return hlInvalidArgument;
  const size_t need = s.size() + 1;
  if (buf && *len >= need) memcpy(buf, s.c_str(), need);
  *len = need;
  return hlSuccess;
}

extern "C" {

hlResult_t hlIrGenerate(const char* collective, const char* numa_pattern, const char* variant, int root, char* buf, size_t* len) {
  if (!collective || !numa_pattern) return hlInvalidArgument;
  ir::Program p;
  HL_CHECK(ir::generate(collective, ir::parsePattern(numa_pattern), variant ? variant : "", root, &p));
  return copyOut(ir::toXml(p), buf, len);
}

int hlTopoPairQuery(const char* bus_a, const char* bus_b, int* same_switch, int* nvlink) {
  bool pix = false, nvl = false;
  const bool ok = hl::nvmlPairQuery(bus_a ? bus_a : "", bus_b ? bus_b : "", &pix, &nvl);
  if (same_switch) *same_switch = pix ? 1 : 0;
  if (nvlink) *nvlink = nvl ? 1 : 0;
  return ok ? 1 : 0;
}
int hlTopoDirectAllowed(const char* collective, const char* pattern, const unsigned char* pix, const unsigned char* nvlink,
                        const unsigned char* peer, int n) {
  hl::PairTopology t;
  t.n = n;
  t.pix.assign(pix, pix + (size_t)n * n);
  t.nvlink.assign(nvlink, nvlink + (size_t)n * n);
  t.peer.assign(peer, peer + (size_t)n * n);
  return hl::directVariantAllowed(collective ? collective : "", pattern ? pattern : "", t) ? 1 : 0;
}

int hlDmaLaneCount(const char* collective, size_t message_bytes, int world, int max_lanes, int forced) {
  return hl::dmaLanePolicy(collective, message_bytes, world, max_lanes, forced);
}

hlResult_t hlIrInspect(const char* xml, const char* numa_pattern, int send_segs, int recv_segs, int in_place, hlIrInfo* info) {
  if (!xml || !info) return hlInvalidArgument;
  ir::Program p;
  HL_CHECK(ir::parseProgram(xml, &p));
  ir::CompileOptions opt;
  opt.send_segs = send_segs;
  opt.recv_segs = recv_segs;
  opt.in_place = (ir::InPlace)in_place;
  if (numa_pattern) opt.gpu_numa = ir::parsePattern(numa_pattern);
  ir::CompiledGraph g;
  HL_CHECK(ir::compile(p, opt, &g));
  memset(info, 0, sizeof(*info));
  info->nranks = p.nranks;
  info->instructions = (int)g.nodes.size();
  info->input_chunks = g.input_chunks;
  info->output_chunks = g.output_chunks;
  info->internal_chunks = g.internal_chunks;
  info->host_chunks = g.host_chunks;
  info->numa_nodes = g.numa_nodes;
  info->uses_remote_device = g.uses_remote_device;
  info->uses_host_reduce = g.uses_host_reduce;
  size_t edges = 0;
  for (auto& n : g.nodes) edges += n.wait_for.size();
  info->dependency_edges = (int)edges;
  return hlSuccess;
}

hlResult_t hlIrRoundTrip(const char* xml, char* buf, size_t* len) {
  if (!xml) return hlInvalidArgument;
  ir::Program p;
  HL_CHECK(ir::parseProgram(xml, &p));
  return copyOut(ir::toXml(p), buf, len);
}

hlResult_t hlSubmitIr(hlComm_t comm, const char* xml, const void* send, void* recv, size_t seg_count, size_t stride,
                      int send_segs, int recv_segs, hlDataType_t t, hlRedOp_t op, hlStream_t stream) {
  if (!comm || !comm->pcie) return fail(hlUnsupported, "the PCIe path is not initialised on this communicator");
  std::lock_guard<std::mutex> lk(comm->mu);
  return comm->pcie->submitIr(xml, send, recv, seg_count, stride, send_segs, recv_segs, t, op, stream);
}

hlResult_t hlCommNumaPattern(hlComm_t comm, char* buf, size_t* len) {
  if (!comm) return hlInvalidArgument;
  std::string s = comm->pcie ? ir::numaPattern(comm->pcie->rankNuma()) : std::string((size_t)comm->nranks, '0');
  return copyOut(s, buf, len);
}

}  // extern "C"
