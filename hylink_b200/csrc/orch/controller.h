// Decision logic of the multipath orchestrator (no device, no I/O):
// size buckets, operation keys, the byte planner, the feedback algorithms that
// retune the PCIe share `alpha`, the per-key controller with its parameter
// cache, and the overlap metrics of one forked call.
//
// Parity (multipath-orchestrator/libampccl/):
//   common/size_bucket.h:13-40      geometric buckets from 4 MiB, two per octave
//   common/op_key.h:17-31           (op, bucket, dtype, nranks, comm)
//   core/planner.h:19-80            alpha split, min message / min part gates, 128-byte alignment
//   controller/algo_factory.h:13-55 static | tcp (inverse proportion) | split_ratio
//   controller/algo_inverse_proportion.h:16-92
//   controller/algo_split_ratio_control.h:39-128
//   controller/controller.h:21-57, cache/param_cache.h:12-97
//   telemetry/path_timing.h:33-77, telemetry/stats.h:8-46
// Defaults differ where the reference is tuned for Ascend HCCS: with NVLink 5
// at ~0.7 TB/s against one PCIe Gen5 x16 link the balanced share is a few
// percent, so the initial share and its floor are lower here; the reference's
// environment variables still override them.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <string>

#include "hylink/hylink.h"

namespace hl {
namespace orch {

enum OpKind { kOpAllReduce = 0, kOpAllGather = 1, kOpReduceScatter = 2, kOpAllToAll = 3, kOpBroadcast = 4 };
const char* opKindName(int op);

// Index of the bucket [4 MiB * 2^(k/2), 4 MiB * 2^((k+1)/2)); below 4 MiB: -1.
int sizeBucket(size_t bytes);
size_t sizeBucketLowerBound(int bucket);

struct OpKey {
  int op = 0;
  int bucket = -1;
  int dtype = 0;
  int nranks = 0;
  uint64_t comm_hash = 0;
  bool operator<(const OpKey& o) const;
  std::string str() const;
};
OpKey makeOpKey(int op, size_t bytes, int dtype, int nranks, uint64_t comm_hash);

struct Plan {
  size_t fast_bytes = 0;
  size_t pcie_bytes = 0;
  bool use_pcie = false;
};
struct PlannerLimits {
  size_t min_msg_bytes = 4u << 20;
  size_t min_part_bytes = 4096;
  size_t align = 128;
};
// `elem`: both parts are also kept multiples of the element size.
Plan createPlan(size_t total_bytes, double alpha, bool pcie_allowed, size_t elem, const PlannerLimits& lim);

struct ExecStat {
  double fast_time = 0;   // seconds, max over ranks
  double pcie_time = 0;
  size_t fast_bytes = 0;
  size_t pcie_bytes = 0;
  bool fast_ok = true, pcie_ok = true;
  double fastBw() const { return fast_time > 0 ? (double)fast_bytes / fast_time : 0; }   // bytes/s
  double pcieBw() const { return pcie_time > 0 ? (double)pcie_bytes / pcie_time : 0; }
};

struct ParamValue {
  double alpha = 0;
  double best_alpha = 0;
  double best_bandwidth = 0;   // bytes/s of the best total seen
  uint64_t updates = 0;
  bool use_pcie = true;        // latched off after a PCIe failure
  int losing_streak = 0;       // consecutive forked calls that were slower than the dedicated link alone would have been
  int cooldown = 0;            // forked calls to skip before the PCIe path is tried again
};

class AdaptiveAlgo {
 public:
  virtual ~AdaptiveAlgo() {}
  virtual const char* name() const = 0;
  virtual double suggest(const ParamValue& current) = 0;
  virtual void update(const ExecStat& stat) = 0;
  virtual double alpha() const = 0;
  virtual void reset() = 0;
};
// kind: "static" | "tcp" | "inverse_proportion" | "split_ratio"; unknown names give split_ratio.
std::unique_ptr<AdaptiveAlgo> makeAlgo(const std::string& kind, int nranks);

class AdaptiveController {
 public:
  AdaptiveController(const std::string& algo_kind, int nranks) : kind_(algo_kind), nranks_(nranks) {}
  double suggestAlpha(const OpKey& key);
  bool usePcie(const OpKey& key) const;
  void update(const OpKey& key, const ExecStat& stat);
  const ParamValue* lookup(const OpKey& key) const;
  void seed(const OpKey& key, const ParamValue& v);
  std::string dumpJson() const;
  // Accepts the text produced by dumpJson(); unknown fields are ignored.
  bool loadJson(const std::string& text);
  size_t size() const { return cache_.size(); }

 private:
  struct Entry {
    ParamValue value;
    std::unique_ptr<AdaptiveAlgo> algo;
  };
  Entry& entry(const OpKey& key);
  std::string kind_;
  int nranks_;
  std::map<OpKey, Entry> cache_;
};

// Overlap of the two paths of one call from their start/end timestamps (seconds).
struct PathTiming {
  double fast = 0, pcie = 0, overlap = 0, span = 0, parallel_efficiency = 0;
};
PathTiming computePathTiming(double fast_start, double fast_end, double pcie_start, double pcie_end);

// busbw factor of the nccl-tests convention.
double busFactor(int op, int nranks);

}  // namespace orch
}  // namespace hl
