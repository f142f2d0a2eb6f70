#include "orch/controller.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "core/core.h"

namespace hl {
namespace orch {

const char* opKindName(int op) {
  switch (op) {
    case kOpAllReduce: return "AllReduce";
    case kOpAllGather: return "AllGather";
    case kOpReduceScatter: return "ReduceScatter";
    case kOpAllToAll: return "AllToAll";
    case kOpBroadcast: return "Broadcast";
    default: return "?";
  }
}

int sizeBucket(size_t bytes) {
  const double base = 4.0 * 1024 * 1024;
  if ((double)bytes < base) return -1;
  return (int)std::floor(2.0 * std::log2((double)bytes / base) + 1e-9);
}
size_t sizeBucketLowerBound(int bucket) {
  if (bucket < 0) return 0;
  return (size_t)std::llround(4.0 * 1024 * 1024 * std::pow(2.0, bucket / 2.0));
}

bool OpKey::operator<(const OpKey& o) const {
  if (op != o.op) return op < o.op;
  if (bucket != o.bucket) return bucket < o.bucket;
  if (dtype != o.dtype) return dtype < o.dtype;
  if (nranks != o.nranks) return nranks < o.nranks;
  return comm_hash < o.comm_hash;
}
std::string OpKey::str() const {
  char b[128];
  snprintf(b, sizeof(b), "%s/b%d/t%d/n%d", opKindName(op), bucket, dtype, nranks);
  return b;
}
OpKey makeOpKey(int op, size_t bytes, int dtype, int nranks, uint64_t comm_hash) {
  OpKey k;
  k.op = op;
  k.bucket = sizeBucket(bytes);
  k.dtype = dtype;
  k.nranks = nranks;
  k.comm_hash = comm_hash;
  return k;
}

Plan createPlan(size_t total, double alpha, bool pcie_allowed, size_t elem, const PlannerLimits& lim) {
  Plan p;
  p.fast_bytes = total;
  if (!pcie_allowed || total < lim.min_msg_bytes || !(alpha > 0.0)) return p;
  if (alpha > 1.0) alpha = 1.0;
  if (elem == 0) elem = 1;
  size_t align = std::max<size_t>(lim.align, 1);
  while (align % elem) align += lim.align ? lim.align : 1;  // smallest multiple of `align` that keeps elements whole
  size_t pcie = (size_t)((double)total * alpha);
  size_t fast = total - pcie;
  // the split point is the end of the fast part: round it up, the PCIe part takes what is left
  fast = (fast + align - 1) / align * align;
  if (fast > total) fast = total;
  pcie = total - fast;
  if (pcie < lim.min_part_bytes) return p;           // not worth a second path
  if (fast < lim.min_part_bytes) {                   // everything over PCIe
    p.fast_bytes = 0;
    p.pcie_bytes = total;
    p.use_pcie = true;
    return p;
  }
  p.fast_bytes = fast;
  p.pcie_bytes = pcie;
  p.use_pcie = true;
  return p;
}

// ------------------------------------------------------------ algorithms
namespace {
double envD(std::initializer_list<const char*> names, double d) { return envDouble(names, d); }

class StaticAlgo : public AdaptiveAlgo {
 public:
  StaticAlgo() { reset(); }
  const char* name() const override { return "static"; }
  double suggest(const ParamValue&) override { return alpha_; }
  void update(const ExecStat& s) override {
    if (!s.fast_ok || !s.pcie_ok) alpha_ *= 0.5;
  }
  double alpha() const override { return alpha_; }
  void reset() override { alpha_ = std::min(1.0, std::max(0.0, Config::get().static_alpha)); }

 private:
  double alpha_ = 0;
};

// "tcp": multiplicative moves driven by the ratio of the two path durations.
class InverseProportionAlgo : public AdaptiveAlgo {
 public:
  explicit InverseProportionAlgo(int nranks) {
    decrease_ = 0.5 * std::sqrt(2.0 / std::max(1, nranks));
    decrease_ = std::min(1.0, std::max(0.2, decrease_));
    lo_ = envD({"HYLINK_TCP_HOLD_RATE_LOW", "AMPCCL_TCP_HOLD_RATE_LOW"}, 0.95);
    hi_ = envD({"HYLINK_TCP_HOLD_RATE_HIGH", "AMPCCL_TCP_HOLD_RATE_HIGH"}, 1.10);
    if (!(lo_ > 0) || !(hi_ > lo_)) {
      lo_ = 0.95;
      hi_ = 1.10;
    }
    reset();
  }
  const char* name() const override { return "tcp"; }
  double suggest(const ParamValue& cur) override {
    if (cur.alpha > 0) alpha_ = cur.alpha;
    clamp();
    return alpha_;
  }
  void update(const ExecStat& s) override {
    if (!s.fast_ok || !s.pcie_ok) {
      alpha_ *= decrease_;
      clamp();
      return;
    }
    if (s.pcie_bytes == 0) return;        // a fast-only sample carries no PCIe timing
    if (++samples_ <= 2) return;          // the first forked calls pay one-off set-up costs
    if (s.pcie_time > 0 && s.fast_time > 0) {
      const double rate = s.fast_time / s.pcie_time;
      if (rate <= lo_) alpha_ *= 0.5;                  // PCIe finishes later: halve its share
      else if (rate >= hi_) alpha_ *= rate * 0.96;     // PCIe has slack: grow towards balance
    }
    clamp();
  }
  double alpha() const override { return alpha_; }
  void reset() override {
    alpha_ = envD({"HYLINK_TCP_INITIAL_ALPHA", "AMPCCL_TCP_INITIAL_ALPHA"}, 0.01);
    if (!(alpha_ >= kMin && alpha_ <= kMax)) alpha_ = 0.01;
    samples_ = 0;
  }

 private:
  void clamp() { alpha_ = std::min(kMax, std::max(kMin, alpha_)); }
  static constexpr double kMin = 0.001, kMax = 0.39;
  double alpha_ = 0.01, decrease_ = 0.5, lo_ = 0.95, hi_ = 1.10;
  int samples_ = 0;
};

// Tracks an EMA of the PCIe bandwidth and steers alpha towards the share that
// makes both paths finish together: x* = Bp / (Bp + Bf).
class SplitRatioAlgo : public AdaptiveAlgo {
 public:
  SplitRatioAlgo() { reset(); }
  const char* name() const override { return "split_ratio"; }
  double suggest(const ParamValue& cur) override {
    if (cur.alpha > 0) alpha_ = cur.alpha;
    clamp();
    return alpha_;
  }
  void update(const ExecStat& s) override {
    ++updates_;
    if (!s.fast_ok || !s.pcie_ok) {
      alpha_ *= 0.5;
      clamp();
      return;
    }
    if (s.pcie_bytes == 0) return;
    const double bp = s.pcieBw(), bf = s.fastBw();
    if (bp <= 0 || bf <= 0) return;
    const double smooth = smooth_, eta = eta_;   // read from the environment once, in reset()
    const size_t warmup = warmup_;
    // tiny PCIe parts measure latency, not bandwidth: keep them out of the estimate
    if (s.pcie_bytes >= (4u << 20) || bp_hat_ <= 0) bp_hat_ = bp_hat_ <= 0 ? bp : smooth * bp + (1 - smooth) * bp_hat_;
    const double x_star = bp_hat_ / (bp_hat_ + bf);
    const double t_pcie = alpha_ / bp_hat_, t_fast = (1 - alpha_) / bf;
    if (updates_ > warmup && t_pcie > 1.05 * t_fast && s.pcie_bytes >= (16u << 20)) alpha_ *= 0.9;  // PCIe is the bottleneck: back off
    else alpha_ += eta * (x_star - alpha_);
    clamp();
  }
  double alpha() const override { return alpha_; }
  void reset() override {
    alpha_ = envD({"HYLINK_SPLIT_RATIO_INITIAL_ALPHA", "AMPCCL_SPLIT_RATIO_INITIAL_ALPHA"}, 0.05);
    min_ = envD({"HYLINK_SPLIT_RATIO_MIN_ALPHA", "AMPCCL_SPLIT_RATIO_MIN_ALPHA"}, 0.005);
    smooth_ = envD({"HYLINK_SPLIT_RATIO_SMOOTHING", "AMPCCL_SPLIT_RATIO_SMOOTHING"}, 0.7);
    eta_ = envD({"HYLINK_SPLIT_RATIO_ETA", "AMPCCL_SPLIT_RATIO_ETA"}, 0.3);
    warmup_ = (size_t)envInt({"HYLINK_SPLIT_RATIO_WARMUP_STEPS", "AMPCCL_SPLIT_RATIO_WARMUP_STEPS"}, 5);
    bp_hat_ = 0;
    updates_ = 0;
    clamp();
  }

 private:
  void clamp() { alpha_ = std::min(0.999, std::max(min_, alpha_)); }
  double alpha_ = 0.05, min_ = 0.005, bp_hat_ = 0, smooth_ = 0.7, eta_ = 0.3;
  size_t updates_ = 0, warmup_ = 5;
};
}  // namespace

std::unique_ptr<AdaptiveAlgo> makeAlgo(const std::string& kind, int nranks) {
  if (kind == "static") return std::unique_ptr<AdaptiveAlgo>(new StaticAlgo());
  if (kind == "tcp" || kind == "inverse_proportion") return std::unique_ptr<AdaptiveAlgo>(new InverseProportionAlgo(nranks));
  return std::unique_ptr<AdaptiveAlgo>(new SplitRatioAlgo());
}

// ------------------------------------------------------------ controller
AdaptiveController::Entry& AdaptiveController::entry(const OpKey& key) {
  auto it = cache_.find(key);
  if (it == cache_.end()) {
    Entry e;
    e.algo = makeAlgo(kind_, nranks_);
    e.value.alpha = e.algo->alpha();
    it = cache_.emplace(key, std::move(e)).first;
  }
  return it->second;
}
double AdaptiveController::suggestAlpha(const OpKey& key) {
  Entry& e = entry(key);
  if (!e.value.use_pcie) return 0.0;
  if (e.value.cooldown > 0) {  // the split was not paying: stay on the dedicated link for a while, then probe again
    --e.value.cooldown;
    return 0.0;
  }
  e.value.alpha = e.algo->suggest(e.value);
  return e.value.alpha;
}
bool AdaptiveController::usePcie(const OpKey& key) const {
  auto it = cache_.find(key);
  return it == cache_.end() ? true : it->second.value.use_pcie;
}
void AdaptiveController::update(const OpKey& key, const ExecStat& s) {
  Entry& e = entry(key);
  e.algo->suggest(e.value);
  e.algo->update(s);
  e.value.alpha = e.algo->alpha();
  e.value.updates++;
  if (!s.pcie_ok) e.value.use_pcie = false;  // degrade to the dedicated link for this key
  // No-gain guard (not in the reference): the host-staged path has a latency floor of several hundred microseconds
  // on this class of machine; when a forked call keeps finishing later than the dedicated link alone would have
  // (estimated from this call's own link bandwidth), stop forking this key for a while instead of paying every call.
  static const bool guard = envBool({"HYLINK_ORCH_GUARD"}, true);
  if (guard && s.fast_ok && s.pcie_ok && s.pcie_bytes && s.fast_bytes && s.fast_time > 0) {
    const double alone = s.fast_time * (double)(s.fast_bytes + s.pcie_bytes) / (double)s.fast_bytes;
    if (std::max(s.fast_time, s.pcie_time) > 1.05 * alone) {
      // The streak is long enough for the controllers to re-balance after a change of conditions first.
      static const int streak = (int)envInt({"HYLINK_ORCH_GUARD_STREAK"}, 16);
      if (++e.value.losing_streak >= streak) {
        e.value.losing_streak = 0;
        static const int cooldown = (int)envInt({"HYLINK_ORCH_COOLDOWN_CALLS"}, 200);
        e.value.cooldown = cooldown;
      }
    } else {
      e.value.losing_streak = 0;
    }
  }
  if (s.fast_ok && s.pcie_ok) {
    const double t = std::max(s.fast_time, s.pcie_time);
    const double bw = t > 0 ? (double)(s.fast_bytes + s.pcie_bytes) / t : 0;
    if (bw > e.value.best_bandwidth) {
      e.value.best_bandwidth = bw;
      e.value.best_alpha = (s.fast_bytes + s.pcie_bytes) ? (double)s.pcie_bytes / (double)(s.fast_bytes + s.pcie_bytes) : 0;
    }
  }
}
const ParamValue* AdaptiveController::lookup(const OpKey& key) const {
  auto it = cache_.find(key);
  return it == cache_.end() ? nullptr : &it->second.value;
}
void AdaptiveController::seed(const OpKey& key, const ParamValue& v) {
  Entry& e = entry(key);
  e.value = v;
}

std::string AdaptiveController::dumpJson() const {
  std::ostringstream o;
  o.precision(9);
  o << "{\"algo\":\"" << kind_ << "\",\"entries\":[";
  bool first = true;
  for (auto& kv : cache_) {
    if (!first) o << ",";
    first = false;
    const OpKey& k = kv.first;
    const ParamValue& v = kv.second.value;
    o << "{\"op\":" << k.op << ",\"bucket\":" << k.bucket << ",\"dtype\":" << k.dtype << ",\"nranks\":" << k.nranks
      << ",\"alpha\":" << v.alpha << ",\"best_alpha\":" << v.best_alpha << ",\"best_bandwidth\":" << v.best_bandwidth
      << ",\"updates\":" << v.updates << ",\"use_pcie\":" << (v.use_pcie ? 1 : 0) << "}";
  }
  o << "]}";
  return o.str();
}

static bool findNumber(const std::string& obj, const char* field, double* out) {
  const std::string pat = std::string("\"") + field + "\":";
  size_t p = obj.find(pat);
  if (p == std::string::npos) return false;
  const char* s = obj.c_str() + p + pat.size();
  char* end = nullptr;
  double v = strtod(s, &end);
  if (end == s) return false;
  *out = v;
  return true;
}

bool AdaptiveController::loadJson(const std::string& text) {
  size_t p = text.find("\"entries\"");
  if (p == std::string::npos) return false;
  p = text.find('[', p);
  if (p == std::string::npos) return false;
  int loaded = 0;
  for (;;) {
    size_t a = text.find('{', p);
    size_t close = text.find(']', p);
    if (a == std::string::npos || (close != std::string::npos && close < a)) break;
    size_t b = text.find('}', a);
    if (b == std::string::npos) return false;
    const std::string obj = text.substr(a, b - a + 1);
    double op, bucket, dtype, nranks, alpha;
    if (findNumber(obj, "op", &op) && findNumber(obj, "bucket", &bucket) && findNumber(obj, "dtype", &dtype) &&
        findNumber(obj, "nranks", &nranks) && findNumber(obj, "alpha", &alpha)) {
      OpKey k;
      k.op = (int)op;
      k.bucket = (int)bucket;
      k.dtype = (int)dtype;
      k.nranks = (int)nranks;
      k.comm_hash = 0;
      ParamValue v;
      v.alpha = alpha;
      double t;
      if (findNumber(obj, "best_alpha", &t)) v.best_alpha = t;
      if (findNumber(obj, "best_bandwidth", &t)) v.best_bandwidth = t;
      if (findNumber(obj, "updates", &t)) v.updates = (uint64_t)t;
      if (findNumber(obj, "use_pcie", &t)) v.use_pcie = t != 0;
      seed(k, v);
      ++loaded;
    }
    p = b + 1;
  }
  return loaded > 0 || text.find("[]") != std::string::npos;
}

PathTiming computePathTiming(double fs, double fe, double ps, double pe) {
  PathTiming t;
  t.fast = std::max(0.0, fe - fs);
  t.pcie = std::max(0.0, pe - ps);
  t.overlap = std::max(0.0, std::min(fe, pe) - std::max(fs, ps));
  t.span = std::max(fe, pe) - std::min(fs, ps);
  t.parallel_efficiency = t.span > 0 ? (t.fast + t.pcie) / (2.0 * t.span) : 0;
  return t;
}

double busFactor(int op, int n) {
  if (n <= 1) return 1.0;
  return op == kOpAllReduce ? 2.0 * (n - 1) / n : (double)(n - 1) / n;
}

}  // namespace orch
}  // namespace hl

// ---- C entry points for tests and tools ---------------------------------
extern "C" {
using namespace hl::orch;
int hlSizeBucket(size_t bytes) { return sizeBucket(bytes); }
void hlPlanCreate(size_t total, double alpha, int pcie_allowed, size_t elem, size_t min_msg, size_t min_part, size_t* fast,
                  size_t* pcie, int* use_pcie) {
  PlannerLimits lim;
  if (min_msg) lim.min_msg_bytes = min_msg;
  if (min_part) lim.min_part_bytes = min_part;
  Plan p = createPlan(total, alpha, pcie_allowed != 0, elem, lim);
  if (fast) *fast = p.fast_bytes;
  if (pcie) *pcie = p.pcie_bytes;
  if (use_pcie) *use_pcie = p.use_pcie ? 1 : 0;
}
void* hlCtlCreate(const char* algo, int nranks) { return new AdaptiveController(algo ? algo : "split_ratio", nranks); }
void hlCtlDestroy(void* c) { delete (AdaptiveController*)c; }
double hlCtlSuggest(void* c, int op, size_t bytes, int dtype, int nranks) {
  return ((AdaptiveController*)c)->suggestAlpha(makeOpKey(op, bytes, dtype, nranks, 0));
}
void hlCtlUpdate(void* c, int op, size_t bytes, int dtype, int nranks, double fast_time, double pcie_time, size_t fast_bytes,
                 size_t pcie_bytes, int fast_ok, int pcie_ok) {
  ExecStat s;
  s.fast_time = fast_time;
  s.pcie_time = pcie_time;
  s.fast_bytes = fast_bytes;
  s.pcie_bytes = pcie_bytes;
  s.fast_ok = fast_ok != 0;
  s.pcie_ok = pcie_ok != 0;
  ((AdaptiveController*)c)->update(makeOpKey(op, bytes, dtype, nranks, 0), s);
}
int hlCtlUsePcie(void* c, int op, size_t bytes, int dtype, int nranks) {
  return ((AdaptiveController*)c)->usePcie(makeOpKey(op, bytes, dtype, nranks, 0)) ? 1 : 0;
}
size_t hlCtlDump(void* c, char* buf, size_t cap) {
  std::string s = ((AdaptiveController*)c)->dumpJson();
  if (buf && cap > s.size()) memcpy(buf, s.c_str(), s.size() + 1);
  return s.size() + 1;
}
int hlCtlLoad(void* c, const char* text) { return ((AdaptiveController*)c)->loadJson(text ? text : "") ? 0 : 1; }
void hlPathTiming(double fs, double fe, double ps, double pe, double* out5) {
  PathTiming t = computePathTiming(fs, fe, ps, pe);
  out5[0] = t.fast;
  out5[1] = t.pcie;
  out5[2] = t.overlap;
  out5[3] = t.span;
  out5[4] = t.parallel_efficiency;
}
}
