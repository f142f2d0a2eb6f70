// hlAllReduceLocalNoAlloc: see nvl/no_alloc.h for the contract.
//
// The staging regions, flag words, status words and the per-rank pointer
// tables that the regular emulated group obtains from cudaMalloc live here in
// one file-scope device array. Host code must never hand the array's NAME to a
// kernel: on the host that symbol is only a stand-in. Its device address is
// obtained once per device with cudaGetSymbolAddress and that pointer is what
// the launch receives.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "nvl/no_alloc.h"
#include "nvl/nvl_launch.h"

namespace {

constexpr size_t kMaxRanks = HL_NOALLOC_MAX_RANKS;
constexpr int kMaxBlocks = 16;                                  // CTAs per buffer this entry point ever uses
constexpr size_t kTableBytes = 512;                             // one HlCommDev, padded
constexpr size_t kTablesOff = 0;                                // [nranks 1..8][rank 0..7] pointer tables
constexpr size_t kTablesBytes = kMaxRanks * kMaxRanks * kTableBytes;
constexpr size_t kWordsOff = kTablesOff + kTablesBytes;         // per rank: status (64 B), poison word, sequence words
constexpr size_t kWordsBytes = kMaxRanks * 128;
constexpr size_t kFlagsOff = kWordsOff + kWordsBytes;           // per rank: kMaxBlocks x 8 flag words
constexpr size_t kFlagsPerRank = (size_t)kMaxBlocks * HL_MAX_RANKS * sizeof(uint64_t);
constexpr size_t kFlagsBytes = kMaxRanks * kFlagsPerRank;
constexpr size_t kStageOff = 64u << 10;                         // staging starts at 64 KiB
constexpr size_t kStagePerRank = HL_NOALLOC_MAX_BYTES;
constexpr size_t kScratchBytes = kStageOff + kMaxRanks * kStagePerRank;  // 2 MiB + 64 KiB
static_assert(kFlagsOff + kFlagsBytes <= kStageOff, "control words must fit below the staging area");
static_assert(sizeof(HlCommDev) <= kTableBytes, "pointer table slot too small");

// The scratch itself. Every GPU that loads this library holds it until exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_noalloc_scratch on this device
  bool ready = false;
};
PerDevice g_dev[64];
std::mutex g_mu;
int g_test_rows = 0;   // test aid: launch only the first k rows (the others never signal); 0 = all

// Once per device, with that device current: find the array and write the
// pointer tables (one per possible rank count) into it.
hlResult_t setUp(int device, unsigned char** base_out) {
  std::lock_guard<std::mutex> lk(g_mu);
  PerDevice& d = g_dev[device];
  if (!d.ready) {
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return hl::fail(hlDeviceError, "no-alloc all-reduce: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    for (size_t n = 1; n <= kMaxRanks; ++n) {
      HlCommDev tab[kMaxRanks];
      memset(tab, 0, sizeof(tab));
      for (size_t r = 0; r < n; ++r) {
        HlCommDev& c = tab[r];
        c.rank = (int)r;
        c.nranks = (int)n;
        c.max_blocks = kMaxBlocks;
        for (size_t q = 0; q < n; ++q) {
          c.stage[q] = ptr + kStageOff + q * kStagePerRank;
          c.flags[q] = reinterpret_cast<uint64_t*>(ptr + kFlagsOff + q * kFlagsPerRank);
        }
        c.mc_stage = nullptr;
        c.status = reinterpret_cast<uint64_t*>(ptr + kWordsOff + r * 128);
        c.abort_word = reinterpret_cast<uint32_t*>(ptr + kWordsOff + r * 128 + 64);
        c.seq_words = reinterpret_cast<uint64_t*>(ptr + kWordsOff + r * 128 + 80);  // three words, cleared with the flags
        c.stage_bytes = kStagePerRank;
        c.timeout_ns = 2000000000ull;  // 2 s: generous for a 256 KiB reduction, still bounded
      }
      // the launch indexes the table as an array of HlCommDev: pack the entries of this rank count contiguously
      e = cudaMemcpy(ptr + kTablesOff + (n - 1) * kMaxRanks * kTableBytes, tab, sizeof(HlCommDev) * n, cudaMemcpyHostToDevice);
      if (e != cudaSuccess) return hl::fail(hlDeviceError, "no-alloc all-reduce: writing the pointer tables failed: %s", cudaGetErrorString(e));
    }
    d.base = ptr;
    d.ready = true;
  }
  *base_out = d.base;
  return hlSuccess;
}

}  // namespace

extern "C" hlResult_t hlAllReduceLocalNoAlloc(int nranks, const void* const* ins, void* const* outs, size_t count,
                                              hlDataType_t dtype, hlRedOp_t op, hlStream_t stream) {
  const size_t es = hlTypeSize(dtype);
  if (!es) return hl::fail(hlInvalidArgument, "no-alloc all-reduce: unknown element type %d", (int)dtype);
  if (nranks < 2 || nranks > (int)kMaxRanks)
    return hl::fail(hlInvalidArgument, "no-alloc all-reduce: %d buffers requested, supported range is 2..%d", nranks, (int)kMaxRanks);
  if ((int)op < 0 || op >= hlNumOps) return hl::fail(hlInvalidArgument, "no-alloc all-reduce: bad reduction operator %d", (int)op);
  if (!ins || !outs) return hl::fail(hlInvalidArgument, "no-alloc all-reduce: null pointer list");
  if (count > kStagePerRank / es)   // compared without multiplying: count * es may wrap
    return hl::fail(hlInvalidArgument, "no-alloc all-reduce: %zu elements of %zu bytes per buffer exceed the fixed scratch of %zu bytes; use the regular group for larger messages",
                    count, es, (size_t)kStagePerRank);
  if (count == 0) return hlSuccess;
  for (int i = 0; i < nranks; ++i)
    if (!ins[i] || !outs[i]) return hl::fail(hlInvalidArgument, "no-alloc all-reduce: buffer %d is null", i);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= 64) return hl::fail(hlDeviceError, "no-alloc all-reduce: no current CUDA device");
  unsigned char* base = nullptr;
  hlResult_t r = setUp(device, &base);
  if (r != hlSuccess) return r;
  cudaStream_t s = (cudaStream_t)stream;
  // The previous call left its flag values (and possibly a poison word) behind: start from zero.
  e = cudaMemsetAsync(base + kWordsOff, 0, kWordsBytes + kFlagsBytes, s);
  if (e != cudaSuccess) return hl::fail(hlDeviceError, "no-alloc all-reduce: clearing the flag words failed: %s", cudaGetErrorString(e));
  HlEmuCalls calls;
  memset(&calls, 0, sizeof(calls));
  for (int i = 0; i < nranks; ++i) {
    HlCallArgs& a = calls.c[i];
    a.in = ins[i];
    a.out = outs[i];
    a.count = count;
    a.scale = op == hlAvg ? 1.0f / (float)nranks : 1.0f;
    a.op = op;
    a.in_dt = dtype;
    a.out_dt = dtype;
    a.int_div = op == hlAvg ? nranks : 0;
  }
  // one CTA per 16 KiB, never more than kMaxBlocks per buffer (all rows must be co-resident)
  int blocks = (int)((count * es + (16u << 10) - 1) / (16u << 10));
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  const HlCommDev* table = reinterpret_cast<const HlCommDev*>(base + kTablesOff + (size_t)(nranks - 1) * kMaxRanks * kTableBytes);
  const int rows = (g_test_rows > 0 && g_test_rows < nranks) ? g_test_rows : nranks;
  return hl::nvl::launch(kNvlAllReduceTwoShot, (int)dtype, table, calls, rows, blocks, s, nranks);
}

extern "C" hlResult_t hlAllReduceLocalNoAllocStatus(hlStream_t stream, int* code) {
  if (code) *code = HL_DEV_OK;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= 64) return hl::fail(hlDeviceError, "no-alloc all-reduce: no current CUDA device");
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev[device].ready) return hlSuccess;   // never called on this device: nothing can have gone wrong
    base = g_dev[device].base;
  }
  e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return hl::fail(hlDeviceError, "no-alloc all-reduce: stream synchronisation failed: %s", cudaGetErrorString(e));
  uint64_t words[kMaxRanks][16];   // 128 bytes per row: status words first
  e = cudaMemcpy(words, base + kWordsOff, sizeof(words), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return hl::fail(hlDeviceError, "no-alloc all-reduce: reading the status words failed: %s", cudaGetErrorString(e));
  for (size_t r = 0; r < kMaxRanks; ++r) {
    if (words[r][0] != HL_DEV_OK) {
      if (code) *code = (int)words[r][0];
      return hl::fail(hlTimeout, "no-alloc all-reduce: row %zu gave up waiting (step %llu, peer row %llu, CTA %llu); its outputs are incomplete",
                      r, (unsigned long long)(words[r][1] >> 32), (unsigned long long)(words[r][1] & 0xffffffffu), (unsigned long long)words[r][2]);
    }
  }
  return hlSuccess;
}

extern "C" void hlNoAllocSetActiveRowsForTest(int rows) { g_test_rows = rows; }
