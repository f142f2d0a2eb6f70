// Plain-data structures shared by host code and the sm_100a kernels of the
// dedicated-link (NVLink 5 / NVSwitch) path.
#pragma once
#include <stdint.h>

#define HL_MAX_RANKS 8        // one NVSwitch domain of an HGX B200 board
#define HL_MAX_BLOCKS 592     // 148 SMs x 4 resident CTAs
#define HL_NVL_THREADS 512
#define HL_SEQ_STRIDE 4       // flag values consumed per collective call
#define HL_FLAG_KINDS 3       // 0: block barriers; 1, 2: tile hand-offs of the pipelined kernels
// Kernel timeline (off unless the communicator was created with it): a ring of the last HL_TL_CALLS launches, for
// the first HL_TL_BLOCKS CTAs of each, HL_TL_PHASES %globaltimer stamps: 0 entry, 2k-1 / 2k arrival at / release
// from the k-th cross-GPU barrier (k = 1..3), 7 exit. Behind the stamps, 4 words per call: flag base, kernel kind
// << 32 | CTAs, element count, 0.
#define HL_TL_CALLS 16
#define HL_TL_BLOCKS 148
#define HL_TL_PHASES 8
#define HL_TL_WORDS (HL_TL_CALLS * HL_TL_BLOCKS * HL_TL_PHASES + HL_TL_CALLS * 4)

// Device status codes written by a kernel whose bounded wait ran out.
#define HL_DEV_OK 0
#define HL_DEV_TIMEOUT 1
#define HL_DEV_ABORTED 2
#define HL_DEV_BOUNDS 3

// Per-communicator constants, resident in device memory. Every pointer table
// holds, for each rank q, the address at which THIS rank maps q's region
// (entry [rank] is the local region itself).
struct HlCommDev {
  int rank;
  int nranks;
  int max_blocks;
  int pad0;
  uint8_t* stage[HL_MAX_RANKS];    // symmetric staging region
  uint64_t* flags[HL_MAX_RANKS];   // [HL_FLAG_KINDS][HL_MAX_BLOCKS][HL_MAX_RANKS] monotonically increasing words
  uint8_t* mc_stage;               // NVSwitch multicast alias of stage (null without NVLS)
  uint64_t* status;                // host-visible: [0] code, [1] detail (step<<32 | peer), [2] block
  uint32_t* abort_word;            // device word: non-zero poisons the communicator
  uint64_t* seq_words;             // device words: [0] flag base of the next call, [1] tile base of the next pipelined
                                   // call, [2] CTAs of the running call that have finished
  uint64_t stage_bytes;
  uint64_t timeout_ns;
  uint64_t* timeline;              // device ring of HL_TL_WORDS words, null when the timeline is off
  // Registered (symmetric) user memory: every rank owns a heap of heap_bytes; buffers handed out by the library's
  // allocator lie at the same offset on every rank, so a kernel reaches a peer's buffer as heap[q] + offset and all
  // ranks' copies at once as mc_heap + offset. Null / 0 until the heap exists.
  uint8_t* heap[HL_MAX_RANKS];
  uint8_t* mc_heap;                // NVSwitch multicast alias of the heap (null without NVLS)
  uint64_t heap_bytes;
  // Low-latency region of the barrier-free kernels (nvl_ll_kernels.cu), behind the flag area of every rank:
  // [2 parities][2 phases][HL_MAX_RANKS sources] slots of ll_slot_bytes; null / 0 when the region does not exist.
  uint8_t* ll[HL_MAX_RANKS];
  uint64_t ll_slot_bytes;
};
// Behind the flag words of every rank sit [HL_MAX_RANKS][2] words in which peer q announces the heap offsets
// (in, out) of its buffers for the running zero-copy call; they must equal the local ones.
#define HL_ZC_ARGS_WORD_OFF ((size_t)HL_FLAG_KINDS * HL_MAX_BLOCKS * HL_MAX_RANKS)

// Per-call arguments (by value in the launch).
struct HlCallArgs {
  const void* in;
  void* out;
  uint64_t count;           // elements: AR/bcast total; AG/RS/A2A the handled prefix of one segment
  uint64_t in_seg_stride;   // elements between segments of `in`  (RS, A2A)
  uint64_t out_seg_stride;  // elements between segments of `out` (AG, A2A)
  uint64_t seq;             // flag base of this call (filled in on the device from seq_words); barrier k waits for seq + k
  float scale;              // applied to the reduced value (floating types)
  int op;                   // hlRedOp_t
  int in_dt;                // hlDataType_t of `in`
  int out_dt;               // hlDataType_t of `out`
  int root;
  int int_div;              // integer types: divide the sum (hlAvg), 0 = off
  uint64_t pipe_seq;        // pipelined kernels (filled in on the device): tile k of a block is announced as pipe_seq + k + 1
  uint64_t tile_packets;    // pipelined kernels: 16-byte packets of one shard handled per tile
  int kind;                 // HlNvlKernel, recorded in the kernel timeline
  int lane_parts;           // lane kernels (reduce-scatter, all-gather): HBM-side CTAs per pusher CTA (1..7)
  uint64_t zc_in_off;       // zero-copy kernels: heap offset of `in` (valid when the kernel reads `in` from peers)
  uint64_t zc_out_off;      // zero-copy kernels: heap offset of `out` (valid when the kernel writes peers' `out`)
};

// One argument block per emulated rank: on a single GPU the N ranks of a test
// run as ONE cooperative launch with gridDim.y == N (kernels that wait on one
// another must never be separate launches on one device).
struct HlEmuCalls {
  HlCallArgs c[HL_MAX_RANKS];
};

enum HlNvlKernel {
  kNvlBarrier = 0,
  kNvlAllReduceOneShot = 1,
  kNvlAllReduceTwoShot = 2,
  kNvlAllReduceNvls = 3,
  kNvlReduceScatter = 4,
  kNvlReduceScatterNvls = 5,
  kNvlAllGather = 6,
  kNvlBroadcast = 7,
  kNvlAllToAll = 8,
  kNvlAllGatherNvls = 9,
  kNvlBroadcastNvls = 10,
  kNvlAllReducePipeP2p = 11,
  kNvlAllReducePipeNvls = 12,
  kNvlReduceScatterPipeP2p = 13,
  kNvlReduceScatterPipeNvls = 14,
  kNvlAllReducePush = 15,
  kNvlReduceScatterPush = 16,
  kNvlAllGatherPush = 17,
  kNvlAllGatherLanes = 18,
  // zero-copy kernels on registered memory: peers' buffers are read / written in place, nothing is staged
  kNvlZcAllReduceNvls = 19,
  kNvlZcAllReduceP2p = 20,
  kNvlZcReduceScatterNvls = 21,
  kNvlZcReduceScatterP2p = 22,
  kNvlZcAllGatherNvls = 23,
  kNvlZcAllGatherP2p = 24,
  kNvlZcBroadcastNvls = 25,
  kNvlZcBroadcastP2p = 26,
  // barrier-free kernels for small messages: every 16-byte store carries its own arrival flag
  kNvlLlAllReduce = 27,
  kNvlLlReduceScatter = 28,
  kNvlLlAllGather = 29,
  kNvlLlAllToAll = 30,
};
#define HL_DEV_ASYMMETRIC 4   // zero-copy call whose buffers do not sit at the same heap offset on every rank
