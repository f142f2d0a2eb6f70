// Schedule IR: the declarative per-rank program that the CPU executor runs on
// the PCIe path. The XML file format is the reference's ("CPU-driven DSL"):
//
//   <ir_program name="allreduce" nranks="2" topology="..." [variant=".."] nnodes="1">
//     <rank id="0">
//       <instruction op="D2H|H2D|D2D|D2DReduce|H2H|H2HReduce|NOP"
//           [src_rank] [src_buf] [dst_buf] src_chunk [src_numa] dst_chunk [dst_numa]
//           [src1_chunk src1_numa src2_chunk src2_numa]/>
//
// with the same defaults (src_buf=input, dst_buf=output, src_rank=own rank,
// host chunks live on the executing rank's logical NUMA node unless a *_numa
// attribute says otherwise).
//
// Parity: data model of pcie-ccl-cuda/src/ir/ir.hpp:12-16,68-143,214-232 and
// loader of src/ir/ir_loader.cpp:16-163,247-334. New here: a writer and a
// generator that emits schedules for ANY gpu->NUMA pattern (the reference
// ships hand-written files for five patterns only, none of which matches an
// 8-GPU two-socket B200 board).
#pragma once
#include <string>
#include <vector>

#include "core/core.h"

namespace hl {
namespace ir {

constexpr int kMaxNodes = 1024;      // instructions per program (all ranks)
constexpr int kMaxChunks = 256;      // chunk indices per space
constexpr int kMaxNuma = 8;

enum class Op : uint8_t { NOP = 0, D2D, D2H, H2D, H2H, H2HReduce, D2DReduce };
enum class Buf : uint8_t { Input = 0, Output, Scratch, Internal, Host };

const char* opName(Op op);
const char* bufName(Buf b);

struct Instr {
  Op op = Op::NOP;
  int rank = 0;        // executing rank
  int src_rank = -1;   // D2D / D2DReduce: whose device buffer is read (-1 = own)
  Buf src_buf = Buf::Input, dst_buf = Buf::Output;
  int src_chunk = 0, dst_chunk = 0;
  int src_numa = -1, dst_numa = -1;              // -1 = the executing rank's NUMA node
  int src1_chunk = 0, src1_numa = -1, src2_chunk = 0, src2_numa = -1;  // H2HReduce
  int line = 0;
};

struct Program {
  std::string name;       // allreduce | allgather | reducescatter | alltoall | broadcast
  std::string topology;
  std::string variant;
  std::string description;
  int nranks = 0;
  int nnodes = 1;
  std::vector<std::vector<Instr>> ranks;  // program order inside each rank
  // derived by finalize()
  int input_chunks = 0;     // 1 + highest INPUT chunk read by anyone
  int output_chunks = 0;    // 1 + highest OUTPUT chunk written by anyone
  int internal_chunks = 0;  // 1 + highest INTERNAL chunk touched
  int scratch_chunks = 0;
  int host_chunks = 0;      // 1 + highest host chunk touched on any NUMA node
  int numa_nodes = 0;       // 1 + highest NUMA id named explicitly
  size_t instructions() const;
};

// Parses XML text; on error returns hlInvalidArgument with the line in the message.
hlResult_t parseProgram(const std::string& xml_text, Program* out);
hlResult_t loadProgramFile(const std::string& path, Program* out);
// Validates indices and fills the derived counts.
hlResult_t finalize(Program* p);
std::string toXml(const Program& p);

// "00001111": logical NUMA id of every GPU, concatenated.
std::string numaPattern(const std::vector<int>& gpu_numa);
std::vector<int> parsePattern(const std::string& pattern);

// Looks for <collective>_<pattern>[_variant].xml in: `extra_dir`, the
// configured IR path, and ./ir next to the library / package / working
// directory. Empty string when nothing matches.
std::string findProgramFile(const std::string& collective, const std::string& pattern, const std::string& variant,
                            const std::string& extra_dir);

// Emits a schedule for any pattern.
//   collective: allreduce | allgather | reducescatter | alltoall | broadcast
//   variant:    "" (device reduce on landing, writer-side placement)
//               "single_d2h" (one upload, readers cross NUMA)
//               "host_reduce" (all-reduce / reduce-scatter folded by the CPU with H2HReduce)
//               "small" (one host round trip, no pipelined sub-steps)
hlResult_t generate(const std::string& collective, const std::vector<int>& gpu_numa, const std::string& variant,
                    int root, Program* out);

}  // namespace ir
}  // namespace hl
