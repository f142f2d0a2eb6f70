// Node scope: is every rank of a communicator a process (or thread) of THIS machine?
//
// The symbol layer sits under programs whose communicators may span nodes; only communicators that are confined
// to one machine get a side communicator. Every rank of a communicator registers itself — rank, pid, device,
// time — in a small shared-memory table named after the communicator's hash and this machine's identity (host
// name, user, boot id) and then looks, for a bounded time, whether all ranks have shown up there with live
// processes. Ranks on other machines write to THEIR machine's table, so they are never seen here.
//
// Parity: multipath-orchestrator/libampccl/core/node_scope.cc:84-108 (machine identity), :155-205 (table),
// :211-252 (liveness and age of entries, device layout), :256-318 (register, then resolve with a bounded wait).
#pragma once
#include <cstdint>

#include "hylink/hylink.h"

namespace hl {

struct NodeScope {
  int seen = 0;             // ranks found on this machine (live processes, fresh entries)
  bool all_local = false;   // seen == nranks
  bool distinct = false;    // no two ranks on one device
  bool contiguous = false;  // device of rank r == device of rank 0 + r
  uint64_t node_hash = 0;
};

// Registers (rank, pid, device) and waits up to wait_ms for the other ranks. Never fails hard: when shared memory
// is unavailable the result says "not all local".
NodeScope detectNodeScope(uint64_t comm_hash, int nranks, int rank, int device, int wait_ms);
// Drops this rank's entry (and the table with the last one).
void leaveNodeScope(uint64_t comm_hash, int nranks, int rank);
uint64_t localNodeHash();

}  // namespace hl
