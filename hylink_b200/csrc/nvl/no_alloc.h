/*
 * An all-reduce entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference implementation.
 *
 * Who it is for: code that must not (or cannot) call cudaMalloc when it needs
 * a reduction across buffers that live on ONE GPU — a library running inside
 * someone else's memory budget where every byte is pre-assigned, a service
 * whose allocator is locked down after start-up, a region of a program in
 * which allocation would serialise the device (cudaMalloc synchronises) or is
 * forbidden by policy. The regular path (hlEmuCreate + hlEmuCollective)
 * allocates its staging and flag memory with cudaMalloc when the group is
 * created; this one keeps that scratch in a fixed array inside the library.
 *
 * What it does: sums (or max/min/prod) `nranks` equally sized buffers of one
 * device element-wise and writes the result to all `nranks` outputs — the same
 * two-shot all-reduce kernel the emulated group runs, one cooperative launch
 * with one grid row per buffer.
 *
 * Limits: 2 <= nranks <= 8 and count * sizeof(element) <= 256 KiB per buffer
 * (HL_NOALLOC_MAX_BYTES). Larger requests are refused with
 * hlInvalidArgument and a message in hlGetLastError(); nothing is launched.
 *
 * Cost: the scratch array (2 MiB + 64 KiB) is part of the library image, so
 * every GPU on which a process uses this library holds that much device memory
 * from module load until the process exits, whether or not this function is
 * ever called.
 *
 * Set-up: the first call on each device looks the array's device address up
 * and writes a small pointer table into it with synchronous copies. Make that
 * first call outside any stream capture; later calls only enqueue work on
 * `stream` (one memset of the flag words, one kernel launch).
 *
 * Errors on the device: every wait inside the kernel is bounded (2 s). A wait
 * that runs out makes the kernel record a status code in the scratch and
 * return with the outputs incomplete; the call that enqueued it has long
 * returned hlSuccess by then. hlAllReduceLocalNoAllocStatus() waits for
 * `stream` and reports that code; call it before trusting the outputs if a
 * silent failure matters to you, and before the next call on the device (which
 * clears the status words together with the flags).
 *
 * Sharing: all calls on a device use the same array, which still holds the
 * previous call's contents; the flag words are cleared on `stream` at the start
 * of every call. Two calls that can overlap on the GPU (different streams
 * without an ordering between them, or two threads) race on the scratch and
 * give wrong results: order them.
 */
#ifndef HYLINK_NVL_NO_ALLOC_H_
#define HYLINK_NVL_NO_ALLOC_H_

#include "hylink/hylink.h"

#define HL_NOALLOC_MAX_RANKS 8
#define HL_NOALLOC_MAX_BYTES (256u << 10) /* per buffer */

#ifdef __cplusplus
extern "C" {
#endif

/* ins / outs: `nranks` device pointers each (host arrays). The current device
 * must be the one that owns the buffers. Returns hlSuccess once the work is
 * enqueued on `stream`. */
hlResult_t hlAllReduceLocalNoAlloc(int nranks, const void* const* ins, void* const* outs, size_t count,
                                   hlDataType_t dtype, hlRedOp_t op, hlStream_t stream);

/* Waits for `stream`, then returns hlSuccess if the last call on the current
 * device ran to completion and hlTimeout (with *code = the device status, see
 * nvl_types.h, and a message in hlGetLastError()) if one of its bounded waits
 * ran out. Copies 1 KiB from the device into a stack buffer; allocates nothing. */
hlResult_t hlAllReduceLocalNoAllocStatus(hlStream_t stream, int* code);

/* Test aid: launch only the first `rows` grid rows of later calls (0 = all), so
 * that the rows which do run meet a peer that never signals and their bounded
 * wait runs out. Nothing faults or hangs; the call ends after the 2 s limit. */
void hlNoAllocSetActiveRowsForTest(int rows);

#ifdef __cplusplus
}
#endif
#endif
