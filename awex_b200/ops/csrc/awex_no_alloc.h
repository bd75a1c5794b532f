// Allocation-free launch of the fused transfer kernel.
//
// This entry point has no counterpart in the reference project.
//
// Who needs it.  The regular launcher takes its descriptor table, arrival
// counter and status words as device buffers, which its callers obtain from an
// allocator.  Some callers cannot allocate device memory at the moment they must
// move weights: a weight update that runs inside an inference server after the
// server has handed almost all of the GPU to its KV cache, so that a fresh
// cudaMalloc may fail or force the server to shrink its pools; a server whose
// caching allocator is asleep while its memory is lent to the trainer; a plug-in
// called from a thread in which the host framework's allocator must not be
// entered.  For them the library itself holds the scratch memory, in a
// file-scope device array that exists from the moment a GPU loads the library
// until the process exits.
//
// Cost.  Every GPU that loads the library carries the array:
// AWEX_NO_ALLOC_SCRATCH_BYTES (256 KiB + 256 B), whether or not this entry point
// is ever called.
//
// Contract.
//  * `host_descs` points to `n_desc` descriptors (xfer_desc.h, 128 bytes each) in
//    HOST memory, tiled exactly as for the regular launcher (`n_tiles` tiles in
//    total).  The source and destination addresses inside them are the caller's
//    own device buffers; the call copies the table into the library's scratch.
//    If the table lives in pinned memory it must stay unchanged until the work
//    queued on `stream` by this call has run.
//  * The table is checked on the host before anything is queued: tile numbering
//    (`tile_begin` starts at 0 and continues the running count, `n_tiles` equals
//    the total), non-zero tile geometry that matches the slab, the alignment and
//    stage-size rules of slabs flagged for bulk copies, and that `src`, `dst`, the
//    scale address of an fp8 slab, `row_table` and `tensor_map` are device
//    addresses (`row_table` and `tensor_map` may be 0).  An encoder's raw output
//    holds indices in `row_table` and no tensor maps: gathered rows and tensor
//    maps must be given device addresses by the caller first.  A table that
//    fails is refused with cudaErrorInvalidValue and a message naming the
//    descriptor; nothing is launched.  The checks cannot see extents: that every
//    slab stays inside the caller's buffers remains the caller's promise.
//  * `n_desc` above AWEX_NO_ALLOC_MAX_DESCS is refused with cudaErrorInvalidValue
//    and a message; nothing is launched.  Split the table and call again.
//  * No flags are waited for or raised: the call is ordered by `stream` alone.
//  * `status_out`, if not null, receives the kernel's four status words (all
//    zero on success); the call then waits for `stream` before it returns.  With
//    a null `status_out` the call only queues work.
//  * `err`, if not null, receives a zero-terminated message of at most
//    `err_cap` bytes when the return value is not cudaSuccess.
//  * The call makes no cudaMalloc / cudaFree and uses no allocating library
//    routine.  The first call on each device looks up the device address of the
//    scratch array and sets the kernel's shared-memory attribute; make that first
//    call before any stream capture begins.
//  * All calls on one device share the one scratch array, which still holds the
//    previous call's table and status.  Each call clears the counter and status
//    words and overwrites the table, in stream order.  Two calls that overlap on
//    the GPU (different streams, no dependency) race on it: serialise them.
//
// Returns a cudaError_t value.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define AWEX_NO_ALLOC_MAX_DESCS 2048u
#define AWEX_NO_ALLOC_HEADER_BYTES 256u
#define AWEX_NO_ALLOC_SCRATCH_BYTES (AWEX_NO_ALLOC_HEADER_BYTES + AWEX_NO_ALLOC_MAX_DESCS * 128u)

#ifdef __cplusplus
extern "C" {
#endif

int awex_fused_transfer_no_alloc(const void* host_descs, uint32_t n_desc, uint64_t n_tiles, uint64_t timeout_ns, int grid,
                                 void* stream, int32_t* status_out, char* err, size_t err_cap);

#ifdef __cplusplus
}
#endif
