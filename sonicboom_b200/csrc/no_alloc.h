// sb_attention_decode_static: decode attention for callers that must not allocate.
//
// This entry point has no counterpart in hardenedlinux/SonicBoom; it exists for users of this
// library who call the attention kernel from a place where device memory cannot be obtained:
// a host thread that runs inside a region where cudaMalloc is forbidden or would stall (a
// real-time loop, a callback of another framework that owns the allocator, a process whose
// memory budget was handed out in full at start-up).  The ordinary entry point, sb_attention,
// asks its caller for scratch memory whenever a sequence is long enough to be cut into more
// than one split (256 keys, 512 in long sequences); such a caller has nowhere to get it from.
//
// Here the scratch is a fixed array inside the library's own device image
// (SB_STATIC_SCRATCH_BYTES, 8 MiB per GPU that loads the library, held until the process
// exits).  The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library
// routine.  Inputs and outputs are still the caller's.
//
// Limits and rules:
//  * Decode steps only: new rows per sequence x (query heads / key-value heads) <= 16.
//  * The step must need at most SB_STATIC_SCRATCH_BYTES of scratch, i.e.
//    rows x query heads x splits x (head size + 4) x 4 bytes, with splits = ceil(max_len / 256)
//    up to 4,096 keys and max(16, ceil(max_len / 512)) beyond; larger steps are
//    refused with SB_ERR_UNSUPPORTED and a message that states both numbers.
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress,
//    with that device current) and remembers it; make that first call outside any stream
//    capture.
//  * At most 16384 (sequence, key/value head) pairs per step (the built-in merge counters).
//  * All calls on a device share the one array.  It keeps whatever the last call left in it;
//    this kernel writes every partial result before it reads it, so nothing needs clearing.
//    Two calls whose kernels overlap on the GPU (different streams, no ordering between them)
//    race on the array and corrupt each other's results: order them.
#pragma once

#include "sonicboom_b200.h"     /* sb_stream_t (the runtime's cudaStream_t) and the ordinary entry points */

#define SB_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// The arguments of sb_attention that describe the step, with the same meanings and results;
// what sb_attention takes besides them is not needed here: no scratch pointer and size, no
// merge counters and their count (both are inside the library), no n_pages and n_sms (this
// entry point runs decode steps only), no L2 hint.
int sb_attention_decode_static(const void* q, void* out, int n_rows, int n_seqs, int max_new,
                               const int32_t* seq_row0, const int32_t* seq_pos0,
                               const int32_t* page_off, const int32_t* page_ids, int page_size,
                               const void* cache, int n_q_heads, int n_kv_heads, int hd,
                               int window, float scale, int max_len, sb_stream_t stream);

// Bytes of the built-in scratch array (SB_STATIC_SCRATCH_BYTES).
size_t sb_attention_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
