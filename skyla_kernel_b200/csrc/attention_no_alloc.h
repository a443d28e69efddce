// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (maulanasdqn/skyla-kernel
// keeps all of its buffers in one arena that its engine plans up front,
// skyla-engine/src/arena.rs:83-181, and never hands a kernel to a foreign caller).
//
// Who needs it: code that wants this library's split-context decode attention but
// runs where cudaMalloc is off limits -- inside another runtime's stream capture or
// graph replay, in a real-time loop whose memory is fixed at start-up, or in a host
// process that only received device pointers from somebody else's allocator and has
// no allocator of its own to ask.  skyla_attention_decode() needs a float scratch
// buffer from its caller for the partial results of its blocks; this variant brings its
// own: one fixed array of SKYLA_NO_ALLOC_SCRATCH_FLOATS floats that lives in the
// library's device image (so every GPU that loads the library holds those 8 MiB
// until the process exits), and beside it SKYLA_NO_ALLOC_COUNTERS small counters
// (16 KiB) with which the blocks of one launch find out which of them finishes
// last, and the launch's plan (which pages each of its blocks reads: 32 bytes for
// each of up to SKYLA_NO_ALLOC_BLOCKS blocks and 8 bytes for each of up to
// SKYLA_NO_ALLOC_ITEMS (sequence, key/value head) pairs, written by a small kernel
// of its own before the attention kernel).  All three are this entry point's own: an engine
// of this library that runs on the same GPU brings its own scratch, counters and
// plans and shares nothing with it.
// It calls no cudaMalloc, no cudaFree and no other routine that allocates, on the
// host or on the device.
//
// Rules for callers:
//  * The problem must fit: skyla_attention_decode_scratch_floats(), that is
//    (n_blocks + n_seqs * nkv) * (nq / nkv) * (hd + 2) + 2 * n_seqs * nkv floats of
//    scratch, must not exceed SKYLA_NO_ALLOC_SCRATCH_FLOATS, n_blocks must not
//    exceed SKYLA_NO_ALLOC_BLOCKS and n_seqs * nkv must not exceed
//    SKYLA_NO_ALLOC_ITEMS; otherwise the call fails with a message and
//    launches nothing.  n_blocks is how many blocks share the step's pages: about
//    two per SM keep the memory busy; fewer when the whole step has few pages.
//  * The first call on a device looks up the arrays' device addresses
//    (cudaGetSymbolAddress, with that device current) and remembers them.  Make that
//    first call outside any stream capture.
//  * All calls on a device share the arrays, and they keep whatever the last call
//    left in them.  Nothing in the float array has to start at zero -- each call writes
//    every slot that its merge step reads -- and the counters are back at zero when a
//    call's kernel ends.  But two calls that overlap on the GPU (different streams, or
//    one stream capture replayed concurrently with another call) race on all three.  Order
//    them on one stream or with events.
//  * With more than SKYLA_NO_ALLOC_COUNTERS (sequence, key/value head) pairs the
//    pieces of a pair that different blocks read are merged by a second small kernel
//    instead of inside the first; the result is the same.
//  * Inputs and outputs are still the caller's: q, out, the cache pools, the page
//    lists and the positions, exactly as for skyla_attention_decode().
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define SKYLA_NO_ALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u) /* 8 MiB */
#define SKYLA_NO_ALLOC_COUNTERS 4096 /* 16 KiB */
#define SKYLA_NO_ALLOC_BLOCKS 1024 /* 32 KiB of plan */
#define SKYLA_NO_ALLOC_ITEMS 16384 /* 128 KiB of plan */

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as skyla_attention_decode() without the scratch and the plan.
// Returns 0, or a negative code whose text skyla_error_message() gives.
int skyla_attention_decode_no_alloc(const void* q, int64_t ldq, void* out, int64_t ldo, int n_seqs, int nq,
                                    int nkv, int hd, const void* k_pool, const void* v_pool,
                                    const int32_t* pages, int max_pages, int page_size,
                                    const int32_t* tok_pos, float scale, int window, int n_blocks,
                                    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
