// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (11Aln0/ginfer); it exists for users of
// this library.  Who cannot allocate: code that runs where cudaMalloc is forbidden or fails by
// design, such as a host program that has handed all device memory to its own pools at start-up, a
// real-time loop that may not take the allocator's locks or its implicit device synchronisation,
// or a plug-in loaded into a process whose memory budget is fixed.  The regular entry point,
// gf_attn_decode, wants a scratch buffer from its caller when it splits the keys; such callers
// have nowhere to get one from.  gf_attn_decode_static brings its own: a fixed array in the
// library's device image.
//
// What to know before using it:
//  * The scratch is a file-scope device array of GF_ATTN_STATIC_SCRATCH_BYTES (4 MiB).  Every GPU
//    on which this library is loaded holds those bytes from load until the process exits, and
//    beside them the 256 KiB of completion counters that every split-KV call through scratch
//    uses, this entry point's and gf_attn_decode's alike (one counter per request and kv head).
//  * A call needs B * nh * splits * (head_dim + 2) * 4 bytes when splits > 1 (nothing when
//    splits == 1).  A call that needs more than the array holds is refused: the function returns
//    GF_ATTN_STATIC_TOO_LARGE, launches nothing, and gf_attn_decode_static_error() describes the
//    sizes.  Use fewer splits or gf_attn_decode with a buffer of your own.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and keeps it.  Make that first call outside of any stream capture.
//    The look-up is guarded by a lock: first calls from several threads may coincide.
//  * No call allocates or frees: no cudaMalloc, cudaFree, nor any library routine that does.
//  * All calls share the one array and it keeps what the last call left.  The kernel writes
//    every word it later reads, so nothing needs clearing.  Two calls that overlap on the GPU
//    (different streams, or one device used from two threads) race on it: serialise them.  The
//    completion counters are shared with gf_attn_decode when that is given a scratch buffer, so
//    a call here must not overlap such a call either (each call leaves the counters at zero;
//    a launch that fails midway may not, after which later calls would skip their merge).
//  * Inputs and outputs are the caller's, exactly as for gf_attn_decode.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define GF_ATTN_STATIC_SCRATCH_BYTES (4u << 20)
#define GF_ATTN_STATIC_TOO_LARGE (-8)

// Same arguments and result as gf_attn_decode, without the scratch pointer.
int gf_attn_decode_static(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                          const int* block_table, int table_stride, const int* cu_seqlens_q,
                          const int* positions, void* out, int B, int nh, int nkv, int page_size,
                          int window, float scale, int splits, void* stream);

// Text of the last refusal or set-up failure of gf_attn_decode_static on this thread ("" if none).
const char* gf_attn_decode_static_error(void);

#ifdef __cplusplus
}
#endif
