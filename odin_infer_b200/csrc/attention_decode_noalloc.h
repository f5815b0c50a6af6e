/* An entry point of this library that has no counterpart in the reference project.
 *
 * odin_attention_decode() needs scratch memory for the partial results of its key
 * splits, and its caller has to allocate that.  Some callers cannot allocate device
 * memory at the moment they need attention: a host program that handed all device
 * memory to an arena of its own at start-up, a plug-in that runs inside another
 * runtime's memory budget, or a latency-critical loop in which cudaMalloc (which may
 * synchronise the whole device) is forbidden.  For them this variant brings its
 * scratch with it: a fixed array in the library's device image.
 *
 * - It allocates nothing: no cudaMalloc, no cudaFree, no allocating library call.
 *   Inputs and outputs are still the caller's.
 * - The scratch is ODIN_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that loads
 *   the library holds that much until the process exits, whether or not this entry
 *   point is ever called.
 * - A call needs B * Hq * n_split * (hd + 2) floats.  More than the maximum is refused
 *   with ODIN_ERR_TOO_LARGE and nothing is launched; use fewer splits or the ordinary
 *   entry point with memory of your own.
 * - The first call on each device looks up the array's device address (with that
 *   device current).  Make that first call before any stream capture begins.
 * - The counters on which the key splits of a launch meet, and the library's error flag,
 *   are fixed arrays in the device image too (for every entry point of the library), so
 *   that this one stays free of allocations on every path.  Because of them the same rule
 *   holds for ALL decode-attention launches of a process, through whichever entry point: two
 *   launches that overlap on the GPU mix their arrivals on the counters.  Keep them in stream
 *   order.
 * - All calls share the one array.  Nothing in it has to be cleared between calls:
 *   each call writes every element it later reads.  But two calls that overlap on
 *   the GPU (different streams, no ordering between them) race on it; keep calls on
 *   one stream or order them yourself.
 *
 * Arguments and return codes are those of odin_attention_decode() without `scratch`.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ODIN_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define ODIN_ERR_TOO_LARGE (-4)

int odin_attention_decode_noalloc(const void* q, long long q_row_stride, void* out, long long out_row_stride, int B,
                                  int Hq, int Hkv, int hd, const void* k_cache, const void* v_cache, int page_size,
                                  int n_pages, const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride,
                                  int window, int n_split, void* stream);

/* The number of floats a call with these sizes needs (compare with the maximum above). */
long long odin_attention_decode_noalloc_need(int B, int Hq, int hd, int n_split);

#ifdef __cplusplus
}
#endif
