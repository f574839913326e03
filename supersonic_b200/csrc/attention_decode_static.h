/* Decode attention without any allocation.
 *
 * This entry point has no counterpart in the reference.  It is for callers that cannot
 * allocate device memory at the moment they need attention: code that runs inside a region
 * where cudaMalloc is forbidden or would synchronise the device (a latency-critical serving
 * loop, a plug-in called from another framework's stream callback, a process whose memory
 * pool has been handed out in full), and that has no scratch buffer of its own to pass in.
 *
 * It computes exactly what ssb_attention_decode computes (one query token per sequence over
 * its paged keys and values, the keys split n_splits ways) but keeps the partial results of
 * the splits and their arrival counters in two arrays that are part of the library image:
 *
 *     SSB_STATIC_SCRATCH_FLOATS   float32 values  (8 MiB)
 *     SSB_STATIC_COUNTERS         int32 counters  (64 KiB)
 *
 * Every GPU on which the library is loaded holds these arrays until the process exits.
 * A call needs  n_seqs * n_q * n_splits * (head_dim + 2)  floats and
 * n_seqs * n_kv * ceil((n_q / n_kv) / 4)  counters; a call that needs more than the arrays
 * hold is refused with SSB_ERR_STATIC_SCRATCH_TOO_SMALL and launches nothing (use fewer
 * splits, or the entry point that takes a caller's scratch).
 *
 * The function calls no cudaMalloc, cudaFree or any other allocating routine.  The caller
 * passes inputs and outputs as device pointers, as for ssb_attention_decode.
 *
 * First call on a device: the addresses of the two arrays on the current device are looked
 * up once (cudaGetSymbolAddress) and remembered per device.  Make this first call, with the
 * device current, before any stream capture begins.  Several host threads that make their
 * first call on one device at the same moment each look the addresses up and store the same
 * two values: harmless, but nothing else about the first call is synchronised.
 *
 * Sharing: all calls on a device use the same arrays, which keep what the last call left.
 * The counters a call uses are cleared on its stream before its kernel runs.  Two calls
 * whose kernels overlap on the GPU (different streams, no ordering between them) race on
 * the arrays and give wrong results: order them.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSB_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define SSB_STATIC_COUNTERS (16 * 1024)
#define SSB_ERR_STATIC_SCRATCH_TOO_SMALL 2005

/* Returns 0, a cudaError_t of the set-up or the launch, SSB_ERR_STATIC_SCRATCH_TOO_SMALL, or
 * one of the size errors of ssb_attention_decode (2002, 2003). */
int ssb_attention_decode_static(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* pos, const int* slot, const int* page_table, int max_pages,
                                void* out, int ldo, int n_seqs, int n_q, int n_kv, int head_dim,
                                int page_shift, int window, float scale, int n_splits,
                                cudaStream_t stream);

/* The limits above, for callers that bind the symbol without this header. */
void ssb_attention_decode_static_limits(long long* scratch_floats, int* counters);

#ifdef __cplusplus
}
#endif
