// ssb_attention_decode_static: the split-key decode attention with its scratch inside the
// library image, for callers that cannot allocate (see attention_decode_static.h, which
// states who they are, the limits, and the rules on the first call and on overlapping calls).
// No counterpart in the reference.
#include "attention_decode.cuh"
#include "attention_decode_static.h"

// Partial results of the splits and arrival counters.  In host code these names are only
// handles for cudaGetSymbolAddress; the kernel gets the device addresses looked up below.
static __device__ __align__(256) float g_static_partials[SSB_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[SSB_STATIC_COUNTERS];

namespace {
constexpr int kMaxDevices = 64;
float* g_partials_on[kMaxDevices];      // device address of g_static_partials, per device
int* g_counters_on[kMaxDevices];

// Once per device, with that device current.
int lookup_for_current_device(int* device) {
    cudaError_t e = cudaGetDevice(device);
    if (e != cudaSuccess) return (int)e;
    if (*device < 0 || *device >= kMaxDevices) return SSB_ERR_UNSUPPORTED;
    if (g_partials_on[*device] && g_counters_on[*device]) return 0;
    float* partials = nullptr;
    int* counters = nullptr;
    e = cudaGetSymbolAddress((void**)&partials, g_static_partials);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress((void**)&counters, g_static_counters);
    if (e != cudaSuccess) return (int)e;
    g_partials_on[*device] = partials;
    g_counters_on[*device] = counters;
    return 0;
}
}  // namespace

SSB_API void ssb_attention_decode_static_limits(long long* scratch_floats, int* counters) {
    if (scratch_floats) *scratch_floats = SSB_STATIC_SCRATCH_FLOATS;
    if (counters) *counters = SSB_STATIC_COUNTERS;
}

SSB_API int ssb_attention_decode_static(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                        const int* pos, const int* slot, const int* page_table,
                                        int max_pages, void* out, int ldo, int n_seqs, int n_q, int n_kv,
                                        int head_dim, int page_shift, int window, float scale, int n_splits,
                                        cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    // every size the kernel refuses is refused here, before anything is enqueued
    if (head_dim <= 0 || head_dim > 32 * AD_MAX_VEC || n_kv <= 0 || n_q <= 0 || n_q % n_kv || n_splits < 1 ||
        n_splits > AD_MAX_SPLITS)
        return SSB_ERR_BAD_SIZE;
    // in 64 bits: a huge batch must not wrap into a small or negative figure
    const long long group_tiles = ((long long)(n_q / n_kv) + AD_GROUP - 1) / AD_GROUP;
    const long long need_floats =
        n_splits > 1 ? (long long)n_seqs * n_q * n_splits * ((long long)head_dim + 2) : 0;
    const long long need_counters = n_splits > 1 ? (long long)n_seqs * n_kv * group_tiles : 0;
    if (need_floats < 0 || need_counters < 0 || need_floats > SSB_STATIC_SCRATCH_FLOATS ||
        need_counters > SSB_STATIC_COUNTERS)
        return SSB_ERR_STATIC_SCRATCH_TOO_SMALL;
    int device = 0;
    const int rc = lookup_for_current_device(&device);
    if (rc) return rc;
    float* partials = g_partials_on[device];
    int* counters = g_counters_on[device];
    if (n_splits > 1) {
        // the arrays keep what the last call left: the counters this call uses start at zero
        cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)need_counters * sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    return ad_launch(q, ldq, k_cache, v_cache, pos, slot, page_table, max_pages, out, ldo, n_seqs, n_q, n_kv,
                     head_dim, page_shift, window, scale, n_splits, partials, counters, stream);
}
