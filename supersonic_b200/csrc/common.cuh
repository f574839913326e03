// Shared declarations of the sm_100a kernel libraries.
//
// Every library exports plain C entry points that take device pointers, sizes
// and a stream, launch on that stream and return the CUDA error code of the
// launch (0 = success), in the manner of the reference's bridges
// (kernels/full_attention_bridge_cuda.cu: `extern "C" int supersonic_*`).
// Nothing here allocates, synchronises or touches the default stream.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SSB_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum { SSB_F32 = 0, SSB_BF16 = 1 };

// status codes beyond cudaError_t (which stay below 1000)
enum {
    SSB_ERR_BAD_DTYPE = 2001,
    SSB_ERR_BAD_SIZE = 2002,
    SSB_ERR_UNSUPPORTED = 2003,
    SSB_ERR_TIMEOUT = 2004,
};

static inline int ssb_launch_status() { return (int)cudaGetLastError(); }

__device__ __forceinline__ float ssb_to_float(float x) { return x; }
__device__ __forceinline__ float ssb_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T ssb_from_float(float x);
template <> __device__ __forceinline__ float ssb_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 ssb_from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Location of token `pos` of sequence slot `slot` in a paged cache entry laid out as
// [page][kv_head][token_in_page][head_dim]; returns the element offset of the head's row.
__device__ __forceinline__ size_t ssb_cache_row(const int* __restrict__ page_table, int max_pages,
                                                int slot, int pos, int page_shift, int n_kv_heads,
                                                int kv_head, int head_dim) {
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    const size_t tok = ((size_t)page * n_kv_heads + kv_head) << page_shift;
    return (tok + (size_t)(pos & ((1 << page_shift) - 1))) * (size_t)head_dim;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor still runs.  Before ssb_pdl_wait() it must only read memory that no kernel of
// the chain writes (weights); after it, everything the predecessor wrote is visible.
// Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void ssb_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void ssb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with or without the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
static inline int ssb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
