// Decode kernels for sm_100a: bandwidth-bound work for a handful of tokens per step.
//
//   ssb_skinny_gemm       out[b, n] = sum_k x[b, k] W[n, k] for b <= 64 rows, bfloat16 in, float32
//                         accumulation on the tensor cores (mma.sync); epilogues: store, add into
//                         the float32 residual, SwiGLU.  The decode projection for shapes the
//                         tcgen05 kernels refuse.
//                         Replaces the reference's cuBLAS GemmEx GEMV per projection
//                         (kernels/full_attention_bridge_4b_cuda.cu:4768-4813) and its separate
//                         rms_norm / swiglu / add kernels (full_attention_cuda.cuh:2826-2873,
//                         1995-2010; prefill_helpers_cuda.cuh:60-70).
//   ssb_attention_decode  one query token per sequence over its paged keys and values, all query
//                         heads of a kv head together, the keys split over several blocks whose
//                         partial results the last block to finish merges.  Replaces
//                         supersonic_qwen35_full_attention_decode_*_kernel, one warp per query
//                         head and two passes over the keys (full_attention_cuda.cuh:476-679).
//
// Softmax statistics, norms and all sums are float32.  No float atomics: every output element
// is produced by one thread in a fixed order, so results do not depend on scheduling.
#include "attention_decode.cuh"
#include "attention_decode_mma.cuh"
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------
// skinny GEMM
// ---------------------------------------------------------------------------------------
// A block owns 16*RM rows of W over all of K.  Its 8 warps take 32-wide chunks of K in turn;
// a lane loads 16 bytes (8 consecutive k) of two W rows per 16-row tile and 16 bytes of one x
// row per 8-row batch tile, and feeds them to mma.m16n8k16 with a k order permuted the same
// way on both sides (a dot product does not care).  Warps' partial sums meet in shared memory.
constexpr int SG_WARPS = 8;
constexpr int SG_THREADS = SG_WARPS * 32;
// chunks whose loads are issued before any is used: fewer for wide batches (registers)
__host__ __device__ constexpr int sg_unroll(int nb) { return nb >= 4 ? 1 : (nb == 2 ? 2 : 4); }

enum { SG_STORE = 0, SG_ACCUMULATE = 1, SG_SWIGLU = 2 };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int RM, int NB>
__global__ void __launch_bounds__(SG_THREADS)
skinny_gemm_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw,
                   void* __restrict__ out, int ldo, int out_is_f32, int n_rows, int N, int K, int mode) {
    extern __shared__ __align__(128) unsigned char adm_smem[];
    constexpr int ROWS = 16 * RM, COLS = 8 * NB, SG_UNROLL = sg_unroll(NB);
    float* red = reinterpret_cast<float*>(adm_smem);    // [SG_WARPS][ROWS][COLS]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = (int)blockIdx.x * ROWS;
    const int n_chunks = (K + 31) / 32;

    // The block's slab of W goes to L2 ahead of use (one bulk prefetch per row): all of it when
    // the whole matrix fits L2 comfortably, else only the head of each row (a full prefetch of a
    // large matrix by every resident block would evict itself).  Weights are written by no
    // kernel, so this may run while the predecessor (attention, a norm) still works.
    if (threadIdx.x < ROWS) {
        const bf16* row = W + (size_t)min(n0 + (int)threadIdx.x, N - 1) * ldw;
        const bool small = (size_t)N * K * 2 <= (size_t)64 << 20;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(small ? K * 2 : min(K * 2, 4096)) : "memory");
    }
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();                                     // x (and out) belong to the predecessor until here

    float acc[RM][NB][4];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    // rows this lane loads (clamped: rows past N are computed but never stored)
    const bf16* w_row[RM][2];
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        w_row[i][0] = W + (size_t)min(n0 + i * 16 + g, N - 1) * ldw;
        w_row[i][1] = W + (size_t)min(n0 + i * 16 + g + 8, N - 1) * ldw;
    }

    for (int c0 = warp; c0 < n_chunks; c0 += SG_WARPS * SG_UNROLL) {
        uint4 wa[SG_UNROLL][RM][2];
        uint4 xb[SG_UNROLL][NB];
#pragma unroll
        for (int u = 0; u < SG_UNROLL; ++u) {
            const int k = (c0 + u * SG_WARPS) * 32 + t * 8;
            const bool live = k < K;                               // K is a multiple of 8: all 8 or none
#pragma unroll
            for (int i = 0; i < RM; ++i) {
                wa[u][i][0] = live ? ldg_stream(w_row[i][0] + k) : make_uint4(0, 0, 0, 0);
                wa[u][i][1] = live ? ldg_stream(w_row[i][1] + k) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = j * 8 + g;
                xb[u][j] = (live && b < n_rows) ? *reinterpret_cast<const uint4*>(x + (size_t)b * ldx + k)
                                                : make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < SG_UNROLL; ++u)
#pragma unroll
            for (int i = 0; i < RM; ++i)
#pragma unroll
                for (int j = 0; j < NB; ++j) {
                    mma_bf16_16816(acc[i][j], wa[u][i][0].x, wa[u][i][1].x, wa[u][i][0].y, wa[u][i][1].y,
                                   xb[u][j].x, xb[u][j].y);
                    mma_bf16_16816(acc[i][j], wa[u][i][0].z, wa[u][i][1].z, wa[u][i][0].w, wa[u][i][1].w,
                                   xb[u][j].z, xb[u][j].w);
                }
    }

    // partial sums of the 8 warps meet in shared memory: red[warp][row][col]
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float* r = red + ((size_t)warp * ROWS + i * 16) * COLS + j * 8;
            r[(g) * COLS + 2 * t] = acc[i][j][0];
            r[(g) * COLS + 2 * t + 1] = acc[i][j][1];
            r[(g + 8) * COLS + 2 * t] = acc[i][j][2];
            r[(g + 8) * COLS + 2 * t + 1] = acc[i][j][3];
        }
    __syncthreads();
    // the warps' partial tiles are summed in place into red[0], in warp order
    for (int e = threadIdx.x; e < ROWS * COLS; e += SG_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < SG_WARPS; ++w) v += red[(size_t)w * ROWS * COLS + e];
        red[e] = v;
    }
    __syncthreads();

    if (mode == SG_SWIGLU) {
        // rows come as [8 gate | 8 up] per 16: out[b, n0/2 + j] = silu(gate_j) * up_j
        for (int e = threadIdx.x; e < (ROWS / 2) * COLS; e += SG_THREADS) {
            const int j = e % (ROWS / 2), b = e / (ROWS / 2);
            const int r_gate = (j / 8) * 16 + (j % 8), n_out = n0 / 2 + j;
            if (b >= n_rows || n0 + r_gate + 8 >= N) continue;
            const float gate = red[(size_t)r_gate * COLS + b], up = red[(size_t)(r_gate + 8) * COLS + b];
            ((bf16*)out)[(size_t)b * ldo + n_out] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
        }
        return;
    }
    for (int e = threadIdx.x; e < ROWS * COLS; e += SG_THREADS) {
        const int r = e % ROWS, b = e / ROWS;
        const int n = n0 + r;
        if (b >= n_rows || n >= N) continue;
        const float s = red[(size_t)r * COLS + b];
        const size_t o = (size_t)b * ldo + n;
        if (mode == SG_ACCUMULATE) ((float*)out)[o] += s;
        else if (out_is_f32) ((float*)out)[o] = s;
        else ((bf16*)out)[o] = __float2bfloat16_rn(s);
    }
}

template <int RM, int NB>
static int launch_skinny(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int out_is_f32,
                         int n_rows, int N, int K, int mode, int pdl, cudaStream_t stream) {
    constexpr int ROWS = 16 * RM, COLS = 8 * NB;
    const size_t smem = (size_t)(SG_WARPS * ROWS * COLS) * sizeof(float);
    auto kern = skinny_gemm_kernel<RM, NB>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return ssb_launch(kern, dim3((N + ROWS - 1) / ROWS), dim3(SG_THREADS), smem, stream, pdl != 0, x, ldx, W, ldw,
                      out, ldo, out_is_f32, n_rows, N, K, mode);
}

// x: bfloat16 [n_rows, K].  W: bfloat16 [N, K].  mode 0: out[b, n] (bfloat16 or float32); mode 1:
// out (float32) += ; mode 2: W's rows come as [8 gate | 8 up] per 16 and out (bfloat16,
// [n_rows, N/2]) = silu(gate) * up.  pdl: launch as a programmatic dependent of the kernel before
// it on the stream (weights are prefetched while that one ends).
SSB_API int ssb_skinny_gemm(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int out_dtype,
                            int n_rows, int N, int K, int mode, int pdl, cudaStream_t stream) {
    if (n_rows <= 0 || N <= 0) return 0;
    if (n_rows > 64 || K <= 0 || K % 8 || ldw % 8 || ldx % 8) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)x | (uintptr_t)W) & 15) return SSB_ERR_BAD_SIZE;
    if (mode == SG_ACCUMULATE && out_dtype != SSB_F32) return SSB_ERR_BAD_DTYPE;
    if (mode == SG_SWIGLU && (out_dtype != SSB_BF16 || N % 16)) return SSB_ERR_BAD_SIZE;
    const int f32o = out_dtype == SSB_F32;
    const bf16* xb = (const bf16*)x;
    const bf16* Wb = (const bf16*)W;
#define SSB_SG(RM, NB) return launch_skinny<RM, NB>(xb, ldx, Wb, ldw, out, ldo, f32o, n_rows, N, K, mode, pdl, stream)
    if (n_rows <= 8) { SSB_SG(1, 1); }
    if (n_rows <= 16) { SSB_SG(2, 2); }
    if (n_rows <= 32) { SSB_SG(2, 4); }
    SSB_SG(2, 8);
#undef SSB_SG
}

// ---------------------------------------------------------------------------------------
// decode attention, keys split over blocks (kernel in attention_decode.cuh)
// ---------------------------------------------------------------------------------------
// Scratch: n_seqs * n_q * n_splits * (head_dim + 2) floats; counters: n_seqs * gridDim.y ints,
// zero before the first launch (every launch leaves them zero).  With cos_t/sin_t
// ([positions, head_dim/2] float32) the rows of q are the raw fused projection [q | k | v]: the
// kernel rotates queries and the token's key itself and appends key and value to the cache.
SSB_API long long ssb_attention_decode_scratch_floats(int n_seqs, int n_q, int head_dim, int n_splits) {
    return ad_scratch_floats(n_seqs, n_q, head_dim, n_splits);
}

SSB_API int ssb_attention_decode_counters(int n_seqs, int n_q, int n_kv) {
    return ad_counters(n_seqs, n_q, n_kv);
}

SSB_API int ssb_attention_decode(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                 const int* pos, const int* slot, const int* page_table, int max_pages,
                                 void* out, int ldo, int n_seqs, int n_q, int n_kv, int head_dim,
                                 int page_shift, int window, float scale, int n_splits, float* scratch,
                                 int* counters, int pdl, const float* cos_t, const float* sin_t,
                                 cudaStream_t stream) {
    return ad_launch(q, ldq, k_cache, v_cache, pos, slot, page_table, max_pages, out, ldo, n_seqs, n_q, n_kv,
                     head_dim, page_shift, window, scale, n_splits, scratch, counters, stream, pdl != 0,
                     cos_t, sin_t);
}

// The tensor-core kernel (attention_decode_mma.cuh): head sizes 64 and 128, at most 16 query heads
// per kv head, 64-token pages, at most 1,024 sequences.  chunk_pages and max_chunks: see adm_launch.
// Scratch: ssb_attention_decode_chunked_scratch_floats floats; counters: n_seqs * n_kv ints, zero
// before the first launch (every launch leaves them zero).  cache_rows: keys either cache has room for;
// error_word: a device int, zero, in which a page load that did not arrive in time is recorded.
// cluster: 0, or 2 / 4 / 8 chunks a sequence as the blocks of a thread-block cluster (see adm_launch).
SSB_API int ssb_attention_decode_chunked_ok(int n_seqs, int n_q, int n_kv, int head_dim, int ldq, int page_shift) {
    return page_shift == 6 && n_seqs <= ADM_MAX_SEQS && adm_supported(n_q, n_kv, head_dim, ldq, false);
}

// Blocks of the kernel that the device holds at once for this case (its persistent grid): callers size
// their chunks by it.
SSB_API long long ssb_attention_decode_chunked_blocks(int n_seqs, int n_q, int n_kv, int head_dim, int fused) {
    if (n_kv <= 0 || n_q % n_kv) return 0;
    return adm_resident_blocks(head_dim, fused != 0, n_q / n_kv, n_seqs);
}

// Clusters of ``cluster`` (2, 4, 8) blocks of the kernel that the device holds at once for this case: a
// caller that wants a sequence's chunks as a cluster needs sequences x kv heads of them.
SSB_API int ssb_attention_decode_chunked_clusters(int n_q, int n_kv, int head_dim, int fused, int cluster) {
    if (n_kv <= 0 || n_q % n_kv) return 0;
    return adm_max_clusters(head_dim, fused != 0, n_q / n_kv, cluster);
}

SSB_API long long ssb_attention_decode_chunked_scratch_floats(int n_seqs, int n_q, int head_dim, int max_chunks) {
    return adm_scratch_floats(n_seqs, n_q, head_dim, max_chunks);
}

SSB_API int ssb_attention_decode_chunked(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                         const int* pos, const int* slot, const int* page_table, int max_pages,
                                         void* out, int ldo, int n_seqs, int n_q, int n_kv, int head_dim,
                                         int page_shift, int window, float scale, int chunk_pages, int max_chunks,
                                         float* scratch, int* counters, int pdl, const float* cos_t,
                                         const float* sin_t, long long cache_rows, int* error_word, int cluster,
                                         cudaStream_t stream) {
    if (!ssb_attention_decode_chunked_ok(n_seqs, n_q, n_kv, head_dim, ldq, page_shift)) return SSB_ERR_UNSUPPORTED;
    return adm_launch(q, ldq, k_cache, v_cache, pos, slot, page_table, max_pages, out, ldo, n_seqs, n_q, n_kv,
                      head_dim, window, scale, chunk_pages, max_chunks, scratch, counters, stream, pdl != 0, cos_t,
                      sin_t, cache_rows, error_word, cluster);
}
