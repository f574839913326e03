// Decode kernels for sm_100a: bandwidth-bound work for a handful of tokens per step.
//
//   ssb_skinny_gemm       out[b, n] = sum_k x[b, k] W[n, k] for b <= 64 rows, bfloat16 in, float32
//                         accumulation on the tensor cores; optional RMSNorm of a float32 input on
//                         the way in; epilogues: store, add into the float32 residual, SwiGLU.
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
// Launched as thread-block clusters, the blocks of a cluster share one row tile and split K: a
// matrix with few rows then still puts several blocks on every SM (bytes in flight are what a
// short projection lacks), and the partial tiles meet in the first block's shared memory over the
// cluster's distributed shared memory, in a fixed order.
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

__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int RM, int NB, bool NORM>
__global__ void __launch_bounds__(SG_THREADS)
skinny_gemm_kernel(const void* __restrict__ x_in, int ldx, const void* __restrict__ norm_w,
                   int norm_w_is_f32, float eps, const bf16* __restrict__ W, int ldw,
                   void* __restrict__ out, int ldo, int out_is_f32, int n_rows, int N, int K, int mode,
                   const void* __restrict__ post_w, int post_w_is_f32, float post_eps, bf16* __restrict__ post_out,
                   int* __restrict__ post_counter) {
    extern __shared__ __align__(128) unsigned char adm_smem[];
    float* smem = reinterpret_cast<float*>(adm_smem);
    constexpr int ROWS = 16 * RM, COLS = 8 * NB, SG_UNROLL = sg_unroll(NB);
    float* red = smem;                                  // [SG_WARPS][ROWS][COLS]
    float* inv_rms = smem + SG_WARPS * ROWS * COLS;     // [COLS] (NORM only)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_split = (int)cluster_size(), split = (int)cluster_rank();   // 1 and 0 without clusters
    const int n0 = ((int)blockIdx.x / n_split) * ROWS;
    const int n_chunks = (K + 31) / 32;
    const int per_split = (n_chunks + n_split - 1) / n_split;
    const int c_lo = split * per_split, c_hi = min(n_chunks, c_lo + per_split);

    // The block's slab of W goes to L2 ahead of use (one bulk prefetch per row): all of it when
    // the whole matrix fits L2 comfortably, else only the head of each row (a full prefetch of a
    // large matrix by every resident block would evict itself).  Weights are written by no
    // kernel, so this may run while the predecessor (attention, a norm) still works.
    if (threadIdx.x < ROWS) {
        const bf16* row = W + (size_t)min(n0 + (int)threadIdx.x, N - 1) * ldw;
        const bool small = (size_t)N * K * 2 <= (size_t)64 << 20;
        const int k_lo = min(c_lo * 32, K), k_n = min(c_hi * 32, K) - k_lo;      // multiples of 8 elements
        if (k_n > 0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row + k_lo), "r"(small ? k_n * 2 : min(k_n * 2, 4096)) : "memory");
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
    // NORM: x is the float32 residual.  RMSNorm's per-row scale factors out of the product,
    //   out[b, n] = rsqrt(mean_k x[b,k]^2 + eps) * sum_k (x[b,k] w[k]) W[n,k],
    // so the loop multiplies by the norm weight only and sums the squares on the side; every
    // x[b, k] passes through exactly one lane of the block, and the epilogue applies the scale.
    float ssq[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) ssq[j] = 0.f;

    for (int c0 = c_lo + warp; c0 < c_hi; c0 += SG_WARPS * SG_UNROLL) {
        uint4 wa[SG_UNROLL][RM][2];
        uint4 xb[SG_UNROLL][NB];
#pragma unroll
        for (int u = 0; u < SG_UNROLL; ++u) {
            const int k = (c0 + u * SG_WARPS) * 32 + t * 8;
            const bool live = k < K && c0 + u * SG_WARPS < c_hi;   // K is a multiple of 8: all 8 or none
#pragma unroll
            for (int i = 0; i < RM; ++i) {
                wa[u][i][0] = live ? ldg_stream(w_row[i][0] + k) : make_uint4(0, 0, 0, 0);
                wa[u][i][1] = live ? ldg_stream(w_row[i][1] + k) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = j * 8 + g;
                if (!live || b >= n_rows) {
                    xb[u][j] = make_uint4(0, 0, 0, 0);
                } else if (NORM) {
                    const float* xp = (const float*)x_in + (size_t)b * ldx + k;
                    const float4 v0 = *reinterpret_cast<const float4*>(xp);
                    const float4 v1 = *reinterpret_cast<const float4*>(xp + 4);
                    float w[8];
                    if (norm_w_is_f32) {
                        const float4 w0 = *reinterpret_cast<const float4*>((const float*)norm_w + k);
                        const float4 w1 = *reinterpret_cast<const float4*>((const float*)norm_w + k + 4);
                        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
                        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
                    } else {
                        const uint4 wq = *reinterpret_cast<const uint4*>((const bf16*)norm_w + k);
                        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wq);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(wp[e]);
                            w[2 * e] = f.x; w[2 * e + 1] = f.y;
                        }
                    }
                    ssq[j] = fmaf(v0.x, v0.x, ssq[j]); ssq[j] = fmaf(v0.y, v0.y, ssq[j]);
                    ssq[j] = fmaf(v0.z, v0.z, ssq[j]); ssq[j] = fmaf(v0.w, v0.w, ssq[j]);
                    ssq[j] = fmaf(v1.x, v1.x, ssq[j]); ssq[j] = fmaf(v1.y, v1.y, ssq[j]);
                    ssq[j] = fmaf(v1.z, v1.z, ssq[j]); ssq[j] = fmaf(v1.w, v1.w, ssq[j]);
                    xb[u][j].x = pack_bf16(v0.x * w[0], v0.y * w[1]);
                    xb[u][j].y = pack_bf16(v0.z * w[2], v0.w * w[3]);
                    xb[u][j].z = pack_bf16(v1.x * w[4], v1.y * w[5]);
                    xb[u][j].w = pack_bf16(v1.z * w[6], v1.w * w[7]);
                } else {
                    xb[u][j] = *reinterpret_cast<const uint4*>((const bf16*)x_in + (size_t)b * ldx + k);
                }
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
    if (NORM) {
        float* part = inv_rms + COLS;                   // [SG_WARPS][COLS]
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float v = ssq[j];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);    // the four lanes that share batch row g
            if (t == 0) part[warp * COLS + j * 8 + g] = v;
        }
    }
    __syncthreads();
    if (NORM) {
        if (threadIdx.x < COLS) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < SG_WARPS; ++w) v += inv_rms[COLS + w * COLS + threadIdx.x];
            inv_rms[threadIdx.x] = 1.0f / sqrtf(v / (float)K + eps);
        }
        __syncthreads();
    }

    // the warps' partial tiles are summed in place into red[0]; a cluster's tiles meet in its first block
    for (int e = threadIdx.x; e < ROWS * COLS; e += SG_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < SG_WARPS; ++w) v += red[(size_t)w * ROWS * COLS + e];
        red[e] = v;
    }
    if (n_split > 1) {
        cluster_sync_all();                             // every block's tile is complete
        if (split != 0) {
            cluster_sync_all();                         // stay until the first block has read it
            return;
        }
        for (int e = threadIdx.x; e < ROWS * COLS; e += SG_THREADS) {
            float v = red[e];
            for (int r = 1; r < n_split; ++r) v += ld_cluster_f32(red + e, (unsigned)r);
            red[e] = v;
        }
        cluster_sync_all();
    }
    __syncthreads();

    if (mode == SG_SWIGLU) {
        // rows come as [8 gate | 8 up] per 16: out[b, n0/2 + j] = silu(gate_j) * up_j
        for (int e = threadIdx.x; e < (ROWS / 2) * COLS; e += SG_THREADS) {
            const int j = e % (ROWS / 2), b = e / (ROWS / 2);
            const int r_gate = (j / 8) * 16 + (j % 8), n_out = n0 / 2 + j;
            if (b >= n_rows || n0 + r_gate + 8 >= N) continue;
            float gate = red[(size_t)r_gate * COLS + b], up = red[(size_t)(r_gate + 8) * COLS + b];
            if (NORM) { gate *= inv_rms[b]; up *= inv_rms[b]; }
            ((bf16*)out)[(size_t)b * ldo + n_out] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
        }
        return;
    }
    for (int e = threadIdx.x; e < ROWS * COLS; e += SG_THREADS) {
        const int r = e % ROWS, b = e / ROWS;
        const int n = n0 + r;
        if (b >= n_rows || n >= N) continue;
        float s = red[(size_t)r * COLS + b];
        if (NORM) s *= inv_rms[b];
        const size_t o = (size_t)b * ldo + n;
        if (mode == SG_ACCUMULATE) ((float*)out)[o] += s;
        else if (out_is_f32) ((float*)out)[o] = s;
        else ((bf16*)out)[o] = __float2bfloat16_rn(s);
    }
    if (post_out == nullptr) return;

    // RMSNorm of the finished rows, by the block that finishes last: out (float32, the residual
    // stream) is complete once every block has added its columns.  Saves the separate norm launch
    // between this projection and the next one.
    __shared__ int post_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(post_counter, 1);
        post_last = (arrived == (int)gridDim.x - 1);
        if (post_last) *post_counter = 0;               // ready for the next launch
    }
    __syncthreads();
    if (!post_last) return;
    __threadfence();
    const float* res = (const float*)out;
    for (int b = warp; b < n_rows; b += SG_WARPS) {     // a warp per row
        float ssq = 0.f;
        for (int k = lane * 4; k < N; k += 128) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(res + (size_t)b * ldo + k));
            ssq = fmaf(v.x, v.x, ssq); ssq = fmaf(v.y, v.y, ssq); ssq = fmaf(v.z, v.z, ssq); ssq = fmaf(v.w, v.w, ssq);
        }
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        const float inv = 1.0f / sqrtf(ssq / (float)N + post_eps);
        for (int k = lane * 4; k < N; k += 128) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(res + (size_t)b * ldo + k));
            float w0, w1, w2, w3;
            if (post_w_is_f32) {
                const float4 w = *reinterpret_cast<const float4*>((const float*)post_w + k);
                w0 = w.x; w1 = w.y; w2 = w.z; w3 = w.w;
            } else {
                const uint2 wq = *reinterpret_cast<const uint2*>((const bf16*)post_w + k);
                const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.x));
                const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.y));
                w0 = fa.x; w1 = fa.y; w2 = fb.x; w3 = fb.y;
            }
            uint2 packed;
            packed.x = pack_bf16(v.x * inv * w0, v.y * inv * w1);
            packed.y = pack_bf16(v.z * inv * w2, v.w * inv * w3);
            *reinterpret_cast<uint2*>(post_out + (size_t)b * N + k) = packed;
        }
    }
}

template <int RM, int NB, bool NORM>
static int launch_skinny(const void* x, int ldx, const void* norm_w, int norm_w_is_f32, float eps,
                         const bf16* W, int ldw, void* out, int ldo, int out_is_f32, int n_rows, int N,
                         int K, int mode, int pdl, const void* post_w, int post_w_is_f32, float post_eps,
                         bf16* post_out, int* post_counter, int k_split, cudaStream_t stream) {
    constexpr int ROWS = 16 * RM, COLS = 8 * NB;
    const size_t smem = (size_t)(SG_WARPS * ROWS * COLS + COLS + SG_WARPS * COLS) * sizeof(float);
    auto kern = skinny_gemm_kernel<RM, NB, NORM>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (k_split <= 1)
        return ssb_launch(kern, dim3((N + ROWS - 1) / ROWS), dim3(SG_THREADS), smem, stream, pdl != 0, x, ldx, norm_w,
                          norm_w_is_f32, eps, W, ldw, out, ldo, out_is_f32, n_rows, N, K, mode, post_w, post_w_is_f32,
                          post_eps, post_out, post_counter);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(((N + ROWS - 1) / ROWS) * k_split);
    cfg.blockDim = dim3(SG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = k_split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, x, ldx, norm_w, norm_w_is_f32, eps, W, ldw, out, ldo, out_is_f32,
                                       n_rows, N, K, mode, post_w, post_w_is_f32, post_eps, post_out, post_counter);
    return e == cudaSuccess ? ssb_launch_status() : (int)e;
}

// x: bfloat16 [n_rows, K] (norm_w == null) or the float32 residual [n_rows, K] normalised on the
// way in with norm_w (bfloat16 or float32) and eps.  W: bfloat16 [N, K].  mode 0: out[b, n]
// (bfloat16 or float32); mode 1: out (float32) += ; mode 2: W's rows come as [8 gate | 8 up] per
// 16 and out (bfloat16, [n_rows, N/2]) = silu(gate) * up.  pdl: launch as a programmatic
// dependent of the kernel before it on the stream (weights are prefetched while that one ends).
// post_out (mode 1 only): bfloat16 [n_rows, N] that receives RMSNorm(out; post_w, post_eps) of the
// finished rows, computed by the block that finishes last; post_counter: a zeroed int, left zero.
// k_split (1..8): blocks per cluster that share a row tile and split K (not with norm_w or post_out).
SSB_API int ssb_skinny_gemm(const void* x, int ldx, const void* norm_w, int norm_w_dtype, float eps,
                            const void* W, int ldw, void* out, int ldo, int out_dtype, int n_rows, int N,
                            int K, int mode, int pdl, const void* post_w, int post_w_dtype, float post_eps,
                            void* post_out, int* post_counter, int k_split, cudaStream_t stream) {
    if (n_rows <= 0 || N <= 0) return 0;
    if (k_split < 1 || k_split > 8 || (k_split > 1 && (norm_w || post_out))) return SSB_ERR_BAD_SIZE;
    if (n_rows > 64 || K <= 0 || K % 8 || ldw % 8 || ldx % 8) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)x | (uintptr_t)W | (uintptr_t)norm_w) & 15) return SSB_ERR_BAD_SIZE;
    if (mode == SG_ACCUMULATE && out_dtype != SSB_F32) return SSB_ERR_BAD_DTYPE;
    if (mode == SG_SWIGLU && (out_dtype != SSB_BF16 || N % 16)) return SSB_ERR_BAD_SIZE;
    const int f32o = out_dtype == SSB_F32, nwf = norm_w_dtype == SSB_F32, pwf = post_w_dtype == SSB_F32;
    if (post_out && (mode != SG_ACCUMULATE || !post_w || !post_counter || N % 4 || ldo % 4 ||
                     (((uintptr_t)post_w | (uintptr_t)post_out | (uintptr_t)out) & 15)))
        return SSB_ERR_BAD_SIZE;
    const bf16* Wb = (const bf16*)W;
#define SSB_SG(RM, NB) \
    return norm_w ? launch_skinny<RM, NB, true>(x, ldx, norm_w, nwf, eps, Wb, ldw, out, ldo, f32o, n_rows, N, K, mode, pdl, post_w, pwf, post_eps, (bf16*)post_out, post_counter, k_split, stream) \
                  : launch_skinny<RM, NB, false>(x, ldx, nullptr, 0, 0.f, Wb, ldw, out, ldo, f32o, n_rows, N, K, mode, pdl, post_w, pwf, post_eps, (bf16*)post_out, post_counter, k_split, stream)
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
// prefetch_ptr/bytes: read-only memory (the next kernels' weights) to pull into L2 meanwhile.
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
                                 const void* prefetch_ptr, long long prefetch_bytes, int kind,
                                 cudaStream_t stream) {
    // kind 0: the tensor-core kernel where it applies, else the general one; 1: general; 2: tensor-core
    const bool mma_ok = page_shift == 6 && adm_supported(n_q, n_kv, head_dim, ldq, cos_t != nullptr);
    if (kind == 2 && !mma_ok) return SSB_ERR_UNSUPPORTED;
    if (kind != 1 && mma_ok)
        return adm_launch(q, ldq, k_cache, v_cache, pos, slot, page_table, max_pages, out, ldo, n_seqs, n_q, n_kv,
                          head_dim, window, scale, n_splits, scratch, counters, stream, pdl != 0, cos_t, sin_t,
                          prefetch_ptr, prefetch_bytes);
    return ad_launch(q, ldq, k_cache, v_cache, pos, slot, page_table, max_pages, out, ldo, n_seqs, n_q, n_kv,
                     head_dim, page_shift, window, scale, n_splits, scratch, counters, stream, pdl != 0,
                     cos_t, sin_t, prefetch_ptr, prefetch_bytes);
}
