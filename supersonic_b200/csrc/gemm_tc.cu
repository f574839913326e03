// Prefill GEMM for sm_100a: C[M, N] = A[M, K] W[N, K]^T, bfloat16 in, float32 accumulators in
// tensor memory.  One 128 x BN output tile per block, or one 256 x 256 tile per pair of blocks on
// neighbouring SMs (tcgen05 cta_group::2, further down); operands arrive through TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared-memory stages; one elected
// thread issues tcgen05.mma (M 128, N BN, K 16 per instruction); tcgen05.commit hands stages
// back and announces the finished accumulators; four warps read them with tcgen05.ld and write
// the result: plain store, add into the float32 residual, or SwiGLU over [8 gate | 8 up] columns.
//
// Replaces the reference's scalar 16x16 tiled matmul used for every prefill projection
// (kernels/full_attention_4b_cuda.cuh:2671-2743, launcher full_attention_bridge_4b_cuda.cu:3567-3613)
// and its separate element_add / swiglu kernels (prefill_helpers_cuda.cuh:60-70;
// full_attention_cuda.cuh:1995-2010).
//
// Every wait on an mbarrier is bounded: when one runs out, the block records a code in the
// caller's error word, lets its copies land, frees its tensor memory and returns.
#include "common.cuh"
#include "tc_helpers.cuh"

typedef __nv_bfloat16 bf16;

constexpr int TC_BM = 128;
constexpr int TC_TILE_PAIR = 512;         // tile_n value that asks for 256 x 256 tiles on SM pairs
constexpr int TC_THREADS = 192;           // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

// ---- kernel ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Mode rope-and-append: the product is the fused query/key/value projection of packed tokens.  The
// epilogue rotates query and key heads by each token's position (float32 tables, pairs d and
// d + head_dim/2, from the float32 accumulators: one rounding), writes the queries as bfloat16
// into C, and the keys and values straight into the paged cache; C's key and value columns are
// not written.  Replaces the separate rope + append launch after the projection of a prompt
// (reference: kernels/prefill_helpers_cuda.cuh:80-111, certified_kv_bridge_cuda.cu:32-51).
struct TcRope {
    const int* pos;            // [M] position of each row's token
    const int* slot;           // [M] cache slot of each row's token
    const int* page_table;     // [slots, max_pages]
    __nv_bfloat16* k_cache;    // [pages, n_kv, page tokens, head_dim]
    __nv_bfloat16* v_cache;
    const float* cos_t;        // [positions, head_dim / 2]
    const float* sin_t;
    int max_pages, n_q, n_kv, head_dim, page_shift;
};

__device__ __forceinline__ void tc_store32_bf16(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        uint4 u;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
        u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
        *reinterpret_cast<uint4*>(dst + j) = u;
    }
}

// One warp's share of a finished tile: tensor-memory lanes 32 * quarter .. + 31 (rows of the
// tile; ``row`` is this thread's row of C) and BN accumulator columns from column address ``acc``.
template <int BN>
__device__ __forceinline__ void tc_epilogue(uint32_t acc, int quarter, int row, int n0, int M, int N, void* __restrict__ C,
                                            int ldc, int out_is_f32, int mode, bool part, const TcRope& rope) {
    if (mode == TC_ROPE_APPEND) {
        // a head at a time: its low and high halves meet in this thread (the row's token)
        const int hd = rope.head_dim, half = hd / 2, halves32 = half / 32;
        const bool live = row < M;
        const int p = live ? rope.pos[row] : 0, sl = live ? rope.slot[row] : -1;
        size_t tok = 0;
        if (sl >= 0) {
            const int page = rope.page_table[(size_t)sl * rope.max_pages + (p >> rope.page_shift)];
            tok = (((size_t)page * rope.n_kv) << rope.page_shift) + (size_t)(p & ((1 << rope.page_shift) - 1));
        }
        for (int hh = 0; hh * hd < BN && n0 + hh * hd < N; ++hh) {
            const int head = (n0 + hh * hd) / hd;
            const bool is_q = head < rope.n_q, is_v = head >= rope.n_q + rope.n_kv;
            const int kvh = is_q ? 0 : (is_v ? head - rope.n_q - rope.n_kv : head - rope.n_q);
            bf16* dst = is_q ? (bf16*)C + (size_t)row * ldc + (size_t)head * hd
                             : (is_v ? rope.v_cache : rope.k_cache) +
                                   (tok + ((size_t)kvh << rope.page_shift)) * hd;
#pragma unroll 1
            for (int pc = 0; pc < halves32; ++pc) {
                uint32_t lo_r[32], hi_r[32];
                const uint32_t at = acc + ((uint32_t)(quarter * 32) << 16) + hh * hd + pc * 32;
                tc_ld32(at, lo_r);                       // every lane takes part in the loads
                tc_ld32(at + half, hi_r);
                if (!live || sl < 0) continue;
                float lo[32], hi[32];
                if (is_v) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) { lo[e] = __uint_as_float(lo_r[e]); hi[e] = __uint_as_float(hi_r[e]); }
                } else {
                    const float4* c4 = reinterpret_cast<const float4*>(rope.cos_t + (size_t)p * half + pc * 32);
                    const float4* s4 = reinterpret_cast<const float4*>(rope.sin_t + (size_t)p * half + pc * 32);
#pragma unroll
                    for (int i4 = 0; i4 < 8; ++i4) {
                        const float4 c = c4[i4], sn = s4[i4];
#define TC_ROTATE(e, cv, sv)                                                                         \
    {                                                                                                \
const float a_ = __uint_as_float(lo_r[4 * i4 + e]), b_ = __uint_as_float(hi_r[4 * i4 + e]);  \
lo[4 * i4 + e] = a_ * cv - b_ * sv;                                                          \
hi[4 * i4 + e] = a_ * sv + b_ * cv;                                                          \
    }
                        TC_ROTATE(0, c.x, sn.x) TC_ROTATE(1, c.y, sn.y) TC_ROTATE(2, c.z, sn.z) TC_ROTATE(3, c.w, sn.w)
#undef TC_ROTATE
                    }
                }
                tc_store32_bf16(dst + pc * 32, lo);
                tc_store32_bf16(dst + half + pc * 32, hi);
            }
        }
    } else
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tc_ld32(acc + ((uint32_t)(quarter * 32) << 16) + c * 32, r);
            const int n = n0 + c * 32;
            if (row >= M || n >= N) continue;
            if (mode == TC_SWIGLU) {
                bf16* dst = (bf16*)C + (size_t)row * ldc + n / 2;
                uint32_t packed[8];
    #pragma unroll
                for (int g = 0; g < 2; ++g)
    #pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float g0 = __uint_as_float(r[g * 16 + j]), u0 = __uint_as_float(r[g * 16 + 8 + j]);
                        const float g1 = __uint_as_float(r[g * 16 + j + 1]), u1 = __uint_as_float(r[g * 16 + 9 + j]);
                        __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.0f + __expf(-g0)) * u0,
                                                                  g1 / (1.0f + __expf(-g1)) * u1);
                        packed[g * 4 + j / 2] = *reinterpret_cast<uint32_t*>(&v);
                    }
                if (n + 32 <= N) {
                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                } else {
                    for (int j = 0; j < 16; ++j)            // N is a multiple of 16: whole groups only
                        if (n + (j / 8) * 16 + 16 <= N) dst[j] = reinterpret_cast<bf16*>(packed)[j];
                }
            } else if (out_is_f32) {
                float* dst = (float*)C + (size_t)row * ldc + n;
                if (n + 32 <= N) {
    #pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                               __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        if (part) { atomicAdd(reinterpret_cast<float4*>(dst + j), v); continue; }
                        if (mode == TC_ACCUMULATE) {
                            const float4 o = *reinterpret_cast<const float4*>(dst + j);
                            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                        }
                        *reinterpret_cast<float4*>(dst + j) = v;
                    }
                } else {
                    for (int j = 0; j < 32 && n + j < N; ++j) {
                        if (part) atomicAdd(dst + j, __uint_as_float(r[j]));
                        else dst[j] = __uint_as_float(r[j]) + (mode == TC_ACCUMULATE ? dst[j] : 0.f);
                    }
                }
            } else {
                bf16* dst = (bf16*)C + (size_t)row * ldc + n;
                if (n + 32 <= N) {
    #pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 v;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                        v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                        v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(dst + j) = v;
                    }
                } else {
                    for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                }
            }
        }
}

// Order of the tiles: bands of ``group_m`` row tiles; inside a band the row tile runs fastest, then
// the column tile.  The tiles that run at one time then share few rows of A and few of W, whatever
// M is (with all row tiles in one band, a wave of a long prompt touches all of A).
struct TcTileAt {
    int m, n;
    __device__ TcTileAt(int tile, int m_tiles, int n_tiles, int group_m) {
        const int band = tile / (group_m * n_tiles), in_band = tile - band * group_m * n_tiles;
        const int rows = min(group_m, m_tiles - band * group_m);
        m = band * group_m + in_band % rows;
        n = in_band / rows;
    }
};

struct TcItem {
    int tile, kb_lo, kb_hi;
    __device__ TcItem(int item, int n_tiles, int k_blocks, int splits) {
        tile = item % n_tiles;
        const int part = item / n_tiles, per = (k_blocks + splits - 1) / splits;
        kb_lo = min(part * per, k_blocks);
        kb_hi = min(kb_lo + per, k_blocks);
    }
};

// Persistent: a block takes tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulators of
// consecutive tiles alternate between two regions of tensor memory, so that the epilogue of one
// tile (tcgen05.ld, conversion, stores) runs while the MMAs of the next are issued.
//
// splits > 1 (float32 output, mode accumulate): a prompt of a few hundred tokens has fewer output
// tiles than the GPU has SMs, and the few blocks cannot pull the weights at the memory's rate.
// The K range of every tile is then cut into ``splits`` parts, each a work item of its own, and
// the parts add into the output with float atomics.
template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               void* __restrict__ C, int ldc, int out_is_f32, int M, int N, int K, int mode, int m_tiles,
               int n_tiles_total, int splits, int* __restrict__ error_word, const TcRope rope) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr int N_ACC = 2;                                        // accumulator regions (2 x BN <= 512 columns)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 2 * N_ACC);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);     // [0]: a role gave up; [1]: stays zero
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + N_ACC);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < N_ACC; ++i) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, 4); }
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {      // the whole warp allocates the accumulator columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(N_ACC * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int c = 0, issued_from = 0;                        // k-blocks issued so far (ring position)
            for (int item = blockIdx.x; item < n_tiles_total * splits && !*abort_flag; item += gridDim.x) {
                const TcItem it(item, n_tiles_total, k_blocks, splits);
                const int m0 = (it.tile % m_tiles) * TC_BM, n0 = (it.tile / m_tiles) * BN;
                for (int kb = it.kb_lo; kb < it.kb_hi; ++kb, ++c) {
                    const int s = c % STAGES;
                    const uint32_t phase = (c / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, phase ^ 1, abort_flag)) {
                        *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_PRODUCER); break;
                    }
                    const uint32_t a_dst = smem_u32(smem + s * STAGE_BYTES), w_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * TC_BK, m0);
                    tma_load_2d(w_dst, &map_w, full0 + 8 * s, kb * TC_BK, n0);
                }
            }
            if (*abort_flag) {
                // let copies that were issued but never consumed land before the block ends
                issued_from = max(0, c - STAGES);
                for (int i = issued_from; i < c; ++i)
                    mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, abort_flag + 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            int c = 0, i = 0;
            for (int item = blockIdx.x; item < n_tiles_total * splits && ok; item += gridDim.x, ++i) {
                const TcItem it(item, n_tiles_total, k_blocks, splits);
                const int buf = i % N_ACC;
                const uint32_t use = (uint32_t)(i / N_ACC) & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, use ^ 1, abort_flag)) {    // the epilogue has drained this region
                    *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); ok = false; break;
                }
                tc_fence_after();
                const uint32_t acc = tmem + buf * BN;
                for (int kb = it.kb_lo; kb < it.kb_hi && ok; ++kb, ++c) {
                    const int s = c % STAGES;
                    const uint32_t phase = (c / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, phase, abort_flag)) {
                        *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = smem_desc(a_addr), dw = smem_desc(a_addr + A_BYTES);
                    static_assert(TC_BK == 64, "four k-steps a k-block");
                    tc_mma_x4(acc, da, dw, idesc, kb > it.kb_lo ? 1u : 0u);     // 16 k = 32 bytes further along the swizzled row
                    tc_commit(empty0 + 8 * s);                  // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(acc_full0 + 8 * buf);         // this tile's accumulators are complete
            }
        }
    } else {
        // epilogue: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31 = rows of the tile
        const int quarter = warp & 3;
        int i = 0;
        const bool part = splits > 1;                            // parts of a tile add with atomics
        for (int item = blockIdx.x; item < n_tiles_total * splits; item += gridDim.x, ++i) {
            const TcItem it(item, n_tiles_total, k_blocks, splits);
            const int m0 = (it.tile % m_tiles) * TC_BM, n0 = (it.tile / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            const int buf = i % N_ACC;
            const uint32_t use = (uint32_t)(i / N_ACC) & 1;
            bool ok = mbar_wait(acc_full0 + 8 * buf, use, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) { *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_EPILOGUE); }
                break;
            }
            tc_fence_after();
            const uint32_t acc = tmem + buf * BN;
            tc_epilogue<BN>(acc, quarter, row, n0, M, N, C, ldc, out_is_f32, mode, part, rope);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);   // this warp has read its quarter of the region
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(N_ACC * BN) : "memory");
    }
}

// The same product on SM pairs: two blocks of a cluster share a 256 x 256 tile.  Each block
// fetches 128 rows of A and 128 rows of W per k-block (32 KB, against 48 KB for a 128 x 256 tile of
// one block: shared memory is filled from L2 at about 64 bytes a clock per SM, which is what
// bounds the one-block kernel), the leader issues tcgen05.mma.cta_group::2 (M 256, N 256) over both
// blocks' shared memory, and each block's tensor memory receives its 128 rows of the 256 columns.
// Barriers: ``full`` lives in the leader and counts both blocks' bytes; ``empty`` and ``acc_full``
// exist in both blocks and are signalled by a commit that arrives in both; ``acc_empty`` lives in
// the leader and counts the epilogue warps of both blocks.
template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ C, int ldc, int out_is_f32, int M, int N, int K, int mode, int m_tiles,
                    int n_tiles_total, int group_m, int* __restrict__ error_word, const TcRope rope) {
    constexpr int BN = 256, HALF = 128;
    constexpr uint32_t A_BYTES = HALF * TC_BK * 2, W_BYTES = HALF * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr int N_ACC = 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 2 * N_ACC);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);     // [0]: a role gave up; [1]: stays zero
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const uint32_t rank = cluster_ctarank();                        // 0: the leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + N_ACC);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int i = 0; i < N_ACC; ++i) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, 8); }
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {      // one warp of each block: the pair's allocation, the same columns in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(N_ACC * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // both blocks' barriers are initialised before either signals the other
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full0 = cluster_map(full0, 0);
            int c = 0;
            for (int tile = pair; tile < n_tiles_total && !*abort_flag; tile += n_pairs) {
                const TcTileAt at(tile, m_tiles, n_tiles_total / m_tiles, group_m);
                const int m0 = at.m * 2 * HALF + (int)rank * HALF;
                const int n0 = at.n * BN + (int)rank * HALF;
                for (int kb = 0; kb < k_blocks; ++kb, ++c) {
                    const int s = c % STAGES;
                    const uint32_t phase = (c / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, phase ^ 1, abort_flag)) {
                        *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_PRODUCER); break;
                    }
                    const uint32_t a_dst = smem_u32(smem + s * STAGE_BYTES), w_dst = a_dst + A_BYTES;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &map_a, leader_full0 + 8 * s, kb * TC_BK, m0);
                    tma_load_2d_pair(w_dst, &map_w, leader_full0 + 8 * s, kb * TC_BK, n0);
                }
            }
            if (*abort_flag) {
                // let copies that were issued but never consumed land before the block ends: the
                // leader sees both blocks' bytes on its barriers, the other block gives them time
                if (rank == 0) {
                    for (int i = max(0, c - STAGES); i < c; ++i)
                        mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, abort_flag + 1);
                } else {
                    const long long t0 = clock64();
                    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N 256, M 256 over the pair
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            bool ok = true;
            int c = 0, i = 0;
            for (int tile = pair; tile < n_tiles_total && ok; tile += n_pairs, ++i) {
                const int buf = i % N_ACC;
                const uint32_t use = (uint32_t)(i / N_ACC) & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, use ^ 1, abort_flag)) {    // both epilogues have drained this region
                    *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); ok = false; break;
                }
                tc_fence_after();
                const uint32_t acc = tmem + buf * BN;
                for (int kb = 0; kb < k_blocks && ok; ++kb, ++c) {
                    const int s = c % STAGES;
                    const uint32_t phase = (c / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, phase, abort_flag)) {
                        *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); ok = false; break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = smem_desc(a_addr), dw = smem_desc(a_addr + A_BYTES);
                    tc_mma_pair_x4(acc, da, dw, idesc, kb > 0 ? 1u : 0u);
                    tc_commit_pair(empty0 + 8 * s, 3);              // the stage is free in both blocks
                }
                if (ok) tc_commit_pair(acc_full0 + 8 * buf, 3);     // both blocks' accumulators are complete
            }
        }
    } else {
        const int quarter = warp & 3;
        const uint32_t leader_acc_empty0 = cluster_map(acc_empty0, 0);
        int i = 0;
        for (int tile = pair; tile < n_tiles_total; tile += n_pairs, ++i) {
            const TcTileAt at(tile, m_tiles, n_tiles_total / m_tiles, group_m);
            const int m0 = at.m * 2 * HALF + (int)rank * HALF, n0 = at.n * BN;
            const int row = m0 + quarter * 32 + lane;
            const int buf = i % N_ACC;
            const uint32_t use = (uint32_t)(i / N_ACC) & 1;
            bool ok = mbar_wait(acc_full0 + 8 * buf, use, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) { *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_EPILOGUE); }
                break;
            }
            tc_fence_after();
            tc_epilogue<BN>(tmem + buf * BN, quarter, row, n0, M, N, C, ldc, out_is_f32, mode, false, rope);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * buf);
        }
    }
    tc_fence_before();
    cluster_sync_all();   // neither block leaves while the other may still read its shared memory or signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(N_ACC * BN) : "memory");
    }
    cluster_sync_all();
}

template <int STAGES>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int out_is_f32, int M, int N,
                          int K, int mode, int* error_word, const TcRope& rope, cudaStream_t stream) {
    constexpr size_t smem = STAGES * 2 * 128 * TC_BK * 2 + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto kern = gemm_tc_pair_kernel<STAGES>;
    static int max_pairs = 0;
    if (!max_pairs) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n_sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 1)
            n_sms = 148;
        // how many pairs the device holds at once (a GPC with an odd SM left over holds one fewer)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_sms & ~1);
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = n_sms / 2;
        }
        max_pairs = clusters < n_sms / 2 ? clusters : n_sms / 2;
    }
    const int m_tiles = (M + 255) / 256, n_tiles = (N + 255) / 256;
    const int total = m_tiles * n_tiles;
    const int pairs = total < max_pairs ? total : max_pairs;
    // bands of 16 row tiles (4,096 rows): at 8,192 rows the gate/up projection took 1,412 us with all row
    // tiles in one band, 1,368 / 1,341 / 1,305 us with bands of 4 / 8 / 16; at 2,048 rows bands of 4 lose 4 %
    const int group_m = 16;
    kern<<<2 * pairs, TC_THREADS, smem, stream>>>(ma, mw, C, ldc, out_is_f32, M, N, K, mode, m_tiles, total,
                                                  group_m < m_tiles ? group_m : m_tiles, error_word, rope);
    return ssb_launch_status();
}

template <int BN, int STAGES>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, int out_is_f32, int M, int N,
                     int K, int mode, int splits, int* error_word, const TcRope& rope, cudaStream_t stream) {
    constexpr size_t smem = STAGES * (TC_BM + BN) * TC_BK * 2 + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto kern = gemm_tc_kernel<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    static int n_sms = 0;
    if (!n_sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0)
            n_sms = 148;
    }
    const int total = m_tiles * n_tiles;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    if (splits > 1) {                                    // no empty parts: every part has at least one k-block
        const int per = (k_blocks + splits - 1) / splits;
        splits = (k_blocks + per - 1) / per;
    }
    const long long items = (long long)total * splits;
    kern<<<items < n_sms ? (int)items : n_sms, TC_THREADS, smem, stream>>>(ma, mw, C, ldc, out_is_f32, M, N, K, mode,
                                                                           m_tiles, total, splits, error_word, rope);
    return ssb_launch_status();
}

// A block that waits on a barrier at which nothing ever arrives: the bounded wait gives up after
// about a second, the kernel records the producer's code in the error word and returns, and the
// context stays usable.  It exercises the give-up path that every mbarrier wait of these kernels
// shares; nothing but tests calls it.
__global__ void tc_wait_probe_kernel(int* __restrict__ error_word) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(smem_u32(&bar), 0, &abort_flag)) atomicCAS(error_word, 0, TC_ERR_PRODUCER);
    }
}

SSB_API int ssb_tc_wait_probe(int* error_word, cudaStream_t stream) {
    if (!error_word) return SSB_ERR_BAD_SIZE;
    tc_wait_probe_kernel<<<1, 32, 0, stream>>>(error_word);
    return ssb_launch_status();
}

// A: bfloat16 [M, K] (row stride lda), W: bfloat16 [N, K] (row stride ldw).  mode 0: C[m, n]
// (bfloat16 or float32); mode 1: C (float32) += ; mode 2: W's rows come as [8 gate | 8 up] per 16
// and C (bfloat16, [M, N/2]) = silu(gate) * up.  splits > 1 (mode 1 only): K is cut into that many
// parts per tile, which add with float atomics.  tile_n: 64, 128 or 256 columns a block, or 512 for
// 256 x 256 tiles on SM pairs (no K parts).  error_word: device int, zero while all is well.
static int gemm_tc_any(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int out_dtype, int M,
                       int N, int K, int mode, int tile_n, int splits, int* error_word, const TcRope& rope,
                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8 || N % 8 || !error_word) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)C) & 15) return SSB_ERR_BAD_SIZE;
    if (mode == TC_ACCUMULATE && out_dtype != SSB_F32) return SSB_ERR_BAD_DTYPE;
    if (splits < 1 || splits > 64 || (splits > 1 && mode != TC_ACCUMULATE)) return SSB_ERR_BAD_SIZE;
    if (mode == TC_SWIGLU && (out_dtype != SSB_BF16 || N % 16 || ldc % 8)) return SSB_ERR_BAD_SIZE;
    if (mode != TC_SWIGLU && (out_dtype == SSB_F32 ? ldc % 4 : ldc % 8)) return SSB_ERR_BAD_SIZE;
    const bool pair = tile_n == TC_TILE_PAIR;
    if (pair && splits > 1) return SSB_ERR_BAD_SIZE;
    const int bn = tile_n == 64 ? 64 : (tile_n == 128 ? 128 : 256);
    CUtensorMap ma, mw;
    int rc = make_map(&ma, A, M, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mw, W, N, K, ldw, pair ? 128 : bn);
    if (rc) return rc;
    const int f32o = out_dtype == SSB_F32;
    // six stages of 32 KB: four to seven measured the same, the ring is not what bounds the kernel
    if (pair) return launch_tc_pair<6>(ma, mw, C, ldc, f32o, M, N, K, mode, error_word, rope, stream);
    if (bn == 64) return launch_tc<64, 8>(ma, mw, C, ldc, f32o, M, N, K, mode, splits, error_word, rope, stream);
    if (bn == 128) return launch_tc<128, 6>(ma, mw, C, ldc, f32o, M, N, K, mode, splits, error_word, rope, stream);
    return launch_tc<256, 4>(ma, mw, C, ldc, f32o, M, N, K, mode, splits, error_word, rope, stream);
}

SSB_API int ssb_gemm_tc(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int out_dtype, int M,
                        int N, int K, int mode, int tile_n, int splits, int* error_word, cudaStream_t stream) {
    if (mode < TC_STORE || mode > TC_SWIGLU) return SSB_ERR_BAD_SIZE;
    return gemm_tc_any(A, lda, W, ldw, C, ldc, out_dtype, M, N, K, mode, tile_n, splits, error_word, TcRope{}, stream);
}

// The fused query/key/value projection of packed tokens with rotation and cache append in the
// epilogue (see TcRope): A [M, K], W [(n_q + 2 n_kv) head_dim, K], C bfloat16 [M, >= n_q head_dim]
// receives the rotated queries.  head_dim 64 or 128; tables [table_positions, head_dim/2] float32.
SSB_API int ssb_gemm_tc_rope_append(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int K,
                                    const int* pos, const int* slot, const int* page_table, int max_pages,
                                    void* k_cache, void* v_cache, const float* cos_t, const float* sin_t,
                                    int n_q, int n_kv, int head_dim, int page_shift, int tile_n, int* error_word,
                                    cudaStream_t stream) {
    if ((head_dim != 64 && head_dim != 128) || n_q <= 0 || n_kv <= 0 || !pos || !slot || !page_table || !cos_t ||
        !sin_t || !k_cache || !v_cache || page_shift < 0 || page_shift > 20)
        return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) return SSB_ERR_BAD_SIZE;
    TcRope rope{pos, slot, page_table, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, cos_t, sin_t,
                max_pages, n_q, n_kv, head_dim, page_shift};
    return gemm_tc_any(A, lda, W, ldw, C, ldc, SSB_BF16, M, (n_q + 2 * n_kv) * head_dim, K, TC_ROPE_APPEND,
                       tile_n == TC_TILE_PAIR ? TC_TILE_PAIR : 256, 1, error_word, rope, stream);
}
