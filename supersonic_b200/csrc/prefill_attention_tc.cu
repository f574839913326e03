// Prefill attention on the fifth-generation tensor cores (head_dim 64 or 128): causal grouped-query
// attention of a ragged batch of new tokens over the paged cache.
//
// One block works on two tiles of 128 query rows that share a key/value head (two query heads of
// the group over the same rows, or neighbouring row tiles), so keys and values are fetched once
// for 256 rows.  Warp 0 feeds TMA: the two query tiles once, then two pages (128 keys) of keys
// and of values per turn into a two-stage ring (128-byte swizzle).  Warp 1 issues tcgen05.mma: per
// tile S = Q K^T (M 128, N 128, K head_dim) into tensor memory, and O += P V (M 128, N head_dim, K 128) with P
// read from tensor memory, where the softmax wrote it over S, and V read MN-major from the pages as
// they lie in the cache.  Warps 2-5 and 6-9 own one query row of the first and second tile per
// thread: scores come with tcgen05.ld, are masked
// on the diagonal only, and leave as bfloat16 probabilities with tcgen05.st.  O stays in tensor
// memory for the whole row of blocks: a row's reference maximum is set by its first block and moves
// only when a later block's probabilities against it sum to more than 2^8 (no probability is ever
// larger than that), and only then is the block's maximum looked for and O rescaled (tcgen05.ld,
// multiply, tcgen05.st); the sum uses the same reference, so the quotient is the exact softmax.
// While one tile's rows are in the softmax the tensor cores work on the other tile.  Every mbarrier
// wait is bounded.
//
// Same arithmetic as prefill_attention.cu (mma.sync), which stays as the kernel for short prompts
// and as this one's reference.  Replaces supersonic_qwen35_full_attention_prefill_kernel of the
// reference (kernels/full_attention_cuda.cuh:360-474).
#include "common.cuh"
#include "tc_helpers.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int FT_BM = 128;                 // query rows per tile
constexpr int FT_BN = 128;                 // keys per turn = two cache pages
constexpr int FT_STAGES = 2;
constexpr int FT_THREADS = 320;
constexpr float FT_LAZY = 8.f;             // log2 of how far a probability may exceed 1
constexpr float FT_LAZY_P = 256.f;         // 2^FT_LAZY
// tensor-memory columns of tile x: scores, later probabilities, at 128 x; output at 256 + 128 x
constexpr uint32_t FT_S0 = 0, FT_O0 = 256;
constexpr int FT_NBARS = 1 + 3 * FT_STAGES + 6;

__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A operand from tensor memory, B from shared memory
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// tc_mma_x4 (tc_helpers.cuh) with A in tensor memory (8 columns a step) and B's descriptor 128 units (16 rows of
// 128 bytes) a step.
__device__ __forceinline__ void tc_mma_ts_x4(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile("{\n.reg .pred p, q;\n.reg .b32 a1, a2, a3;\n.reg .b64 b1, b2, b3;\n"
                 "setp.ne.b32 p, %4, 0;\nsetp.eq.b32 q, %5, 0;\n"
                 "add.u32 a1, %1, 8;\nadd.u32 a2, %1, 16;\nadd.u32 a3, %1, 24;\n"
                 "add.u64 b1, %2, 128;\nadd.u64 b2, %2, 256;\nadd.u64 b3, %2, 384;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, {%5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, {%5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, {%5, %5, %5, %5}, q;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// MN-major operand (values: [key][dim], dim contiguous) in two 64-column boxes 8 KB apart, rows of
// 128 bytes with the 128-byte swizzle: 64-element blocks along N are 8192 bytes apart (leading
// offset), groups of 8 keys 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (512ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

template <int FT_HD>                       // head size: 64 or 128 (one or two 64-column boxes a row)
__global__ void __launch_bounds__(FT_THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ cu_new,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                            const int* __restrict__ page_table, int max_pages, bf16* __restrict__ out, int ldo,
                            int n_q, int n_kv, int window, float scale_log2, int* __restrict__ error_word) {
    constexpr int HALVES = FT_HD / 64;                           // 64-column boxes a row
    constexpr uint32_t FT_Q_BYTES = FT_BM * FT_HD * 2;           // a query tile
    constexpr uint32_t FT_PAGE_BYTES = 64 * FT_HD * 2;           // a page of keys (or values) of one kv head
    constexpr uint32_t FT_KV_BYTES = 2 * FT_PAGE_BYTES;          // keys (or values) of a turn
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                                   // two tiles of 32 KB
    unsigned char* kv_s = smem + 2 * FT_Q_BYTES;                 // stages of [keys of two pages | values of two pages]
    uint64_t* bars = (uint64_t*)(kv_s + FT_STAGES * 2 * FT_KV_BYTES);
    // q_full, k_full[S], v_full[S], kv_empty[S], s_full[tile], p_full[tile], o_full[tile]: the scores of a
    // tile's next block are issued only after its probabilities were handed over, so no role ever
    // meets a barrier two phases on
    const uint32_t q_full = smem_u32(bars), k_full0 = q_full + 8, v_full0 = k_full0 + 8 * FT_STAGES,
                   kv_empty0 = v_full0 + 8 * FT_STAGES, s_full0 = kv_empty0 + 8 * FT_STAGES, p_full0 = s_full0 + 16,
                   o_full0 = p_full0 + 16;
    uint32_t* tmem_slot = (uint32_t*)(bars + FT_NBARS);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);   // [0]: a role gave up; [1]: stays zero

    // blocks start in the order of blockIdx.x, then y: every head's longest tiles come first
    const int kvh = blockIdx.x % n_kv, b = blockIdx.x / n_kv;
    const int row0 = cu_new[b], n_new = cu_new[b + 1] - row0;
    const int slot = seq_slot[b];
    if (slot < 0 || n_new <= 0) return;
    const int group = n_q / n_kv;
    const int n_items = ((n_new + FT_BM - 1) / FT_BM) * group;   // (row tile, head of the group), heads fastest
    const int pair = (int)gridDim.y - 1 - (int)blockIdx.y;       // long tiles first
    if (2 * pair >= n_items) return;
    const int start = seq_start[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // the two tiles of this block
    int t_head[2], t_row[2], t_p0[2], t_rows[2], t_last[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int item = 2 * pair + x;
        const int tile = item / group;
        t_head[x] = kvh * group + item % group;
        t_row[x] = row0 + tile * FT_BM;
        t_p0[x] = start + tile * FT_BM;
        t_rows[x] = item < n_items ? min(FT_BM, n_new - tile * FT_BM) : 0;
        t_last[x] = t_p0[x] + t_rows[x] - 1;
    }
    const int p_first = t_p0[0];                                 // tile 0 is never the later one
    const int kb_lo = (window > 0 && p_first - window + 1 > 0) ? (p_first - window + 1) >> 6 : 0;
    int nb[2];                                                   // turns of two pages, from page kb_lo on
    nb[0] = ((t_last[0] >> 6) - kb_lo + 2) >> 1;
    nb[1] = t_rows[1] > 0 ? ((t_last[1] >> 6) - kb_lo + 2) >> 1 : 0;
    const int last_page = (start + n_new - 1) >> 6;              // the last page the sequence holds
    const int nb_max = max(nb[0], nb[1]);
    const int* pt = page_table + (size_t)slot * max_pages;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < FT_STAGES; ++s) {
            mbar_init(k_full0 + 8 * s, 1); mbar_init(v_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(s_full0 + 8 * i, 1); mbar_init(p_full0 + 8 * i, 4); mbar_init(o_full0 + 8 * i, 1); }
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, (nb[1] > 0 ? 2 : 1) * FT_Q_BYTES);
#pragma unroll
            for (int x = 0; x < 2; ++x)
                if (nb[x] > 0) {
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(smem_u32(q_s) + x * FT_Q_BYTES + h * (FT_Q_BYTES / HALVES), &map_q, q_full,
                                    t_head[x] * FT_HD + 64 * h, t_row[x]);
                }
            int issued = 0;
            for (int j = 0; j < nb_max; ++j) {
                const int s = j % FT_STAGES;
                if (!mbar_wait(kv_empty0 + 8 * s, ((j / FT_STAGES) & 1) ^ 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_PRODUCER); break;
                }
                // keys: [64-column box][page][64 keys x 128 bytes], a K-major tile of 128 rows per box;
                // values: [page][64-column box][64 keys x 128 bytes].  A page past the sequence's last one
                // (odd page counts) is the last one again: its keys lie beyond every query and are masked.
                const uint32_t k_dst = smem_u32(kv_s + s * 2 * FT_KV_BYTES), v_dst = k_dst + FT_KV_BYTES;
                mbar_expect_tx(k_full0 + 8 * s, FT_KV_BYTES);
                mbar_expect_tx(v_full0 + 8 * s, FT_KV_BYTES);
#pragma unroll
                for (int pg = 0; pg < 2; ++pg) {
                    const int y = (pt[min(kb_lo + 2 * j + pg, last_page)] * n_kv + kvh) * 64;   // first row of the page in the 2-D view
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        tma_load_2d(k_dst + h * (FT_KV_BYTES / HALVES) + pg * 8192, &map_k, k_full0 + 8 * s, 64 * h, y);
                        tma_load_2d(v_dst + pg * FT_PAGE_BYTES + h * 8192, &map_v, v_full0 + 8 * s, 64 * h, y);
                    }
                }
                issued = j + 1;
            }
            if (*abort_flag) {                                   // let issued copies land
                mbar_wait(q_full, 0, abort_flag + 1);
                for (int j = max(0, issued - FT_STAGES); j < issued; ++j) {
                    mbar_wait(k_full0 + 8 * (j % FT_STAGES), (j / FT_STAGES) & 1, abort_flag + 1);
                    mbar_wait(v_full0 + 8 * (j % FT_STAGES), (j / FT_STAGES) & 1, abort_flag + 1);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // S: D float32, A and B bfloat16 K-major, M 128, N 128.  PV: B MN-major (bit 16), N 128.
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FT_BN >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(FT_HD >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            const uint64_t q_desc = smem_desc(smem_u32(q_s)), k_desc = smem_desc(smem_u32(kv_s));
            const uint64_t v_desc = smem_desc_mn(smem_u32(kv_s) + FT_KV_BYTES);
            auto issue_s = [&](int x, int j) -> bool {           // scores of block j of tile x
                const int s = j % FT_STAGES;
                if (!mbar_wait(k_full0 + 8 * s, (j / FT_STAGES) & 1, abort_flag)) return false;
                tc_fence_after();
                const uint64_t da = q_desc + (uint64_t)(x * (FT_Q_BYTES >> 4));
                const uint64_t db = k_desc + (uint64_t)(s * (2 * FT_KV_BYTES >> 4));
#pragma unroll
                for (int h = 0; h < HALVES; ++h)                 // 64 dims a box, four steps of 16; descriptors count in units of 16 bytes
                    tc_mma_x4(tmem + FT_S0 + x * FT_BN, da + h * (FT_Q_BYTES / HALVES >> 4),
                              db + h * (FT_KV_BYTES / HALVES >> 4), idesc_s, h ? 1u : 0u);
                tc_commit(s_full0 + 8 * x);
                return true;
            };
            for (int x = 0; x < 2 && ok; ++x)
                if (nb[x] > 0) ok = issue_s(x, 0);
            for (int j = 0; j < nb_max && ok; ++j) {
                const int s = j % FT_STAGES;
                for (int x = 0; x < 2 && ok; ++x) {
                    if (j >= nb[x]) continue;
                    if (!mbar_wait(p_full0 + 8 * x, j & 1, abort_flag) ||
                        !mbar_wait(v_full0 + 8 * s, (j / FT_STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t dv = v_desc + (uint64_t)(s * (2 * FT_KV_BYTES >> 4));
#pragma unroll
                    for (int pg = 0; pg < 2; ++pg)               // a page: four steps of 16 keys, 16 rows of 128 bytes apart
                        tc_mma_ts_x4(tmem + FT_O0 + x * FT_HD, tmem + FT_S0 + x * FT_BN + pg * 32,
                                     dv + pg * (FT_PAGE_BYTES >> 4), idesc_o, (j > 0 || pg > 0) ? 1u : 0u);
                    tc_commit(o_full0 + 8 * x);
                    // the next scores go where these probabilities lie: the tensor cores take
                    // their work in the order of issue
                    if (j + 1 < nb[x]) ok = issue_s(x, j + 1);
                }
                tc_commit(kv_empty0 + 8 * s);
            }
            if (!ok) { *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); }
        }
    } else {
        // softmax and output: one query row per thread; warps 2-5 tile 0, warps 6-9 tile 1
        const int x = (warp - 2) >> 2;
        const int n_mine = nb[x];
        if (n_mine > 0) {
            const int quarter = warp & 3;                        // the lanes of tensor memory this warp may touch
            const int r = quarter * 32 + lane;
            const int p0 = t_p0[x];
            const int pos = p0 + r;
            const uint32_t t_s = tmem + ((uint32_t)(quarter * 32) << 16) + FT_S0 + x * FT_BN;
            const uint32_t t_o = tmem + ((uint32_t)(quarter * 32) << 16) + FT_O0 + x * FT_HD;
            const uint32_t s_full = s_full0 + 8 * x, p_full = p_full0 + 8 * x, o_full = o_full0 + 8 * x;
            float m_ref = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < n_mine; ++j) {
                bool w = mbar_wait(s_full, j & 1, abort_flag);
                w = __all_sync(0xffffffffu, w);
                if (!w) { ok = false; break; }
                tc_fence_after();
                const int key0 = (kb_lo + 2 * j) * 64;
                const bool edge = key0 + FT_BN - 1 > p0 || window > 0;   // on the diagonal or at a window's edge
                const int hi = pos - key0;                       // keys 0..hi of the block are seen
                const int lo = window > 0 ? hi - window + 1 : 0;
                // the row's 128 scores in registers: four loads in flight, one wait
                uint32_t raw[FT_BN];
#pragma unroll
                for (int c = 0; c < FT_BN / 32; ++c) tc_ld32_issue(t_s + c * 32, raw + c * 32);
                tc_ld_wait();
                if (edge) {
#pragma unroll
                    for (int i = 0; i < FT_BN; ++i)
                        if (i > hi || i < lo) raw[i] = 0xff800000u;
                }
                // probabilities 2^(score * scale - reference) of the row's 128 scores, as bfloat16 over the scores
                // in tensor memory (those of 64 keys go over the scores of 32 keys; all scores are in
                // registers); returns their sum
                auto probabilities = [&](float neg_ref) -> float {
                    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t packed[32];
#pragma unroll
                        for (int i = 0; i < 64; i += 2) {
                            const float pa = ex2(fmaf(__uint_as_float(raw[half * 64 + i]), scale_log2, neg_ref));
                            const float pb = ex2(fmaf(__uint_as_float(raw[half * 64 + i + 1]), scale_log2, neg_ref));
                            sum[(i >> 1) & 3] += pa + pb;
                            __nv_bfloat162 v = __floats2bfloat162_rn(pa, pb);
                            packed[i / 2] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        tc_st32(t_s + half * 32, packed);
                    }
                    return (sum[0] + sum[1]) + (sum[2] + sum[3]);
                };
                // After a row's first block the probabilities are taken against the reference as it stands,
                // without looking for the block's maximum first (a third of a block's softmax time, which
                // is the one step of a tile that its own products cannot overlap): a probability above
                // 2^FT_LAZY makes the row's sum exceed 2^FT_LAZY too, and only then (or while a row has
                // seen no key yet) is the maximum found, the output rescaled and the block done again.
                float sum = 0.f;
                bool find_max = j == 0;
                if (!find_max) {
                    sum = probabilities(m_ref == -INFINITY ? 0.f : -m_ref);
                    find_max = __any_sync(0xffffffffu, !(sum <= FT_LAZY_P) || m_ref == -INFINITY);
                }
                if (find_max) {
                    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < FT_BN; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(raw[i]));
                    const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
                    const float m_new = fmaxf(m_ref, m_blk);
                    if (j > 0 && __any_sync(0xffffffffu, m_new > m_ref)) {
                        // rescale what this warp's rows have summed so far to their new maxima
                        bool wo = mbar_wait(o_full, (j - 1) & 1, abort_flag);
                        wo = __all_sync(0xffffffffu, wo);
                        if (!wo) { ok = false; break; }
                        tc_fence_after();
                        const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m_ref - m_new);
#pragma unroll 1
                        for (int c = 0; c < FT_HD / 32; ++c) {
                            uint32_t o[32];
                            tc_ld32_issue(t_o + c * 32, o);
                            tc_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tc_st32(t_o + c * 32, o);
                        }
                        l_run *= alpha;
                    }
                    m_ref = m_new;
                    tc_st_wait();                                // what was written against the old reference has landed
                    sum = probabilities(m_ref == -INFINITY ? 0.f : -m_ref);
                }
                tc_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cta(p_full);
                l_run += sum;
            }
            if (ok) {
                bool w = mbar_wait(o_full, (n_mine - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, w);
            }
            if (!ok) {
                if (lane == 0) { *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_EPILOGUE); }
            } else {
                tc_fence_after();
                const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
                uint4* dst = reinterpret_cast<uint4*>(out + (size_t)(t_row[x] + r) * ldo + (size_t)t_head[x] * FT_HD);
#pragma unroll
                for (int c = 0; c < FT_HD / 32; ++c) {
                    uint32_t o[32];
                    tc_ld32_issue(t_o + c * 32, o);
                    tc_ld_wait();
                    if (r < t_rows[x]) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 v;
                            __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
                            __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
                            __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
                            __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
                            v.x = *reinterpret_cast<uint32_t*>(&a0); v.y = *reinterpret_cast<uint32_t*>(&a1);
                            v.z = *reinterpret_cast<uint32_t*>(&a2); v.w = *reinterpret_cast<uint32_t*>(&a3);
                            dst[c * 4 + i] = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// 2-D bfloat16 tensor map with boxes of box_rows x 64 columns, 128-byte swizzle (tc_helpers.cuh).
// q: packed rows [n_rows_q, ldq]; caches: [n_pages, n_kv, 64, 128] seen as [n_pages * n_kv * 64, 128].
SSB_API int ssb_attention_prefill_tc(const void* q, int ldq, int n_rows_q, const void* k_cache, const void* v_cache,
                                     int n_pages, const int* cu_new, const int* seq_start, const int* seq_slot,
                                     const int* page_table, int max_pages, void* out, int ldo, int n_seqs, int max_new,
                                     int n_q, int n_kv, int head_dim, int page_shift, int window, float scale,
                                     int* error_word, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if ((head_dim != 64 && head_dim != 128) || page_shift != 6) return SSB_ERR_UNSUPPORTED;
    if (n_kv <= 0 || n_q % n_kv || ldq % 8 || ldo % 8 || !error_word ) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return SSB_ERR_BAD_SIZE;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, n_rows_q, n_q * head_dim, ldq, FT_BM);
    if (rc) return rc;
    const long long cache_rows = (long long)n_pages * n_kv * 64;
    if (cache_rows > 0x7fffffffLL) return SSB_ERR_BAD_SIZE;
    rc = make_map(&mk, k_cache, (int)cache_rows, head_dim, head_dim, 64);
    if (rc) return rc;
    rc = make_map(&mv, v_cache, (int)cache_rows, head_dim, head_dim, 64);
    if (rc) return rc;
    const int group = n_q / n_kv;
    const int pairs = (((max_new + FT_BM - 1) / FT_BM) * group + 1) / 2;
    if (pairs > 65535) return SSB_ERR_BAD_SIZE;
    dim3 grid(n_kv * n_seqs, pairs);
#define SSB_FT(HD_) do { \
        constexpr size_t smem = 2 * FT_BM * HD_ * 2 + FT_STAGES * 4 * 64 * HD_ * 2 + FT_NBARS * 8 + 32 + 1024; \
        static bool configured = false; \
        if (!configured) { \
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        prefill_attention_tc_kernel<HD_><<<grid, FT_THREADS, smem, stream>>>( \
            mq, mk, mv, cu_new, seq_start, seq_slot, page_table, max_pages, (bf16*)out, ldo, n_q, n_kv, window, \
            scale * 1.4426950408889634f, error_word); \
    } while (0)
    if (head_dim == 64) SSB_FT(64); else SSB_FT(128);
#undef SSB_FT
    return ssb_launch_status();
}
