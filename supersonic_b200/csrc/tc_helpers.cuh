// tcgen05 / TMA / mbarrier wrappers and the tensor-map helper shared by the kernels that run on
// the fifth-generation tensor cores.
#pragma once
#include "common.cuh"
#include <cuda.h>

constexpr int TC_BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
enum { TC_STORE = 0, TC_ACCUMULATE = 1, TC_SWIGLU = 2, TC_ROPE_APPEND = 3 };
enum { TC_ERR_PRODUCER = 1, TC_ERR_MMA = 2, TC_ERR_EPILOGUE = 3 };   // which role's wait ran out

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false if the phase did not complete within about a second, or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred P1;\nmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\nselp.b32 %0, 1, 0, P1;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255) == 255) {
            if (*abort_flag) return false;
            if (clock64() - t0 > 2000000000LL) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// The same with an L2 eviction policy (ssb_policy_evict_first / ssb_policy_evict_last).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                                 uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
// Data that is read once and not again before far more than L2 holds has passed (a step's weights, its
// keys and values) should leave L2 first, so that what every layer reads again stays: activations, the
// residual stream, positions, page tables, rotation tables.
__device__ __forceinline__ uint64_t ssb_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t ssb_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Four k-steps (16 elements, 32 bytes along the swizzled row: 2 descriptor units) of one product in a
// row.  Issued as statements of their own, every tcgen05.mma pays for its own predicate set-up and the
// issuing thread gets one out every 93 cycles on an idle SM and every 168 beside busy warps (measured);
// four in one block with one set-up go out at the tensor cores' own pace (64 cycles at M 128, N 128; 74
// beside busy warps).  The first step accumulates only if ``accumulate`` is set, the others always do.
__device__ __forceinline__ void tc_mma_x4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n.reg .pred p, q;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n"
                 "setp.ne.b32 p, %4, 0;\nsetp.eq.b32 q, %5, 0;\n"
                 "add.u64 a1, %1, 2;\nadd.u64 a2, %1, 4;\nadd.u64 a3, %1, 6;\n"
                 "add.u64 b1, %2, 2;\nadd.u64 b2, %2, 4;\nadd.u64 b3, %2, 6;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, {%5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, {%5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, {%5, %5, %5, %5}, q;\n}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- an SM pair (two blocks of a cluster, cta_group::2) ---------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of this block's shared-memory address ``addr`` in block ``rank`` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    __syncthreads();      // the roles' branches have ended for every thread of the block
    asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// A TMA load into this block's shared memory whose bytes count at a barrier that may live in the
// pair's other block (a shared::cluster address).  No multicast: each block fetches its own half.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
// Arrives at the barrier at this shared-memory offset in every block of ``mask`` once the pair's
// earlier MMAs have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// M 256 over the pair: rows 0-127 from the leader's shared memory into its tensor memory, rows
// 128-255 from the other block's; each block supplies half of B's N rows.
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// Four k-steps of a pair's product in one block (see tc_mma_x4).
__device__ __forceinline__ void tc_mma_pair_x4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile("{\n.reg .pred p, q;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n"
                 "setp.ne.b32 p, %4, 0;\nsetp.eq.b32 q, %5, 0;\n"
                 "add.u64 a1, %1, 2;\nadd.u64 a2, %1, 4;\nadd.u64 a3, %1, 6;\n"
                 "add.u64 b1, %2, 2;\nadd.u64 b2, %2, 4;\nadd.u64 b3, %2, 6;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// 8-row groups 1024 bytes apart (stride offset), leading offset unused (1), version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}


// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// rows x cols bfloat16, row stride ld elements; boxes of box_rows x 64 elements, 128-byte swizzle
static inline int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return SSB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : SSB_ERR_BAD_SIZE;
}

