// Decode attention on the tensor cores, for head sizes 64 and 128 and up to 16 query heads per
// kv head.  The products are taken transposed, S^T = K Q^T and O^T = V^T P^T: a warp's 16 keys of a
// page are the 16 rows of an m16n8k16 tile (all used) and the query heads that share the kv head its 8
// columns, so a page costs a warp 8 + 8 MMAs for up to 8 heads per kv head (16 + 16 for 9 to 16).
// With the heads as rows, as the kernel first had it, three quarters of a tile's rows were padding at
// four heads per kv head, it took twice the MMAs, and mma.sync is what bounds a page's arithmetic here
// (64 x 520: 30.0 to 24.8 us; 8 x 8,192: 45.8 to 41.9).
//
// Work items and a persistent grid.  A sequence's pages are cut into chunks of about
// ``chunk_pages`` pages (as many chunks as that needs, of even size: the cut depends on the
// sequence alone, never on what else is in the batch); an item is (sequence, chunk, kv head).
// About two blocks per SM are launched and block j takes items j, j + grid, j + 2 grid, ...:
// every block first counts the chunks of all sequences (a prefix sum over the batch in shared
// memory), so no host-made work list is needed and a captured graph serves any lengths.  A batch
// of very unequal lengths then keeps every SM busy to the end, which a grid of (sequence, head,
// split) with one split count for all does not.
//
// Per item one thread asks the TMA unit for a page of keys and values (tiled loads of 64 keys x 64
// dims with the 128-byte swizzle, two stages, an mbarrier per stage that counts the bytes; every
// wait is bounded and a wait that runs out is recorded in a device word); each warp takes 16 of
// the page's 64 keys: S^T = K Q^T (16 keys x 8 heads), online softmax in float32, O^T += V^T P^T.  Warps merge in
// shared memory; a sequence of several chunks leaves partial results in scratch and the item that
// arrives last for its (sequence, kv head) merges them in chunk order (maxima kept in the log2
// domain; a partial result is head_dim sums, the maximum, the sum of weights, in 16-byte units).
// Nothing waits on another block; at small batch a sequence's chunks are instead the blocks of a
// thread-block cluster that merges through distributed shared memory (CL).
// With FUSE the rows of q are the raw fused projection [q | k | v]: queries are rotated while
// the fragments are built, and the item that owns the token's page rotates its key, appends key
// and value to the cache and attends to them from registers.
//
// Replaces supersonic_qwen35_full_attention_decode_*_kernel of the reference (one warp per query
// head, two passes over the keys: kernels/full_attention_cuda.cuh:476-679).
#pragma once
#include "attention_decode.cuh"
#include "mma_helpers.cuh"
#include "tc_helpers.cuh"
#include <mutex>

constexpr int ADM_WARPS = 4;
constexpr int ADM_THREADS = ADM_WARPS * 32;
// floats of one partial result in scratch: the head's sums, its maximum and its sum of weights, padded to 16 bytes
#define ADM_PITCH(hd) ((hd) + 4)
constexpr int ADM_ROWS = 16;          // query heads per kv head, padded to the MMA's 16 rows
// Stages of the page ring (a stage: one page of keys and one of values, 32 KB at head size 128).  Three
// and four stages measured the same as two at every batch and context tried: with two blocks on every
// SM the loads in flight already cover the memory's latency.
__host__ __device__ constexpr int adm_stages(int /*head_dim*/) { return 2; }
constexpr int ADM_MAX_SEQS = 1024;    // sequences a launch can take (their slots, positions and chunk counts sit in shared memory)
// Transpose an 8 x 8 matrix of 16-bit values held across the warp (lane 4 r + c holds row r, columns 2 c, 2 c + 1).
__device__ __forceinline__ uint32_t adm_transpose8(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// One work item, decoded from its index (everything block-uniform).
struct AdmItem {
    int b, kvh, chunk, n_chunks, slot, p, key_lo, key_hi, page_hi, pf, units, page0, page1;
    bool owns_new;
};

// Byte offset of 16-byte chunk ``chunk`` of key ``row`` in a page tile as the TMA unit leaves it: one
// box of 64 keys x 64 dims (128-byte rows, chunk c of row r at c ^ (r & 7)) per 64 dims, 8 KB apart.
__device__ __forceinline__ uint32_t adm_tile_offset(int row, int chunk) {
    return (uint32_t)(((chunk >> 3) << 13) + (row << 7) + (((chunk & 7) ^ (row & 7)) << 4));
}

// Thread-block clusters (CL): the chunks of one (sequence, kv head) are the blocks of one cluster and
// merge through the cluster's shared memory.
__device__ __forceinline__ unsigned adm_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned adm_cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void adm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 adm_ld_cluster4(const float* local, unsigned rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float2 adm_ld_cluster2(const float* local, unsigned rank) {
    uint32_t remote;
    float2 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
    return v;
}

template <int HD, bool FUSE, bool CL, int NT>   // NT: tiles of 8 query heads per kv head (1: up to 8 heads, 2: up to 16)
__global__ void __launch_bounds__(ADM_THREADS)
attention_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* k_cache,
                            __nv_bfloat16* v_cache, const int* __restrict__ pos, const int* __restrict__ slot,
                            const int* __restrict__ page_table, int max_pages, __nv_bfloat16* __restrict__ out,
                            int ldo, int n_seqs, int n_q, int n_kv, int window, float scale_log2, int chunk_pages,
                            int max_chunks, float* __restrict__ scratch, int* __restrict__ counters,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            int* __restrict__ error_word) {
    constexpr int CHUNKS = HD / 8, TILE_BYTES = 64 * HD * 2, KS = HD / 16, HALF = HD / 2, STAGES = adm_stages(HD);
    const int group = n_q / n_kv;
    // a query buffer: the item's query rows, the rotation tables' row, the token's own key and value
    const int Q_OFF = 0, COS_OFF = group * HD * 2, SIN_OFF = COS_OFF + HALF * 4, KN_OFF = SIN_OFF + HALF * 4,
              VN_OFF = KN_OFF + HD * 2, QBUF_BYTES = VN_OFF + HD * 2;
    // dynamic shared memory (adm_smem_bytes): tiles, warp sums, two query buffers, the batch's integers
    extern __shared__ __align__(128) unsigned char adm_smem[];
    // the stages' key tiles, then their value tiles: swizzled tiles start on 1,024-byte boundaries
    unsigned char* smem = adm_smem + ((1024u - (smem_u32(adm_smem) & 1023u)) & 1023u);
    constexpr int ACC_LD = HD + 4;       // row pitch of the warp sums: rows g and g + 1 land four banks apart
    float* sm_acc = reinterpret_cast<float*>(smem + 2 * STAGES * TILE_BYTES);          // [ADM_WARPS][group][ACC_LD]
    unsigned char* qbufs = smem + 2 * STAGES * TILE_BYTES + ADM_WARPS * group * ACC_LD * 4;
    int* cum = reinterpret_cast<int*>(qbufs + 2 * QBUF_BYTES);   // [n_seqs + 1] chunks of the sequences before each one
    int* sm_slot = cum + n_seqs + 1;                             // [n_seqs] the batch's slots and positions, read once
    int* sm_pos = sm_slot + n_seqs;
    __shared__ float sm_m[ADM_WARPS][ADM_ROWS], sm_l[ADM_WARPS][ADM_ROWS];
    __shared__ int is_last;
    __shared__ float2 cl_ml[ADM_ROWS];                           // CL: this chunk's maximum and sum of weights per head
    __shared__ __align__(8) unsigned long long full_bar[STAGES];      // a stage's bytes have landed
    __shared__ int sm_abort[2];                                  // [0]: a wait ran out; [1]: stays zero
    volatile int* abort_flag = sm_abort;
    const uint32_t full0 = smem_u32(full_bar);
    __shared__ int warp_total[ADM_WARPS], warp_longest[ADM_WARPS], warp_live[ADM_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    ssb_pdl_launch_dependents();
    // Positions, slots and page tables were written before this chain of kernels began: they may be
    // read before the dependency wait, and so may pages of earlier steps' keys.
    for (int b = threadIdx.x; b < n_seqs; b += ADM_THREADS) { sm_slot[b] = slot[b]; sm_pos[b] = pos[b]; }
    if (threadIdx.x == 0) {
        for (int st = 0; st < STAGES; ++st) mbar_init(full0 + 8 * st, 1);
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    auto pages_of = [&](int b) {
        if (sm_slot[b] < 0) return 0;                            // a padding row is no work item (zeros below)
        const int p = sm_pos[b];
        const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
        return (p >> 6) - (key_lo >> 6) + 1;
    };
    // chunk_pages <= 0: the kernel sizes the chunks itself from the batch's pages; every block computes
    // the same figure.  Sequences of about equal length: items about as many as the blocks (a fifth of
    // them spare, for the items that rounding adds), since an item's fixed cost is worth some six pages
    // of streaming.  Very unequal lengths (the longest more than one and a half times the mean) with
    // enough work for it: two to three items a block, of at least eight pages, so that the blocks end
    // together.  A caller that wants a sequence cut the same way in every batch gives chunk_pages itself.
    const int n_cl = CL ? (int)adm_cluster_size() : 1;          // blocks of a cluster: the chunks of every sequence
    if (!CL && chunk_pages <= 0) {
        int local = 0, longest = 0, live = 0;
        for (int b = threadIdx.x; b < n_seqs; b += ADM_THREADS) {
            const int n = pages_of(b);
            local += n;
            longest = max(longest, n);
            live += n > 0;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            local += __shfl_xor_sync(0xffffffffu, local, o);
            live += __shfl_xor_sync(0xffffffffu, live, o);
            longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
        }
        if (lane == 0) { warp_total[warp] = local; warp_longest[warp] = longest; warp_live[warp] = live; }
        __syncthreads();
        long long units = 0;
        int seqs = 0;
        longest = 0;
        for (int w = 0; w < ADM_WARPS; ++w) { units += warp_total[w]; seqs += warp_live[w]; longest = max(longest, warp_longest[w]); }
        const bool unequal = 2LL * longest * seqs > 3LL * units;            // longest > 1.5 x mean
        units *= n_kv;
        const long long coarse = max(1LL, (long long)gridDim.x * 4 / 5), fine = max(1LL, (long long)gridDim.x * 5 / 2);
        const long long fine_pages = (units + fine - 1) / fine;
        chunk_pages = (unequal && fine_pages >= 8) ? (int)fine_pages : (int)max(2LL, (units + coarse - 1) / coarse);
        __syncthreads();                                         // warp_total is used again below
    }
    auto chunks_of = [&](int b) {
        const int n = pages_of(b);
        return n == 0 ? 0 : min((n + chunk_pages - 1) / chunk_pages, max_chunks);
    };
    if (CL) {
        // every sequence has as many chunks as its clusters have blocks (some may be empty)
        for (int b = threadIdx.x; b <= n_seqs; b += ADM_THREADS) cum[b] = b * n_cl;
        __syncthreads();
    } else {
        const int per = (n_seqs + ADM_THREADS - 1) / ADM_THREADS;
        const int b0 = (int)threadIdx.x * per;
        int local = 0;
        for (int i = 0; i < per; ++i)
            if (b0 + i < n_seqs) local += chunks_of(b0 + i);
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_total[warp] = incl;
        __syncthreads();
        int base = 0;
        for (int w = 0; w < warp; ++w) base += warp_total[w];
        int running = base + incl - local;
        for (int i = 0; i < per; ++i)
            if (b0 + i < n_seqs) { cum[b0 + i] = running; running += chunks_of(b0 + i); }
        if (threadIdx.x == ADM_THREADS - 1) cum[n_seqs] = base + incl;
        __syncthreads();
    }
    const int total_items = cum[n_seqs] * n_kv;

    // An item is decoded two items ahead of its turn: the ids of its first two pages are asked for here
    // and are in registers long before its pages are issued.
    auto decode = [&](int idx, AdmItem& I) {
        int lo;
        if (CL) {                                                // block = (sequence, kv head, chunk), the chunk fastest
            I.chunk = idx % n_cl;
            I.kvh = (idx / n_cl) % n_kv;
            lo = idx / (n_cl * n_kv);
            I.n_chunks = n_cl;
        } else {
            const int gc = idx / n_kv;
            I.kvh = idx - gc * n_kv;
            lo = 0;
            int hi = n_seqs - 1;                                 // the last sequence whose first chunk is <= gc
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (cum[mid] <= gc) lo = mid; else hi = mid - 1;
            }
            I.chunk = gc - cum[lo];
            I.n_chunks = cum[lo + 1] - cum[lo];
        }
        I.b = lo;
        I.slot = sm_slot[lo];
        I.p = sm_pos[lo];
        I.key_lo = (window > 0 && I.p - window + 1 > 0) ? I.p - window + 1 : 0;
        I.key_hi = FUSE ? I.p - 1 : I.p;                         // with FUSE the token's own key is not cached yet
        const int page_lo = I.key_lo >> 6;
        I.page_hi = I.p >> 6;
        const int per = (I.page_hi - page_lo + I.n_chunks) / I.n_chunks;     // even chunks: ceil(pages / chunks)
        I.pf = page_lo + I.chunk * per;
        const int pl = min(I.page_hi, I.pf + per - 1);
        I.units = max(pl - I.pf + 1, 1);                         // an empty chunk still loads a page (all its keys masked)
        I.owns_new = FUSE && I.pf <= I.page_hi && I.page_hi <= pl;
        const int* pt = page_table + (size_t)I.slot * max_pages;
        I.page0 = pt[min(I.pf, I.page_hi)];
        I.page1 = pt[min(I.pf + 1, I.page_hi)];
    };
    // keys and values pass through L2 once a step: they leave it first, so that what every layer reads
    // again (positions, page tables, rotation tables, activations) stays
    const uint64_t kv_policy = ssb_policy_evict_first();
    int page_ahead = 0, page_ahead_of = -1;      // id of the page STAGES after the one in work, asked for one turn early
    auto load_page = [&](const AdmItem& I, int i, int stage) {
        if (threadIdx.x != 0) return;
        const int page = i == 0 ? I.page0 : (i == 1 ? I.page1 : (i == page_ahead_of ? page_ahead
                         : page_table[(size_t)I.slot * max_pages + min(I.pf + i, I.page_hi)]));
        const int y = (page * n_kv + I.kvh) << 6;                // the page's first key among the cache's rows
        const uint32_t kd = smem_u32(smem + stage * TILE_BYTES), vd = smem_u32(smem + (STAGES + stage) * TILE_BYTES);
        const uint32_t bar = full0 + 8 * stage;
        mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
            tma_load_2d_hint(kd + h * 8192, &map_k, bar, 64 * h, y, kv_policy);
            tma_load_2d_hint(vd + h * 8192, &map_v, bar, 64 * h, y, kv_policy);
        }
    };
    // The rotation tables' row of the item's position: written by no kernel of a step, so it may be
    // asked for before the dependency wait (it joins the next cp.async group that is committed).
    auto load_tables = [&](const AdmItem& I, int which) {
        if (!FUSE) return;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(qbufs + which * QBUF_BYTES);
        const int e = threadIdx.x;                               // HALF / 4 chunks per table row
        if (e < HALF / 4) {
            cp_async16(dst + COS_OFF + e * 16, cos_t + (size_t)I.p * HALF + e * 4);
            cp_async16(dst + SIN_OFF + e * 16, sin_t + (size_t)I.p * HALF + e * 4);
        }
    };
    auto load_query = [&](const AdmItem& I, int which) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(qbufs + which * QBUF_BYTES);
        const __nv_bfloat16* row = q + (size_t)I.b * ldq;
        for (int e = threadIdx.x; e < group * CHUNKS; e += ADM_THREADS)
            cp_async16(dst + Q_OFF + e * 16, row + (size_t)I.kvh * group * HD + e * 8);
        if (FUSE) {
            const int e = threadIdx.x;                           // CHUNKS per vector
            if (e < CHUNKS) {
                cp_async16(dst + KN_OFF + e * 16, row + (size_t)(n_q + I.kvh) * HD + e * 8);
                cp_async16(dst + VN_OFF + e * 16, row + (size_t)(n_q + n_kv + I.kvh) * HD + e * 8);
            }
        }
    };

    // rows without a sequence (a captured step's warm-up): zeros, shared out over the blocks
    bool waited = !FUSE;
    if (!FUSE) ssb_pdl_wait();                                   // the cache holds this step's key already
    if (CL) {
        // a row without a sequence: its cluster's first block writes the kv head's zeros, and the whole
        // cluster leaves before any of its barriers
        const int b = (int)blockIdx.x / (n_cl * n_kv), kvh = ((int)blockIdx.x / n_cl) % n_kv;
        if (sm_slot[b] < 0) {
            if (!waited) ssb_pdl_wait();
            if (blockIdx.x % n_cl == 0)
                for (int e = threadIdx.x; e < group * HD; e += ADM_THREADS)
                    out[(size_t)b * ldo + (size_t)kvh * group * HD + e] = __float2bfloat16_rn(0.f);
            return;
        }
    } else {
        for (int b = blockIdx.x; b < n_seqs; b += gridDim.x)
            if (sm_slot[b] < 0) {
                if (!waited) { ssb_pdl_wait(); waited = true; }
                for (int e = threadIdx.x; e < n_q * HD; e += ADM_THREADS)
                    out[(size_t)b * ldo + e] = __float2bfloat16_rn(0.f);
            }
    }
    if ((int)blockIdx.x >= total_items) {
        if (!waited) ssb_pdl_wait();                             // a block without items still ends after its predecessor
        return;
    }

    // The stream of loads: for every item of this block its query buffer (cp.async by all threads, one
    // group), then its pages one by one (TMA, thread 0).  A page goes to stage (page unit % STAGES), a
    // query to buffer (item & 1); up to STAGES page units are in flight, across item borders, so the
    // fixed cost of an item (its slot, position, page ids, query rows) hides behind the item before it.
    // A chunk's arrival at its (sequence, kv head) counter is counted when the chunk's sums are
    // written, but the answer (was it the last?) is looked at only when the next item's sums are
    // written, so that the atomic's round trip hides behind that item's work.
    int pend_b = -1, pend_kvh = 0, pend_chunks = 0;              // the counted chunk whose answer is still out
    int pend_arrived = 0;                                        // thread 0: what its atomic returned
    auto settle = [&]() {                                        // block-uniform; ends with the merge if it was the last
        if (pend_b < 0) return;
        if (threadIdx.x == 0) {
            is_last = (pend_arrived == pend_chunks - 1);
            if (is_last) counters[(size_t)pend_b * n_kv + pend_kvh] = 0;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            const int ph0 = pend_kvh * group;
            // every thread owns four neighbouring dims of a head's output and goes through the chunks
            // itself, in chunk order, eight at a time: a chunk's four sums come as one 16-byte load and
            // all of the loads are in flight together, so the merge costs one trip to L2, not one per dim
            for (int e = threadIdx.x; e < group * (HD / 4); e += ADM_THREADS) {
                const int row = e / (HD / 4), d = (e % (HD / 4)) * 4;
                const float* base = scratch + ((size_t)pend_b * n_q + ph0 + row) * max_chunks * ADM_PITCH(HD);
                float mm = -INFINITY, ll = 0.f, a[4] = {0.f, 0.f, 0.f, 0.f};
                for (int s0 = 0; s0 < pend_chunks; s0 += 8) {
                    float pm[8], pl[8];
                    float4 pv[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const bool live = s0 + i < pend_chunks;
                        const float* part = base + (size_t)(live ? s0 + i : s0) * ADM_PITCH(HD);
                        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part + HD));
                        pm[i] = live ? ml.x : -INFINITY;
                        pl[i] = ml.y;
                        pv[i] = __ldcg(reinterpret_cast<const float4*>(part + d));
                    }
                    float m_new = mm;
#pragma unroll
                    for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, pm[i]);
                    const float keep = (mm == -INFINITY) ? 0.f : exp2f(mm - m_new);
                    ll *= keep;
#pragma unroll
                    for (int k = 0; k < 4; ++k) a[k] *= keep;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float f = (pm[i] == -INFINITY) ? 0.f : exp2f(pm[i] - m_new);
                        ll = fmaf(pl[i], f, ll);
                        a[0] = fmaf(pv[i].x, f, a[0]); a[1] = fmaf(pv[i].y, f, a[1]);
                        a[2] = fmaf(pv[i].z, f, a[2]); a[3] = fmaf(pv[i].w, f, a[3]);
                    }
                    mm = m_new;
                }
                const float inv = ll > 0.f ? 1.f / ll : 0.f;
                uint2 w;
                w.x = pack2(a[0] * inv, a[1] * inv);
                w.y = pack2(a[2] * inv, a[3] * inv);
                *reinterpret_cast<uint2*>(out + (size_t)pend_b * ldo + (size_t)(ph0 + row) * HD + d) = w;
            }
        }
        __syncthreads();                                         // is_last is free again
        pend_b = -1;
    };

    AdmItem cur, nxt, nn;                // the item in work, the one after it, and the one after that
    int item = blockIdx.x;
    const int G = (int)gridDim.x;
    decode(item, cur);
    bool has_nxt = item + G < total_items, has_nn = item + 2 * G < total_items;
    if (has_nxt) decode(item + G, nxt);
    if (has_nn) decode(item + 2 * G, nn);
    int pu_issued = 0, pu_done = 0;      // page units issued / consumed
    int cursor_item = 0, cursor_pos = 0; // next load to issue: item 0 = cur, 1 = nxt; position -1 = query, else page
    int parity = 0;                      // of cur among this block's items
    bool dead = false;                   // a bounded wait ran out: the block stops (block-uniform)

    auto issue_group = [&]() -> bool {
        if (cursor_item > 1 || (cursor_item == 1 && !has_nxt)) return false;
        const AdmItem& I = cursor_item == 0 ? cur : nxt;
        if (cursor_pos < 0) {
            load_tables(I, parity ^ cursor_item);
            load_query(I, parity ^ cursor_item);
            cp_async_commit();
            cursor_pos = 0;
        } else {
            load_page(I, cursor_pos, pu_issued % STAGES);
            ++pu_issued;
            if (++cursor_pos == I.units) { ++cursor_item; cursor_pos = -1; }
        }
        return true;
    };
    auto fill = [&]() { while (pu_issued < pu_done + STAGES && issue_group()) {} };

    // the first item: its pages may be asked for before the dependency wait; its query, and anything
    // of the item after it, only after
    while (pu_issued < STAGES && cursor_item == 0) issue_group();
    load_tables(cur, 0);
    if (!waited) { ssb_pdl_wait(); waited = true; }
    load_query(cur, 0);
    cp_async_commit();
    fill();

    while (true) {
        const int b = cur.b, kvh = cur.kvh, h0 = kvh * group, p = cur.p;
        const int key_lo = cur.key_lo, key_hi = cur.key_hi;
        const unsigned char* qb = qbufs + parity * QBUF_BYTES;
        cp_async_wait<0>();                                      // this item's query (and, harmlessly, the next one's)
        __syncthreads();

        // Query fragments, the B operand of S^T = K Q^T: head g (and, with two tiles of heads, g + 8),
        // this lane's dims 16 ks + 2t (+1, +8, +9).  Rotation pairs (d, d + HD/2) are both in this lane
        // (k-steps ks and ks + KS/2).  qf[ks][0], [2]: heads 0-7; [1], [3]: heads 8-15.
        uint32_t qf[KS][4];
        {
            float qa[2][KS][4];                                  // [tile of heads][k-step][element]
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int row = g + 8 * i;
                const unsigned char* qr = qb + Q_OFF + row * HD * 2;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t w0 = 0u, w1 = 0u;
                    if (row < group) {
                        w0 = *reinterpret_cast<const uint32_t*>(qr + (16 * ks + 2 * t) * 2);
                        w1 = *reinterpret_cast<const uint32_t*>(qr + (16 * ks + 2 * t + 8) * 2);
                    }
                    qa[i][ks][0] = bf16lo(w0); qa[i][ks][1] = bf16hi(w0);
                    qa[i][ks][2] = bf16lo(w1); qa[i][ks][3] = bf16hi(w1);
                }
            }
            if (FUSE) {
                const float* cs = reinterpret_cast<const float*>(qb + COS_OFF);
                const float* sn_ = reinterpret_cast<const float*>(qb + SIN_OFF);
#pragma unroll
                for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int idx = 16 * ks + 2 * t + (e & 1) + (e >> 1) * 8;      // < HD/2
                        const float c = cs[idx], sn = sn_[idx];
#pragma unroll
                        for (int i = 0; i < NT; ++i) {
                            const float x1 = qa[i][ks][e], x2 = qa[i][ks + KS / 2][e];
                            qa[i][ks][e] = x1 * c - x2 * sn;
                            qa[i][ks + KS / 2][e] = x1 * sn + x2 * c;
                        }
                    }
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                qf[ks][0] = pack2(qa[0][ks][0] * scale_log2, qa[0][ks][1] * scale_log2);
                qf[ks][2] = pack2(qa[0][ks][2] * scale_log2, qa[0][ks][3] * scale_log2);
                if (NT == 2) {
                    qf[ks][1] = pack2(qa[1][ks][0] * scale_log2, qa[1][ks][1] * scale_log2);
                    qf[ks][3] = pack2(qa[1][ks][2] * scale_log2, qa[1][ks][3] * scale_log2);
                } else {
                    qf[ks][1] = qf[ks][3] = 0u;
                }
            }
        }
        // O^T = V^T P^T: ot[jm][nt][e] is dim 16 jm + g + 8 (e >> 1) of head 8 nt + 2t + (e & 1)
        float ot[HD / 16][NT][4];
        float m_run[NT][2], l_run[NT][2];                        // per head 8 nt + 2t + c; l: this lane's keys' share of the sum
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m_run[nt][0] = m_run[nt][1] = -INFINITY;
            l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) { ot[j][nt][0] = ot[j][nt][1] = ot[j][nt][2] = ot[j][nt][3] = 0.f; }
        }

        for (int i = 0; i < cur.units; ++i) {
            if (i + STAGES < cur.units) {     // needed when this turn ends: a turn's arithmetic hides the load
                page_ahead = page_table[(size_t)cur.slot * max_pages + min(cur.pf + i + STAGES, cur.page_hi)];
                page_ahead_of = i + STAGES;
            }
            const int stage = pu_done % STAGES;
            const bool landed = mbar_wait(full0 + 8 * stage, (pu_done / STAGES) & 1, abort_flag);
            if (!landed) abort_flag[0] = 1;
            if (!__syncthreads_and(landed)) { dead = true; break; }
            const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(smem + stage * TILE_BYTES);
            const uint32_t vbase = (uint32_t)__cvta_generic_to_shared(smem + (STAGES + stage) * TILE_BYTES);
            const int key0 = ((cur.pf + i) << 6) + 16 * warp;    // this warp's 16 keys of the page
            if (key0 <= key_hi && key0 + 15 >= key_lo) {
                // S^T = K Q^T: the page's 16 keys of this warp are the rows (all 16 used), the heads the columns
                float st[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) { st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.f; }
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t a0, a1, a2, a3;
                    const int key = 16 * warp + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4(kbase + adm_tile_offset(key, ks * 2 + (lane >> 4)), a0, a1, a2, a3);
                    mma16816(st[0], a0, a1, a2, a3, qf[ks][0], qf[ks][2]);
                    if (NT == 2) mma16816(st[NT - 1], a0, a1, a2, a3, qf[ks][1], qf[ks][3]);
                }
                // st[nt][e]: key key0 + g + 8 (e >> 1), head 8 nt + 2t + (e & 1)
                float m_new[NT][2], alpha[NT][2], row_sum[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    m_new[nt][0] = m_run[nt][0]; m_new[nt][1] = m_run[nt][1];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + g + 8 * (e >> 1);
                        const float v = (key >= key_lo && key <= key_hi) ? st[nt][e] : -INFINITY;
                        st[nt][e] = v;
                        m_new[nt][e & 1] = fmaxf(m_new[nt][e & 1], v);
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) {                // over the 16 keys: the lanes that differ in g
                        m_new[nt][c] = fmaxf(m_new[nt][c], __shfl_xor_sync(0xffffffffu, m_new[nt][c], 4));
                        m_new[nt][c] = fmaxf(m_new[nt][c], __shfl_xor_sync(0xffffffffu, m_new[nt][c], 8));
                        m_new[nt][c] = fmaxf(m_new[nt][c], __shfl_xor_sync(0xffffffffu, m_new[nt][c], 16));
                        alpha[nt][c] = (m_new[nt][c] == -INFINITY) ? 1.f : exp2f(m_run[nt][c] - m_new[nt][c]);
                        row_sum[nt][c] = 0.f;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = e & 1;
                        const float pj = (m_new[nt][c] == -INFINITY) ? 0.f : exp2f(st[nt][e] - m_new[nt][c]);
                        st[nt][e] = pj;
                        row_sum[nt][c] += pj;
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) { l_run[nt][c] = l_run[nt][c] * alpha[nt][c] + row_sum[nt][c]; m_run[nt][c] = m_new[nt][c]; }
#pragma unroll
                    for (int j = 0; j < HD / 16; ++j) {
                        ot[j][nt][0] *= alpha[nt][0]; ot[j][nt][1] *= alpha[nt][1];
                        ot[j][nt][2] *= alpha[nt][0]; ot[j][nt][3] *= alpha[nt][1];
                    }
                }
                // P^T as the B operand (keys 2t, 2t + 1 (+ 8) of head g): the 8 x 8 halves of the scores, transposed
                uint32_t pb0[NT], pb1[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    pb0[nt] = adm_transpose8(pack2(st[nt][0], st[nt][1]));
                    pb1[nt] = adm_transpose8(pack2(st[nt][2], st[nt][3]));
                }
                // O^T += V^T P^T: 16 dims a tile are the rows
#pragma unroll
                for (int jm = 0; jm < HD / 16; ++jm) {
                    uint32_t a0, a1, a2, a3;
                    const int mi = lane >> 3;
                    const int key = 16 * warp + (lane & 7) + ((mi >> 1) << 3);
                    ldmatrix_x4_trans(vbase + adm_tile_offset(key, jm * 2 + (mi & 1)), a0, a1, a2, a3);
                    mma16816(ot[jm][0], a0, a1, a2, a3, pb0[0], pb1[0]);
                    if (NT == 2) mma16816(ot[jm][NT - 1], a0, a1, a2, a3, pb0[NT - 1], pb1[NT - 1]);
                }
            }
            __syncthreads();                                     // the stage may be refilled
            ++pu_done;
            fill();                                              // this item's next pages, or the next item's query and pages
        }
        if (dead) break;

        if (FUSE && cur.owns_new && warp == 0) {
            // the token's own key and value, from the projection's output; all of this is lane-local
            const unsigned char* k_src = qb + KN_OFF;
            const unsigned char* v_src = qb + VN_OFF;
            const float* cs = reinterpret_cast<const float*>(qb + COS_OFF);
            const float* sn_ = reinterpret_cast<const float*>(qb + SIN_OFF);
            float kn[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const uint32_t w0 = *reinterpret_cast<const uint32_t*>(k_src + (16 * ks + 2 * t) * 2);
                const uint32_t w1 = *reinterpret_cast<const uint32_t*>(k_src + (16 * ks + 2 * t + 8) * 2);
                kn[ks][0] = bf16lo(w0); kn[ks][1] = bf16hi(w0); kn[ks][2] = bf16lo(w1); kn[ks][3] = bf16hi(w1);
            }
#pragma unroll
            for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int idx = 16 * ks + 2 * t + (e & 1) + (e >> 1) * 8;
                    const float c = cs[idx], sn = sn_[idx];
                    const float x1 = kn[ks][e], x2 = kn[ks + KS / 2][e];
                    kn[ks][e] = __bfloat162float(__float2bfloat16_rn(x1 * c - x2 * sn));          // as the cache holds it
                    kn[ks + KS / 2][e] = __bfloat162float(__float2bfloat16_rn(x1 * sn + x2 * c));
                }
            const int page = page_table[(size_t)cur.slot * max_pages + (p >> 6)];
            const size_t row = ((((size_t)page * n_kv + kvh) << 6) + (p & 63)) * HD;
            if (g == 0) {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    *reinterpret_cast<uint32_t*>(k_cache + row + 16 * ks + 2 * t) = pack2(kn[ks][0], kn[ks][1]);
                    *reinterpret_cast<uint32_t*>(k_cache + row + 16 * ks + 2 * t + 8) = pack2(kn[ks][2], kn[ks][3]);
                }
            }
            // the token's value: four dims a lane, copied into the cache as they are
            for (int d = lane * 4; d < HD; d += 128)
                *reinterpret_cast<uint2*>(v_cache + row + d) = *reinterpret_cast<const uint2*>(v_src + d * 2);
            // scores (log2 domain) of head g, and g + 8, from the query fragments; then each lane fetches
            // those of its own heads 2t, 2t + 1 from the lanes that hold them
            float sn2[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                sn2[nt] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
                    sn2[nt] += bf16lo(qf[ks][nt]) * kn[ks][0] + bf16hi(qf[ks][nt]) * kn[ks][1]
                             + bf16lo(qf[ks][2 + nt]) * kn[ks][2] + bf16hi(qf[ks][2 + nt]) * kn[ks][3];
                sn2[nt] += __shfl_xor_sync(0xffffffffu, sn2[nt], 1);
                sn2[nt] += __shfl_xor_sync(0xffffffffu, sn2[nt], 2);
            }
            float pn[NT][2], al[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float sc_new = __shfl_sync(0xffffffffu, sn2[nt], (2 * t + c) * 4);
                    const float m_new = fmaxf(m_run[nt][c], sc_new);
                    al[nt][c] = exp2f(m_run[nt][c] - m_new);     // exp2(-inf) = 0 when nothing came before
                    pn[nt][c] = exp2f(sc_new - m_new);
                    l_run[nt][c] = l_run[nt][c] * al[nt][c] + (g == 0 ? pn[nt][c] : 0.f);   // l is shared out over the keys' lanes: count once
                    m_run[nt][c] = m_new;
                }
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) {
                const float v0 = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(v_src)[16 * j + g]);
                const float v1 = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(v_src)[16 * j + g + 8]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    ot[j][nt][0] = fmaf(pn[nt][0], v0, ot[j][nt][0] * al[nt][0]); ot[j][nt][1] = fmaf(pn[nt][1], v0, ot[j][nt][1] * al[nt][1]);
                    ot[j][nt][2] = fmaf(pn[nt][0], v1, ot[j][nt][2] * al[nt][0]); ot[j][nt][3] = fmaf(pn[nt][1], v1, ot[j][nt][3] * al[nt][1]);
                }
            }
        }

        // merge the 4 warps (each saw different keys) in warp order
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float l = l_run[nt][c];
                l += __shfl_xor_sync(0xffffffffu, l, 4);
                l += __shfl_xor_sync(0xffffffffu, l, 8);
                l += __shfl_xor_sync(0xffffffffu, l, 16);
                const int head = 8 * nt + 2 * t + c;
                if (g == 0 && head < ADM_ROWS) { sm_m[warp][head] = m_run[nt][c]; sm_l[warp][head] = l; }
            }
#pragma unroll
        for (int j = 0; j < HD / 16; ++j)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int head = 8 * nt + 2 * t + (e & 1), dim = 16 * j + g + 8 * (e >> 1);
                    if (head < group) sm_acc[((size_t)warp * group + head) * ACC_LD + dim] = ot[j][nt][e];
                }
        __syncthreads();
        const int n_chunks = cur.n_chunks;
        for (int e = threadIdx.x; e < group * (HD / 4); e += ADM_THREADS) {
            const int row = e / (HD / 4), d = (e % (HD / 4)) * 4;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < ADM_WARPS; ++w) mm = fmaxf(mm, sm_m[w][row]);
            float ll = 0.f, a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < ADM_WARPS; ++w) {
                const float f = (sm_m[w][row] == -INFINITY) ? 0.f : exp2f(sm_m[w][row] - mm);
                ll += sm_l[w][row] * f;
                const float4 v = *reinterpret_cast<const float4*>(sm_acc + ((size_t)w * group + row) * ACC_LD + d);
                a[0] += v.x * f; a[1] += v.y * f; a[2] += v.z * f; a[3] += v.w * f;
            }
            if (n_chunks == 1) {
                const float inv = ll > 0.f ? 1.f / ll : 0.f;
                uint2 w;
                w.x = pack2(a[0] * inv, a[1] * inv);
                w.y = pack2(a[2] * inv, a[3] * inv);
                *reinterpret_cast<uint2*>(out + (size_t)b * ldo + (size_t)(h0 + row) * HD + d) = w;
            } else if (CL) {
                // the chunk's result stays in this block's shared memory (over the first warp's sums, which
                // only this thread has read) for the cluster to merge
                *reinterpret_cast<float4*>(sm_acc + (size_t)row * ACC_LD + d) = make_float4(a[0], a[1], a[2], a[3]);
                if (d == 0) cl_ml[row] = make_float2(mm, ll);
            } else {
                float* part = scratch + (((size_t)b * n_q + h0 + row) * max_chunks + cur.chunk) * ADM_PITCH(HD);
                *reinterpret_cast<float4*>(part + d) = make_float4(a[0], a[1], a[2], a[3]);
                if (d == 0) *reinterpret_cast<float2*>(part + HD) = make_float2(mm, ll);
            }
        }
        __syncthreads();                                         // the sums are read, the partial results written
        settle();                                                // the chunk counted an item ago: was it the last?
        if (!CL && n_chunks > 1) {
            // The block's partial results are ordered before the count by the barrier above and one
            // fence (cumulative at device scope) in the thread that counts.
            if (threadIdx.x == 0) {
                __threadfence();
                pend_arrived = atomicAdd(counters + (size_t)b * n_kv + kvh, 1);
            }
            pend_b = b; pend_kvh = kvh; pend_chunks = n_chunks;
        }

        // next item: the window moves on
        if (!has_nxt) break;
        item += G;
        cur = nxt;
        nxt = nn;
        has_nxt = has_nn;
        parity ^= 1;
        --cursor_item;                                           // what pointed at nxt now points at cur
        fill();
        has_nn = item + 2 * G < total_items;
        if (has_nn) decode(item + 2 * G, nn);
    }
    cp_async_wait<0>();
    if (CL && n_cl > 1) {
        // The cluster's blocks hold the chunks of one (sequence, kv head): after the barrier every block
        // merges a share of the output's elements from all blocks' shared memory, in chunk order, and
        // nobody leaves before all have read.  A block whose wait ran out still keeps both appointments.
        adm_cluster_sync();
        if (!dead) {
            const int crank = (int)adm_cluster_rank(), h0 = cur.kvh * group;
            for (int e = crank + n_cl * (int)threadIdx.x; e < group * (HD / 4); e += n_cl * ADM_THREADS) {
                const int row = e / (HD / 4), d = (e % (HD / 4)) * 4;
                float pm[8], pl[8];
                float4 pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool live = i < n_cl;
                    const float2 ml = adm_ld_cluster2(reinterpret_cast<const float*>(&cl_ml[row]), live ? i : 0);
                    pm[i] = live ? ml.x : -INFINITY;
                    pl[i] = ml.y;
                    pv[i] = adm_ld_cluster4(sm_acc + (size_t)row * ACC_LD + d, live ? i : 0);
                }
                float mm = -INFINITY;
#pragma unroll
                for (int i = 0; i < 8; ++i) mm = fmaxf(mm, pm[i]);
                float ll = 0.f, a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float f = (pm[i] == -INFINITY) ? 0.f : exp2f(pm[i] - mm);
                    ll = fmaf(pl[i], f, ll);
                    a[0] = fmaf(pv[i].x, f, a[0]); a[1] = fmaf(pv[i].y, f, a[1]);
                    a[2] = fmaf(pv[i].z, f, a[2]); a[3] = fmaf(pv[i].w, f, a[3]);
                }
                const float inv = ll > 0.f ? 1.f / ll : 0.f;
                uint2 w;
                w.x = pack2(a[0] * inv, a[1] * inv);
                w.y = pack2(a[2] * inv, a[3] * inv);
                *reinterpret_cast<uint2*>(out + (size_t)cur.b * ldo + (size_t)(h0 + row) * HD + d) = w;
            }
        }
        adm_cluster_sync();
    }
    if (!dead) { settle(); return; }
    // A page did not land in time: the launch's result is invalid and the host is told.  Loads that were
    // asked for may still arrive, so the block stays (for a bounded time) until its shared memory is quiet.
    if (threadIdx.x == 0) {
        atomicCAS(error_word, 0, TC_ERR_PRODUCER);
        for (int u = pu_done; u < pu_issued; ++u) mbar_wait(full0 + 8 * (u % STAGES), (u / STAGES) & 1, abort_flag + 1);
    }
    __syncthreads();
}

// Whether the tensor-core kernel takes this case (else attention_decode.cuh's kernel does).
static inline bool adm_supported(int n_q, int n_kv, int head_dim, int ldq, bool fuse) {
    return (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0 && n_q / n_kv <= ADM_ROWS &&
           ldq % 8 == 0;
}

// Scratch one launch needs: floats for the chunks' partial results, ints (zero on entry, left zero)
// for the arrival counters.
static inline long long adm_scratch_floats(int n_seqs, int n_q, int head_dim, int max_chunks) {
    return max_chunks > 1 ? (long long)n_seqs * n_q * max_chunks * ADM_PITCH(head_dim) : 0;
}
static inline int adm_counters(int n_seqs, int n_kv) { return n_seqs * n_kv; }

// Dynamic shared memory of a block: the ring's tiles (two stages of keys and values), the warps' sums, two
// query buffers, and three integers per sequence of the batch.  Head size 128 with four query heads
// per kv head and 64 sequences: 78 KB, so two blocks share an SM with room to spare.
static inline int adm_smem_bytes(int head_dim, int group, int n_seqs) {
    const int tiles = 2 * adm_stages(head_dim) * 64 * head_dim * 2, sums = ADM_WARPS * group * (head_dim + 4) * 4;
    const int query = group * head_dim * 2 + head_dim * 4 + head_dim * 4;
    return 1024 + tiles + sums + 2 * query + ((3 * n_seqs + 1) * 4 + 15) / 16 * 16;      // 1,024: the tiles' alignment
}

static inline int adm_sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        else
            return 148;
    }
    return sms;
}

// Blocks of the kernel that are resident at once on the current device (what the persistent grid is
// sized to): as many per SM as registers and shared memory allow, asked of the runtime once per case.
// The kernel's limit on dynamic shared memory only ever grows (a launch needs at most what was set).
template <int HD, bool FUSE, bool CL, int NT>
static inline cudaError_t adm_ensure_smem(int smem_bytes) {
    static int allowed = 0;
    if (smem_bytes <= allowed) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, FUSE, CL, NT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) allowed = smem_bytes;
    return e;
}

template <int HD, bool FUSE, int NT>
static inline int adm_blocks_per_sm(int smem_bytes) {
    auto kern = attention_decode_mma_kernel<HD, FUSE, false, NT>;
    if (adm_ensure_smem<HD, FUSE, false, NT>(smem_bytes) != cudaSuccess) return 0;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, ADM_THREADS, (size_t)smem_bytes) != cudaSuccess) return 0;
    return n;
}

static inline long long adm_resident_blocks(int head_dim, bool fuse, int group, int n_seqs) {
    static int cached[2][2][ADM_ROWS + 1][4];                    // [head size][fuse][group][batch class]
    const int cls = n_seqs <= 64 ? 0 : (n_seqs <= 256 ? 1 : (n_seqs <= 512 ? 2 : 3));
    const int cls_seqs = cls == 0 ? 64 : (cls == 1 ? 256 : (cls == 2 ? 512 : ADM_MAX_SEQS));
    if (group < 1 || group > ADM_ROWS || (head_dim != 64 && head_dim != 128)) return 0;
    int& per_sm = cached[head_dim == 128][fuse ? 1 : 0][group][cls];
    if (per_sm == 0) {
        const int smem = adm_smem_bytes(head_dim, group, cls_seqs);
        if (group <= 8)
            per_sm = head_dim == 64 ? (fuse ? adm_blocks_per_sm<64, true, 1>(smem) : adm_blocks_per_sm<64, false, 1>(smem))
                                    : (fuse ? adm_blocks_per_sm<128, true, 1>(smem) : adm_blocks_per_sm<128, false, 1>(smem));
        else
            per_sm = head_dim == 64 ? (fuse ? adm_blocks_per_sm<64, true, 2>(smem) : adm_blocks_per_sm<64, false, 2>(smem))
                                    : (fuse ? adm_blocks_per_sm<128, true, 2>(smem) : adm_blocks_per_sm<128, false, 2>(smem));
        if (per_sm <= 0) per_sm = -1;
    }
    return per_sm > 0 ? (long long)per_sm * adm_sm_count() : 0;
}

// Clusters of ``cluster`` blocks of the kernel that the device holds at once (0 if it cannot place one):
// what the runtime says for the kernel's registers and shared memory, asked once per case.
template <int HD, bool FUSE, int NT>
static inline int adm_max_clusters_of(int cluster, int smem_bytes) {
    auto kern = attention_decode_mma_kernel<HD, FUSE, true, NT>;
    if (adm_ensure_smem<HD, FUSE, true, NT>(smem_bytes) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(cluster * 64));
    cfg.blockDim = dim3(ADM_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

static inline int adm_max_clusters(int head_dim, bool fuse, int group, int cluster) {
    static int cached[2][2][2][4];                               // [head size][fuse][tiles of heads][cluster 2/4/8]
    if (group < 1 || group > ADM_ROWS || (head_dim != 64 && head_dim != 128)) return 0;
    const int ci = cluster == 2 ? 1 : (cluster == 4 ? 2 : (cluster == 8 ? 3 : 0));
    if (!ci) return 0;
    int& n = cached[head_dim == 128][fuse ? 1 : 0][group > 8][ci];
    if (n == 0) {
        const int smem = adm_smem_bytes(head_dim, group, 64);
        if (group <= 8)
            n = head_dim == 64 ? (fuse ? adm_max_clusters_of<64, true, 1>(cluster, smem) : adm_max_clusters_of<64, false, 1>(cluster, smem))
                               : (fuse ? adm_max_clusters_of<128, true, 1>(cluster, smem) : adm_max_clusters_of<128, false, 1>(cluster, smem));
        else
            n = head_dim == 64 ? (fuse ? adm_max_clusters_of<64, true, 2>(cluster, smem) : adm_max_clusters_of<64, false, 2>(cluster, smem))
                               : (fuse ? adm_max_clusters_of<128, true, 2>(cluster, smem) : adm_max_clusters_of<128, false, 2>(cluster, smem));
        if (n <= 0) n = -1;
    }
    return n > 0 ? n : 0;
}

// The tensor map of a cache (keys or values): cache_rows x head_dim bfloat16, boxes of one page's 64
// keys x 64 dims.  Encoding one costs the host a microsecond or two, so the maps of the caches seen
// so far are kept (a map depends on the address and the sizes alone).
struct AdmMapEntry { const void* base; long long rows; int head_dim; CUtensorMap map; };
static inline int adm_cache_map(const void* base, long long rows, int head_dim, CUtensorMap* map) {
    constexpr int KEPT = 256;
    static AdmMapEntry kept[KEPT];
    static int n_kept = 0;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_kept; ++i)
        if (kept[i].base == base && kept[i].rows == rows && kept[i].head_dim == head_dim) { *map = kept[i].map; return 0; }
    if (rows <= 0 || rows > 0x7fffffffLL) return SSB_ERR_BAD_SIZE;
    const int rc = make_map(map, base, (int)rows, head_dim, head_dim, 64);
    if (rc) return rc;
    if (n_kept == KEPT) n_kept = 0;
    kept[n_kept].base = base; kept[n_kept].rows = rows; kept[n_kept].head_dim = head_dim; kept[n_kept].map = *map;
    ++n_kept;
    return 0;
}

// chunk_pages: pages per chunk, or 0 for the kernel to size the chunks from the batch (see there);
// max_chunks: the most chunks a sequence is cut into (it sizes the scratch): a sequence that would need
// more gets max_chunks larger ones.  cache_rows: keys the caches have room for (pages x kv heads x 64);
// error_word: where a wait that ran out is recorded (zero otherwise).
// cluster > 1: every sequence is cut into that many chunks (2, 4 or 8), one block each, the chunks of a
// (sequence, kv head) forming a thread-block cluster that merges through its shared memory: no scratch,
// no counters, no trips to L2 for the merge.  For batches whose blocks all fit the device at once.
// Launch with the programmatic-dependent-launch attribute and the cluster size.
template <typename... KArgs, typename... Args>
static inline int adm_launch_cluster(void (*kernel)(KArgs...), dim3 grid, int cluster, size_t smem, cudaStream_t stream,
                                     bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ADM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int adm_launch(const void* q, int ldq, const void* k_cache, const void* v_cache, const int* pos,
                             const int* slot, const int* page_table, int max_pages, void* out, int ldo,
                             int n_seqs, int n_q, int n_kv, int head_dim, int window, float scale, int chunk_pages,
                             int max_chunks, float* scratch, int* counters, cudaStream_t stream, bool pdl,
                             const float* cos_t, const float* sin_t, long long cache_rows, int* error_word,
                             int cluster = 0) {
    typedef __nv_bfloat16 bf16;
    if (n_seqs <= 0) return 0;
    if (!error_word) return SSB_ERR_BAD_SIZE;
    if (cluster != 0 && cluster != 2 && cluster != 4 && cluster != 8) return SSB_ERR_BAD_SIZE;
    if (n_seqs > ADM_MAX_SEQS || chunk_pages < 0 || max_chunks < 1 ||
        (cluster == 0 && max_chunks > 1 && (!scratch || !counters)))
        return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)scratch) & 15) return SSB_ERR_BAD_SIZE;
    if (ldo % 4 || ((uintptr_t)out & 7)) return SSB_ERR_BAD_SIZE;      // four dims of a head leave as one 8-byte store
    const bool fuse = cos_t != nullptr;
    if (fuse && !sin_t) return SSB_ERR_BAD_SIZE;
    const float scale_log2 = scale * 1.4426950408889634f;
    const long long items = (long long)n_seqs * n_kv * max_chunks;
    const long long resident = adm_resident_blocks(head_dim, fuse, n_q / n_kv, n_seqs);
    if (resident <= 0) return SSB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(items < resident ? items : resident));
    if (cluster) {
        const long long blocks = (long long)n_seqs * n_kv * cluster;
        // the clusters' blocks are meant to run all at once
        if (blocks > resident || (long long)n_seqs * n_kv > adm_max_clusters(head_dim, fuse, n_q / n_kv, cluster)) return SSB_ERR_BAD_SIZE;
        grid = dim3((unsigned)blocks);
    }
    CUtensorMap map_k, map_v;
    int rc = adm_cache_map(k_cache, cache_rows, head_dim, &map_k);
    if (!rc) rc = adm_cache_map(v_cache, cache_rows, head_dim, &map_v);
    if (rc) return rc;
#define SSB_ADM(HD_, FUSE_, NT_) do { \
        const int smem_bytes = adm_smem_bytes(HD_, n_q / n_kv, n_seqs); \
        cudaError_t e = adm_ensure_smem<HD_, FUSE_, false, NT_>(smem_bytes); \
        if (e != cudaSuccess) return (int)e; \
        if (cluster) { \
            e = adm_ensure_smem<HD_, FUSE_, true, NT_>(smem_bytes); \
            if (e != cudaSuccess) return (int)e; \
            rc = adm_launch_cluster(attention_decode_mma_kernel<HD_, FUSE_, true, NT_>, grid, cluster, (size_t)smem_bytes, stream, pdl, \
                            (const bf16*)q, ldq, (bf16*)k_cache, (bf16*)v_cache, pos, slot, page_table, max_pages, \
                            (bf16*)out, ldo, n_seqs, n_q, n_kv, window, scale_log2, 1, cluster, scratch, \
                            counters, cos_t, sin_t, map_k, map_v, error_word); \
        } else \
        rc = ssb_launch(attention_decode_mma_kernel<HD_, FUSE_, false, NT_>, grid, dim3(ADM_THREADS), (size_t)smem_bytes, stream, pdl, \
                        (const bf16*)q, ldq, (bf16*)k_cache, (bf16*)v_cache, pos, slot, page_table, max_pages, \
                        (bf16*)out, ldo, n_seqs, n_q, n_kv, window, scale_log2, chunk_pages, max_chunks, scratch, \
                        counters, cos_t, sin_t, map_k, map_v, error_word); \
    } while (0)
#define SSB_ADM_NT(HD_, FUSE_) do { if (n_q / n_kv <= 8) SSB_ADM(HD_, FUSE_, 1); else SSB_ADM(HD_, FUSE_, 2); } while (0)
    if (head_dim == 64) { if (fuse) SSB_ADM_NT(64, true); else SSB_ADM_NT(64, false); }
    else if (head_dim == 128) { if (fuse) SSB_ADM_NT(128, true); else SSB_ADM_NT(128, false); }
    else return SSB_ERR_UNSUPPORTED;
#undef SSB_ADM_NT
#undef SSB_ADM
    return rc ? rc : ssb_launch_status();
}
