// Decode attention on the tensor cores, for head sizes 64 and 128 and up to 16 query heads per
// kv head: the query heads that share a kv head are the rows of one m16n8k16 tile, so a page of
// 64 keys costs a block 16 + 16 MMAs per warp instead of thousands of scalar instructions.
//
// Grid (sequence, kv head, split).  The block's 4 warps fetch a page of keys and values into
// shared memory together (cp.async, two stages, the swizzled tile layout of the prefill kernel);
// each warp then takes 16 of the page's 64 keys: S = Q K^T (16 x 16), online softmax in float32,
// O += P V.  Warps merge in shared memory, splits through scratch and the last block to arrive,
// exactly as in attention_decode.cuh (same scratch layout, maxima kept in the log2 domain).
// With FUSE the rows of q are the raw fused projection [q | k | v]: queries are rotated while
// the fragments are built, and the block that owns the token's page rotates its key, appends key
// and value to the cache and attends to them from registers.
//
// Replaces supersonic_qwen35_full_attention_decode_*_kernel of the reference (one warp per query
// head, two passes over the keys: kernels/full_attention_cuda.cuh:476-679).
#pragma once
#include "attention_decode.cuh"
#include "mma_helpers.cuh"

constexpr int ADM_WARPS = 4;
constexpr int ADM_THREADS = ADM_WARPS * 32;
constexpr int ADM_ROWS = 16;          // query heads per kv head, padded to the MMA's 16 rows
// Shared memory asked for beyond the four 16 KB tiles of head size 128: 80 KB a block lets two blocks
// share an SM, not three.  Measured inside decode steps of Llama-3.1-8B sizes: 3.44 ms a step at
// batch 8 with 76 to 113 KB a block, 3.50 ms with 64 to 72 KB, 3.61 ms with 128 KB (batch 64: 13.6k,
// 13.1k and 12.1k tokens/s).
constexpr int ADM_PAD_BYTES = 16384;

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <int HD, bool FUSE>
__global__ void __launch_bounds__(ADM_THREADS)
attention_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* k_cache,
                            __nv_bfloat16* v_cache, const int* __restrict__ pos, const int* __restrict__ slot,
                            const int* __restrict__ page_table, int max_pages, __nv_bfloat16* __restrict__ out,
                            int ldo, int n_q, int n_kv, int window, float scale_log2, int n_splits,
                            float* __restrict__ scratch, int* __restrict__ counters,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const char* __restrict__ prefetch_ptr, long long prefetch_bytes) {
    constexpr int CHUNKS = HD / 8, TILE_BYTES = 64 * HD * 2, KS = HD / 16, HALF = HD / 2;
    extern __shared__ __align__(128) unsigned char adm_smem[];   // K stage 0, K stage 1, V stage 0, V stage 1
    unsigned char* smem = adm_smem;
    __shared__ float sm_m[ADM_WARPS][ADM_ROWS], sm_l[ADM_WARPS][ADM_ROWS];
    __shared__ int is_last;
    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int group = n_q / n_kv, h0 = kvh * group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    ssb_pdl_launch_dependents();
    if (split >= n_splits) {
        // Extra blocks of the grid that only ask L2 to fetch a slice of the weights the next
        // kernels will stream.  They wait for the predecessor first: the point is to use the
        // memory system while attention waits on its small loads, not to compete with the
        // projection before it.  One SM can only feed so many of these requests, so they are
        // spread over many blocks.
        ssb_pdl_wait();
        const long long n_pre = (long long)gridDim.x * gridDim.y * (gridDim.z - n_splits);
        const long long me = ((long long)blockIdx.x * gridDim.y + blockIdx.y) * (gridDim.z - n_splits) + (split - n_splits);
        const long long slice = ((prefetch_bytes + n_pre - 1) / n_pre + 15) & ~15LL;
        const long long lo_b = me * slice, hi_b = min(lo_b + slice, prefetch_bytes & ~15LL);
        for (long long o = lo_b + (long long)threadIdx.x * 32768; o < hi_b; o += (long long)blockDim.x * 32768) {
            const unsigned n = (unsigned)min(32768LL, hi_b - o);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(prefetch_ptr + o), "r"(n) : "memory");
        }
        return;
    }
    if (!FUSE) ssb_pdl_wait();                                   // the cache holds this step's key already
    const int s = slot[b];
    if (s < 0) {                                                 // padding row
        if (FUSE) ssb_pdl_wait();
        if (split == 0)
            for (int e = threadIdx.x; e < group * HD; e += ADM_THREADS)
                out[(size_t)b * ldo + (size_t)h0 * HD + e] = __float2bfloat16_rn(0.f);
        return;
    }
    const int p = pos[b];
    const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int key_hi = FUSE ? p - 1 : p;                         // with FUSE the token's own key is not cached yet
    const int page_lo = key_lo >> 6, page_hi = p >> 6;
    const int per = (page_hi - page_lo + n_splits) / n_splits;   // ceil(pages / splits)
    const int pf = page_lo + split * per, pl = min(page_hi, pf + per - 1);
    const int n_my = pl - pf + 1;                                // pages of this split (<= 0: none)
    const bool owns_new = FUSE && pf <= page_hi && page_hi <= pl;
    const int* pt = page_table + (size_t)s * max_pages;

    auto load_page = [&](int i, int stage) {
        const size_t base = ((size_t)pt[pf + i] * n_kv + kvh) * (size_t)(64 * HD);
        const uint32_t kd = (uint32_t)__cvta_generic_to_shared(smem + stage * TILE_BYTES);
        const uint32_t vd = (uint32_t)__cvta_generic_to_shared(smem + (2 + stage) * TILE_BYTES);
        for (int e = threadIdx.x; e < 64 * CHUNKS; e += ADM_THREADS) {
            const int r = e / CHUNKS, c = e % CHUNKS;
            cp_async16(kd + tile_offset<HD>(r, c), k_cache + base + (size_t)r * HD + c * 8);
            cp_async16(vd + tile_offset<HD>(r, c), v_cache + base + (size_t)r * HD + c * 8);
        }
        cp_async_commit();
    };
    // earlier steps' keys: safe before the wait.  Both stages are filled here (a cp.async group each,
    // empty if there is no such page), so that two pages are on their way while the projection
    // before this kernel still runs.
    if (n_my > 0) load_page(0, 0); else cp_async_commit();
    if (n_my > 1) load_page(1, 1); else cp_async_commit();
    if (FUSE) ssb_pdl_wait();                                    // the query comes from the predecessor

    // Query fragments: row = head (g and g + 8), this lane's columns 16 ks + 2t (+1, +8, +9).
    // Rotation pairs (d, d + HD/2) are both in this lane (k-steps ks and ks + KS/2).
    uint32_t qf[KS][4];
    {
        float qa[2][KS][4];                                      // [row half][k-step][element]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = g + 8 * i;
            const __nv_bfloat16* qr = q + (size_t)b * ldq + (size_t)(h0 + row) * HD;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t w0 = 0u, w1 = 0u;
                if (row < group) {
                    w0 = *reinterpret_cast<const uint32_t*>(qr + 16 * ks + 2 * t);
                    w1 = *reinterpret_cast<const uint32_t*>(qr + 16 * ks + 2 * t + 8);
                }
                qa[i][ks][0] = bf16lo(w0); qa[i][ks][1] = bf16hi(w0);
                qa[i][ks][2] = bf16lo(w1); qa[i][ks][3] = bf16hi(w1);
            }
        }
        if (FUSE) {
#pragma unroll
            for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int idx = 16 * ks + 2 * t + (e & 1) + (e >> 1) * 8;          // < HD/2
                    const float c = cos_t[(size_t)p * HALF + idx], sn = sin_t[(size_t)p * HALF + idx];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float x1 = qa[i][ks][e], x2 = qa[i][ks + KS / 2][e];
                        qa[i][ks][e] = x1 * c - x2 * sn;
                        qa[i][ks + KS / 2][e] = x1 * sn + x2 * c;
                    }
                }
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = pack2(qa[0][ks][0] * scale_log2, qa[0][ks][1] * scale_log2);
            qf[ks][1] = pack2(qa[1][ks][0] * scale_log2, qa[1][ks][1] * scale_log2);
            qf[ks][2] = pack2(qa[0][ks][2] * scale_log2, qa[0][ks][3] * scale_log2);
            qf[ks][3] = pack2(qa[1][ks][2] * scale_log2, qa[1][ks][3] * scale_log2);
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // l: this lane's share of the row sum

    for (int i = 0; i < n_my; ++i) {
        const int stage = i & 1;
        cp_async_wait<1>();                                      // all but the newest group: page i is in
        __syncthreads();
        const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(smem + stage * TILE_BYTES);
        const uint32_t vbase = (uint32_t)__cvta_generic_to_shared(smem + (2 + stage) * TILE_BYTES);
        const int key0 = ((pf + i) << 6) + 16 * warp;            // this warp's 16 keys of the page
        if (key0 <= key_hi && key0 + 15 >= key_lo) {
            float sc[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b0, b1, b2, b3;
                const int key = 16 * warp + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(kbase + tile_offset<HD>(key, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
                mma16816(sc[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma16816(sc[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + 2 * t + (e & 1);
                    const float v = (key >= key_lo && key <= key_hi) ? sc[j][e] : -INFINITY;
                    sc[j][e] = v;
                    m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            }
            float alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) alpha[r] = (m_new[r] == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new[r]);
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const float pj = (m_new[r] == -INFINITY) ? 0.f : exp2f(sc[j][e] - m_new[r]);
                    sc[j][e] = pj;
                    row_sum[r] += pj;
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) { l_run[r] = l_run[r] * alpha[r] + row_sum[r]; m_run[r] = m_new[r]; }
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) { o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
            const uint32_t a0 = pack2(sc[0][0], sc[0][1]), a1 = pack2(sc[0][2], sc[0][3]);
            const uint32_t a2 = pack2(sc[1][0], sc[1][1]), a3 = pack2(sc[1][2], sc[1][3]);
#pragma unroll
            for (int jp = 0; jp < HD / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int key = 16 * warp + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldmatrix_x4_trans(vbase + tile_offset<HD>(key, jp * 2 + (lane >> 4)), b0, b1, b2, b3);
                mma16816(o[2 * jp], a0, a1, a2, a3, b0, b1);
                mma16816(o[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();                                         // the stage may be refilled
        if (i + 2 < n_my) load_page(i + 2, stage); else cp_async_commit();
    }
    cp_async_wait<0>();

    if (FUSE && owns_new && warp == 0) {
        // the token's own key and value, from the projection's output; all of this is lane-local
        const __nv_bfloat16* k_src = q + (size_t)b * ldq + (size_t)(n_q + kvh) * HD;
        const __nv_bfloat16* v_src = k_src + (size_t)n_kv * HD;
        float kn[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(k_src + 16 * ks + 2 * t);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(k_src + 16 * ks + 2 * t + 8);
            kn[ks][0] = bf16lo(w0); kn[ks][1] = bf16hi(w0); kn[ks][2] = bf16lo(w1); kn[ks][3] = bf16hi(w1);
        }
#pragma unroll
        for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int idx = 16 * ks + 2 * t + (e & 1) + (e >> 1) * 8;
                const float c = cos_t[(size_t)p * HALF + idx], sn = sin_t[(size_t)p * HALF + idx];
                const float x1 = kn[ks][e], x2 = kn[ks + KS / 2][e];
                kn[ks][e] = __bfloat162float(__float2bfloat16_rn(x1 * c - x2 * sn));          // as the cache holds it
                kn[ks + KS / 2][e] = __bfloat162float(__float2bfloat16_rn(x1 * sn + x2 * c));
            }
        const size_t row = ((((size_t)pt[p >> 6] * n_kv + kvh) << 6) + (p & 63)) * HD;
        if (g == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                *reinterpret_cast<uint32_t*>(k_cache + row + 16 * ks + 2 * t) = pack2(kn[ks][0], kn[ks][1]);
                *reinterpret_cast<uint32_t*>(k_cache + row + 16 * ks + 2 * t + 8) = pack2(kn[ks][2], kn[ks][3]);
            }
        }
        float sn2[2] = {0.f, 0.f};                               // scores of rows g and g + 8 (log2 domain)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            sn2[0] += bf16lo(qf[ks][0]) * kn[ks][0] + bf16hi(qf[ks][0]) * kn[ks][1]
                    + bf16lo(qf[ks][2]) * kn[ks][2] + bf16hi(qf[ks][2]) * kn[ks][3];
            sn2[1] += bf16lo(qf[ks][1]) * kn[ks][0] + bf16hi(qf[ks][1]) * kn[ks][1]
                    + bf16lo(qf[ks][3]) * kn[ks][2] + bf16hi(qf[ks][3]) * kn[ks][3];
        }
        float pn[2], al[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sn2[r] += __shfl_xor_sync(0xffffffffu, sn2[r], 1);
            sn2[r] += __shfl_xor_sync(0xffffffffu, sn2[r], 2);
            const float m_new = fmaxf(m_run[r], sn2[r]);
            al[r] = exp2f(m_run[r] - m_new);                     // exp2(-inf) = 0 when nothing came before
            pn[r] = exp2f(sn2[r] - m_new);
            l_run[r] = l_run[r] * al[r] + (t == 0 ? pn[r] : 0.f);   // l is shared out over the quad: count once
            m_run[r] = m_new;
        }
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            const uint32_t vw = *reinterpret_cast<const uint32_t*>(v_src + 8 * j + 2 * t);
            if (g == 0) *reinterpret_cast<uint32_t*>(v_cache + row + 8 * j + 2 * t) = vw;
            const float v0 = bf16lo(vw), v1 = bf16hi(vw);
            o[j][0] = fmaf(pn[0], v0, o[j][0] * al[0]); o[j][1] = fmaf(pn[0], v1, o[j][1] * al[0]);
            o[j][2] = fmaf(pn[1], v0, o[j][2] * al[1]); o[j][3] = fmaf(pn[1], v1, o[j][3] * al[1]);
        }
    }

    // merge the 4 warps (each saw different keys) in warp order; the stages are free now
    float* sm_acc = reinterpret_cast<float*>(smem);              // [ADM_WARPS][ADM_ROWS][HD]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        if (t == 0) { sm_m[warp][g + 8 * r] = m_run[r]; sm_l[warp][g + 8 * r] = l_run[r]; }
    }
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
        float* d0 = sm_acc + ((size_t)warp * ADM_ROWS + g) * HD + 8 * j + 2 * t;
        float* d1 = sm_acc + ((size_t)warp * ADM_ROWS + g + 8) * HD + 8 * j + 2 * t;
        d0[0] = o[j][0]; d0[1] = o[j][1]; d1[0] = o[j][2]; d1[1] = o[j][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < group * HD; e += ADM_THREADS) {
        const int row = e / HD, d = e % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < ADM_WARPS; ++w) mm = fmaxf(mm, sm_m[w][row]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < ADM_WARPS; ++w) {
            const float f = (sm_m[w][row] == -INFINITY) ? 0.f : exp2f(sm_m[w][row] - mm);
            ll += sm_l[w][row] * f;
            a += sm_acc[((size_t)w * ADM_ROWS + row) * HD + d] * f;
        }
        if (n_splits == 1) {
            out[(size_t)b * ldo + (size_t)(h0 + row) * HD + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
        } else {
            float* part = scratch + (((size_t)b * n_q + h0 + row) * n_splits + split) * (HD + 2);
            part[d] = a;
            if (d == 0) { part[HD] = mm; part[HD + 1] = ll; }
        }
    }
    if (n_splits == 1) return;

    // the block that arrives last merges the splits, in split order
    __threadfence();
    __syncthreads();
    int* counter = counters + (size_t)b * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(counter, 1);
        is_last = (arrived == n_splits - 1);
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // every thread owns elements (head, dim) of the output and goes through the splits itself, in
    // split order, eight at a time so that their loads are in flight together (see attention_decode.cuh)
    for (int e = threadIdx.x; e < group * HD; e += ADM_THREADS) {
        const int row = e / HD, d = e % HD;
        const float* base = scratch + ((size_t)b * n_q + h0 + row) * n_splits * (HD + 2);
        float mm = -INFINITY, ll = 0.f, a = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float pm[8], pl[8], pv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool live = s0 + i < n_splits;
                const float* part = base + (size_t)(live ? s0 + i : s0) * (HD + 2);
                pm[i] = live ? __ldcg(part + HD) : -INFINITY;
                pl[i] = __ldcg(part + HD + 1);
                pv[i] = __ldcg(part + d);
            }
            float m_new = mm;
#pragma unroll
            for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, pm[i]);
            const float keep = (mm == -INFINITY) ? 0.f : exp2f(mm - m_new);
            ll *= keep; a *= keep;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float f = (pm[i] == -INFINITY) ? 0.f : exp2f(pm[i] - m_new);
                ll = fmaf(pl[i], f, ll);
                a = fmaf(pv[i], f, a);
            }
            mm = m_new;
        }
        out[(size_t)b * ldo + (size_t)(h0 + row) * HD + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
    }
}

// Whether the tensor-core kernel takes this case (else attention_decode.cuh's kernel does).
static inline bool adm_supported(int n_q, int n_kv, int head_dim, int ldq, bool fuse) {
    return (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0 && n_q / n_kv <= ADM_ROWS &&
           ldq % 8 == 0;
}

static inline int adm_launch(const void* q, int ldq, const void* k_cache, const void* v_cache, const int* pos,
                             const int* slot, const int* page_table, int max_pages, void* out, int ldo,
                             int n_seqs, int n_q, int n_kv, int head_dim, int window, float scale, int n_splits,
                             float* scratch, int* counters, cudaStream_t stream, bool pdl, const float* cos_t,
                             const float* sin_t, const void* prefetch_ptr, long long prefetch_bytes) {
    typedef __nv_bfloat16 bf16;
    if (n_seqs <= 0) return 0;
    if (n_splits < 1 || n_splits > AD_MAX_SPLITS || (n_splits > 1 && (!scratch || !counters))) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return SSB_ERR_BAD_SIZE;
    const bool fuse = cos_t != nullptr;
    if (fuse && !sin_t) return SSB_ERR_BAD_SIZE;
    const float scale_log2 = scale * 1.4426950408889634f;
    const long long pre = (!prefetch_ptr || ((uintptr_t)prefetch_ptr & 15)) ? 0LL : prefetch_bytes;
    // about 128 extra blocks do the prefetching (see the kernel)
    const int extra = pre > 0 ? (128 + n_seqs * n_kv - 1) / (n_seqs * n_kv) : 0;
    dim3 grid(n_seqs, n_kv, n_splits + extra);
    int rc = 0;
#define SSB_ADM(HD_, FUSE_) do { \
        constexpr int smem_bytes = 4 * 64 * HD_ * 2 + (HD_ == 128 ? ADM_PAD_BYTES : 0); \
        static bool configured = false; \
        if (!configured) { \
            cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD_, FUSE_>, \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        rc = ssb_launch(attention_decode_mma_kernel<HD_, FUSE_>, grid, dim3(ADM_THREADS), (size_t)smem_bytes, stream, pdl, \
                        (const bf16*)q, ldq, (bf16*)k_cache, (bf16*)v_cache, pos, slot, page_table, max_pages, \
                        (bf16*)out, ldo, n_q, n_kv, window, scale_log2, n_splits, scratch, counters, cos_t, sin_t, \
                        (const char*)prefetch_ptr, pre); \
    } while (0)
    if (head_dim == 64) { if (fuse) SSB_ADM(64, true); else SSB_ADM(64, false); }
    else if (head_dim == 128) { if (fuse) SSB_ADM(128, true); else SSB_ADM(128, false); }
    else return SSB_ERR_UNSUPPORTED;
#undef SSB_ADM
    return rc ? rc : ssb_launch_status();
}
