// Prefill attention for sm_100a: causal grouped-query attention of a ragged batch of new tokens
// over the paged cache, flash style: one block per (64 query rows, query head, sequence); keys
// and values arrive a page (64 tokens) at a time through a two-stage cp.async ring; scores and
// the weighted sum run on the tensor cores (mma.m16n8k16, bfloat16 in, float32 out); the softmax
// is online, in float32, one pass over the keys.  Keys are read from the cache, where this
// step's own keys already lie, so a prompt that continues a cached prefix needs nothing else.
//
// Replaces supersonic_qwen35_full_attention_prefill_kernel of the reference: one warp per
// (head, query) row found by an atomic counter, two passes over the keys, float32 output that a
// cast kernel then rounds (kernels/full_attention_cuda.cuh:360-474; bridge_cuda.cu:83-144, 1157-1180).
#include "common.cuh"
#include "mma_helpers.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int PA_BM = 64;            // query rows per block: 4 warps x 16
constexpr int PA_BN = 64;            // keys per turn = one cache page
constexpr int PA_THREADS = 128;

template <int HD>
__global__ void __launch_bounds__(PA_THREADS, 3)
prefill_attention_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, const int* __restrict__ cu_new,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                         const int* __restrict__ page_table, int max_pages, bf16* __restrict__ out, int ldo,
                         int n_q, int n_kv, int window, float scale_log2) {
    constexpr int CHUNKS = HD / 8;                       // 16-byte chunks per row
    constexpr int TILE_BYTES = PA_BN * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    // four tiles: K stage 0, K stage 1, V stage 0, V stage 1; the Q tile borrows V stage 1 until
    // its fragments are in registers (three blocks fit an SM this way)
    unsigned char* k_s = smem;                           // 2 stages
    unsigned char* v_s = smem + 2 * TILE_BYTES;          // 2 stages
    unsigned char* q_s = smem + 3 * TILE_BYTES;          // [64][HD], dead after the fragment load
    // long tiles (late queries see many keys) first, so that the tail of the grid is short work
    // blocks start in the order of blockIdx.x, then y: the longest tiles of all heads come first
    const int tile = (int)gridDim.y - 1 - (int)blockIdx.y, head = blockIdx.x % n_q, b = blockIdx.x / n_q;
    const int row0 = cu_new[b], n_new = cu_new[b + 1] - row0;
    if (tile * PA_BM >= n_new) return;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int start = seq_start[b];
    const int total = start + n_new;                     // keys the sequence holds after this step
    const int kvh = head / (n_q / n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int p0 = start + tile * PA_BM;                 // position of the tile's first query
    const int rows_here = min(PA_BM, n_new - tile * PA_BM);
    const int p_last = p0 + rows_here - 1;
    const int kb_lo = (window > 0 && p0 - window + 1 > 0) ? (p0 - window + 1) >> 6 : 0;
    const int kb_hi = p_last >> 6;
    const int* pt = page_table + (size_t)slot * max_pages;

    // Q tile -> shared memory (rows past the sequence's end are zero)
    for (int e = threadIdx.x; e < PA_BM * CHUNKS; e += PA_THREADS) {
        const int r = e / CHUNKS, c = e % CHUNKS;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_here)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + tile * PA_BM + r) * ldq + (size_t)head * HD + c * 8);
        *reinterpret_cast<uint4*>(q_s + tile_offset<HD>(r, c)) = v;
    }
    auto load_page = [&](int kb, int stage) {
        const size_t base = ((size_t)pt[kb] * n_kv + kvh) * (size_t)(PA_BN * HD);
        const uint32_t kd = (uint32_t)__cvta_generic_to_shared(k_s + stage * TILE_BYTES);
        const uint32_t vd = (uint32_t)__cvta_generic_to_shared(v_s + stage * TILE_BYTES);
        for (int e = threadIdx.x; e < PA_BN * CHUNKS; e += PA_THREADS) {
            const int r = e / CHUNKS, c = e % CHUNKS;
            cp_async16(kd + tile_offset<HD>(r, c), k_cache + base + (size_t)r * HD + c * 8);
            cp_async16(vd + tile_offset<HD>(r, c), v_cache + base + (size_t)r * HD + c * 8);
        }
        cp_async_commit();
    };
    load_page(kb_lo, 0);
    __syncthreads();

    // this warp's 16 query rows as A fragments, kept in registers for the whole loop
    uint32_t qf[HD / 16][4];
    {
        const uint32_t qb = (uint32_t)__cvta_generic_to_shared(q_s);
        const int r = warp * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
            ldmatrix_x4(qb + tile_offset<HD>(r, ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    __syncthreads();                                     // the Q tile's memory is V stage 1 from here on
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // positions of this thread's two rows (g and g + 8 of the warp's 16); -1 = no such query
    int pos_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + i * 8;
        pos_r[i] = r < rows_here ? p0 + r : -1;
    }

    for (int kb = kb_lo; kb <= kb_hi; ++kb) {
        const int stage = (kb - kb_lo) & 1;
        if (kb < kb_hi) { load_page(kb + 1, stage ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const uint32_t kbase = (uint32_t)__cvta_generic_to_shared(k_s + stage * TILE_BYTES);
        const uint32_t vbase = (uint32_t)__cvta_generic_to_shared(v_s + stage * TILE_BYTES);

        // S = Q K^T: 16 rows x 64 keys per warp
        float s[PA_BN / 8][4];
#pragma unroll
        for (int j = 0; j < PA_BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
#pragma unroll
            for (int jp = 0; jp < PA_BN / 16; ++jp) {            // two 8-key tiles per ldmatrix.x4
                uint32_t b0, b1, b2, b3;
                const int key = jp * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(kbase + tile_offset<HD>(key, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
                mma16816(s[2 * jp], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma16816(s[2 * jp + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }

        // mask (causal, window, end of sequence), scale, running maximum
        const int key0 = kb * PA_BN;
        const bool edge = (key0 + PA_BN - 1 > p0) || window > 0 || key0 + PA_BN > total;
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int j = 0; j < PA_BN / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                float v = s[j][e] * scale_log2;
                if (edge) {
                    const int key = key0 + j * 8 + 2 * t + (e & 1);
                    const bool seen = key <= pos_r[i] && (window <= 0 || key > pos_r[i] - window);
                    v = seen ? v : -INFINITY;
                }
                s[j][e] = v;
                m_new[i] = fmaxf(m_new[i], v);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
        }
        float alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i)
            alpha[i] = (m_new[i] == -INFINITY) ? 1.f : exp2f(m_run[i] - m_new[i]);   // nothing seen yet: keep zeros
#pragma unroll
        for (int j = 0; j < PA_BN / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const float p = (m_new[i] == -INFINITY) ? 0.f : exp2f(s[j][e] - m_new[i]);
                s[j][e] = p;
                row_sum[i] += p;
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l_run[i] = l_run[i] * alpha[i] + row_sum[i];       // quad lanes hold partial sums; joined at the end
            m_run[i] = m_new[i];
        }
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
        }

        // O += P V
#pragma unroll
        for (int ks = 0; ks < PA_BN / 16; ++ks) {
            const uint32_t a0 = pack2(s[2 * ks][0], s[2 * ks][1]), a1 = pack2(s[2 * ks][2], s[2 * ks][3]);
            const uint32_t a2 = pack2(s[2 * ks + 1][0], s[2 * ks + 1][1]), a3 = pack2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int jp = 0; jp < HD / 16; ++jp) {                 // two 8-wide slices of head_dim per ldmatrix.x4
                uint32_t b0, b1, b2, b3;
                const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldmatrix_x4_trans(vbase + tile_offset<HD>(key, jp * 2 + (lane >> 4)), b0, b1, b2, b3);
                mma16816(o[2 * jp], a0, a1, a2, a3, b0, b1);
                mma16816(o[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();                                        // the stage is free for the page after next
    }

    // finish: row sums across the quad, normalise, store
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + i * 8;
        if (r >= rows_here) continue;
        const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
        bf16* dst = out + (size_t)(row0 + tile * PA_BM + r) * ldo + (size_t)head * HD;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = pack2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
    }
}

// q: packed rows of new tokens [sum n_new, ldq] (query head h at column h * head_dim); cu_new
// [n_seqs + 1]: first row of each sequence; seq_start: keys each sequence held before this step
// (its new keys are already in the cache); max_new: longest run of new tokens.
SSB_API int ssb_attention_prefill(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                  const int* cu_new, const int* seq_start, const int* seq_slot,
                                  const int* page_table, int max_pages, void* out, int ldo, int n_seqs,
                                  int max_new, int n_q, int n_kv, int head_dim, int page_shift, int window,
                                  float scale, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (page_shift != 6 || n_kv <= 0 || n_q % n_kv || ldq % 8 || ldo % 2) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return SSB_ERR_BAD_SIZE;
    if ((max_new + PA_BM - 1) / PA_BM > 65535) return SSB_ERR_BAD_SIZE;
    dim3 grid(n_q * n_seqs, (max_new + PA_BM - 1) / PA_BM);
    const float scale_log2 = scale * 1.4426950408889634f;
#define SSB_PA(HD) do { \
        constexpr int smem = 4 * PA_BN * HD * 2; \
        static bool configured = false; \
        if (!configured) { \
            cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        prefill_attention_kernel<HD><<<grid, PA_THREADS, smem, stream>>>( \
            (const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, cu_new, seq_start, seq_slot, \
            page_table, max_pages, (bf16*)out, ldo, n_q, n_kv, window, scale_log2); \
    } while (0)
    if (head_dim == 64) SSB_PA(64);
    else if (head_dim == 128) SSB_PA(128);
    else return SSB_ERR_UNSUPPORTED;
#undef SSB_PA
    return ssb_launch_status();
}
