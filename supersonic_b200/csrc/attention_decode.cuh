// Decode attention for sm_100a: one query token per sequence over its paged keys and values.
//
// Grid (sequence, kv head x query-head group, split).  A block's 4 warps walk the split's keys,
// 8 keys per warp and turn, all 16 loads of a turn in flight before any is used; a lane owns VEC
// consecutive elements of the head dimension, so a key or value row is one coalesced load per
// warp.  Up to AD_GROUP query heads share each key and value.  Partial (max, sum, weighted
// values) go to scratch; the block that finishes last for a (sequence, head group) merges the
// splits in index order and writes the output.  Nothing waits on another block.
//
// Replaces supersonic_qwen35_full_attention_decode_*_kernel of the reference: one warp per
// query head, two passes over the keys (kernels/full_attention_cuda.cuh:476-679).
#pragma once
#include "common.cuh"
#include <math.h>

constexpr int AD_WARPS = 4;          // warps of a block when many blocks fill the GPU; 8 when few do
constexpr int AD_THREADS = AD_WARPS * 32;
constexpr int AD_GROUP = 4;
constexpr int AD_MAX_VEC = 8;
constexpr int AD_TOK = 8;            // keys per warp and turn
constexpr int AD_MAX_SPLITS = 64;

template <int VEC>
__device__ __forceinline__ void ad_load_row(const __nv_bfloat16* p, int lane, int head_dim, float (&v)[VEC]) {
    const int d = lane * VEC;
    if (d + VEC <= head_dim) {
        if (VEC == 8) {
            const uint4 q = *reinterpret_cast<const uint4*>(p + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        } else if (VEC == 4) {
            const uint2 q = *reinterpret_cast<const uint2*>(p + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
            for (int e = 0; e < 2; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        } else if (VEC == 2) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + d));
            v[0] = f.x; v[1] = f.y;
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = __bfloat162float(p[d + e]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = (d + e < head_dim) ? __bfloat162float(p[d + e]) : 0.f;
    }
}

// A lane's VEC elements of a row as raw bits.  The loads are volatile asm so that the compiler
// issues all of a turn's loads back to back and converts afterwards: a conversion right after
// each load would make every load wait for the one before it.
template <int VEC> struct AdRaw { uint32_t w[(VEC + 1) / 2]; };

template <int VEC, bool FULL = false>
__device__ __forceinline__ AdRaw<VEC> ad_load_raw(const __nv_bfloat16* p, int lane, int head_dim) {
    AdRaw<VEC> r;
    const int d = lane * VEC;
#pragma unroll
    for (int i = 0; i < (VEC + 1) / 2; ++i) r.w[i] = 0u;
    if (FULL || d + VEC <= head_dim) {                   // FULL: head_dim == 32 * VEC, no ragged lanes
        if (VEC == 8) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]) : "l"(p + d));
        } else if (VEC == 4) {
            asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.w[0]), "=r"(r.w[1]) : "l"(p + d));
        } else if (VEC == 2) {
            asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r.w[0]) : "l"(p + d));
        } else {
            unsigned short h;
            asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(h) : "l"(p + d));
            r.w[0] = h;
        }
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            if (d + e < head_dim) {
                unsigned short h;
                asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(h) : "l"(p + d + e));
                r.w[e / 2] |= (uint32_t)h << (16 * (e & 1));
            }
    }
    return r;
}

template <int VEC>
__device__ __forceinline__ void ad_unpack(const AdRaw<VEC>& r, float (&v)[VEC]) {
#pragma unroll
    for (int e = 0; e < VEC; ++e)
        v[e] = __uint_as_float(((r.w[e / 2] >> (16 * (e & 1))) & 0xffffu) << 16);      // bfloat16 -> float32
}

// FUSE: the rows of ``q`` are the raw output of the fused q/k/v projection
// ([q heads | k heads | v heads]); the kernel rotates the queries by the token's position, and
// the block that owns the token's page also rotates its key, writes key and value into the
// cache and attends to them from registers.  Needs head_dim == 32 * VEC and a full-width rotation.
template <int VEC, bool FUSE, bool FULL, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* k_cache,
                        __nv_bfloat16* v_cache, const int* __restrict__ pos,
                        const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages,
                        __nv_bfloat16* __restrict__ out, int ldo, int n_q, int n_kv, int head_dim, int page_shift,
                        int window, float scale, int n_splits, float* __restrict__ scratch,
                        int* __restrict__ counters, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t) {
    __shared__ float sm_m[NW][AD_GROUP], sm_l[NW][AD_GROUP];
    __shared__ float sm_acc[NW][AD_GROUP][32 * VEC];
    __shared__ int is_last;
    const int b = blockIdx.x, split = blockIdx.z;
    const int group = n_q / n_kv;
    const int groups_per_kv = (group + AD_GROUP - 1) / AD_GROUP;
    const int kvh = blockIdx.y / groups_per_kv, sub = blockIdx.y % groups_per_kv;
    const int h0 = kvh * group + sub * AD_GROUP;                 // first query head of this block
    const int n_heads = min(AD_GROUP, group - sub * AD_GROUP);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ssb_pdl_launch_dependents();
    // Without FUSE the predecessor (rope + append) wrote this step's key into the cache: wait
    // before reading anything.  With FUSE the cache holds earlier steps' keys only, and slots,
    // positions and page tables are written before the step starts: the first keys and values
    // are fetched before the wait, and only the query needs the predecessor.
    if (!FUSE) ssb_pdl_wait();
    const int s = slot[b];
    if (s < 0) {                                                 // padding row: zeros, no bookkeeping
        if (FUSE) ssb_pdl_wait();
        if (split == 0)
            for (int e = threadIdx.x; e < n_heads * head_dim; e += (NW * 32))
                out[(size_t)b * ldo + (size_t)h0 * head_dim + e] = __float2bfloat16_rn(0.f);
        return;
    }
    const int p = pos[b];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    // this split's keys: whole pages, split evenly
    const int page_lo = lo >> page_shift, page_hi = p >> page_shift;
    const int n_pages = page_hi - page_lo + 1;
    const int per = (n_pages + n_splits - 1) / n_splits;
    const int my_lo = max(lo, (page_lo + split * per) << page_shift);
    const bool owns_new = FUSE && my_lo <= p && p <= ((page_lo + (split + 1) * per) << page_shift) - 1;
    // with FUSE the token's own key is not in the cache yet: cached keys end at p - 1
    const int my_hi = min(FUSE ? p - 1 : p, ((page_lo + (split + 1) * per) << page_shift) - 1);

    const int* pt = page_table + (size_t)s * max_pages;
    const int page_mask = (1 << page_shift) - 1;
    constexpr int TURN = NW * AD_TOK;
    // one turn = AD_TOK keys of this warp: all loads are issued first, into raw registers
    // the block's page ids sit in the lanes of each warp (one global load up front) when there
    // are at most 32 of them; a key's page is then a shuffle away instead of a dependent load
    const int first_page = my_lo >> page_shift;
    const int n_my_pages = (max(my_hi, my_lo) >> page_shift) - first_page + 1;
    const bool pages_in_lanes = n_my_pages <= 32;
    const int lane_page = (pages_in_lanes && lane < n_my_pages && first_page + lane <= page_hi)
                              ? pt[first_page + lane] : 0;      // never past the sequence's last page
    auto issue = [&](int j0, AdRaw<VEC> (&k_raw)[AD_TOK], AdRaw<VEC> (&v_raw)[AD_TOK]) {
        size_t row[AD_TOK];
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u) {
            const int jj = min(j0 + u, my_hi);
            const int idx = jj >> page_shift;
            const int page = pages_in_lanes ? __shfl_sync(0xffffffffu, lane_page, idx - first_page) : pt[idx];
            row[u] = ((((size_t)page * n_kv + kvh) << page_shift) + (jj & page_mask)) * head_dim;
        }
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u) k_raw[u] = ad_load_raw<VEC, FULL>(k_cache + row[u], lane, head_dim);
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u) v_raw[u] = ad_load_raw<VEC, FULL>(v_cache + row[u], lane, head_dim);
    };
    AdRaw<VEC> ka[AD_TOK], va[AD_TOK];
    int j0 = my_lo + warp * AD_TOK;
    if (j0 <= my_hi) issue(j0, ka, va);
    // rotation of this lane's elements: pairs (i, i + head_dim/2) live in lanes l and l ^ 16.  The
    // tables are written by no kernel of the step: fetched before the wait as well.
    float rc[VEC], rs[VEC];
    if (FUSE) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const int i = (lane & 15) * VEC + e;
            rc[e] = cos_t[(size_t)p * (head_dim / 2) + i];
            rs[e] = (lane < 16 ? -1.f : 1.f) * sin_t[(size_t)p * (head_dim / 2) + i];
        }
    }
    if (FUSE) ssb_pdl_wait();                                    // the query (and this token's k, v) come from the predecessor
    float qv[AD_GROUP][VEC];
#pragma unroll
    for (int gi = 0; gi < AD_GROUP; ++gi) {
        if (gi < n_heads) {
            ad_load_row<VEC>(q + (size_t)b * ldq + (size_t)(h0 + gi) * head_dim, lane, head_dim, qv[gi]);
            if (FUSE) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float other = __shfl_xor_sync(0xffffffffu, qv[gi][e], 16);
                    qv[gi][e] = qv[gi][e] * rc[e] + other * rs[e];
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) qv[gi][e] *= scale;
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) qv[gi][e] = 0.f;
        }
    }
    float m[AD_GROUP], l[AD_GROUP], acc[AD_GROUP][VEC];
#pragma unroll
    for (int gi = 0; gi < AD_GROUP; ++gi) {
        m[gi] = -INFINITY; l[gi] = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[gi][e] = 0.f;
    }

    auto consume = [&](int j0, const AdRaw<VEC> (&k_raw)[AD_TOK], const AdRaw<VEC> (&v_raw)[AD_TOK]) {
        float sc[AD_TOK][AD_GROUP];
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u)
#pragma unroll
            for (int gi = 0; gi < AD_GROUP; ++gi) sc[u][gi] = 0.f;
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u) {
            float kr[VEC];
            ad_unpack<VEC>(k_raw[u], kr);
#pragma unroll
            for (int gi = 0; gi < AD_GROUP; ++gi)
#pragma unroll
                for (int e = 0; e < VEC; ++e) sc[u][gi] = fmaf(qv[gi][e], kr[e], sc[u][gi]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < AD_TOK; ++u)
#pragma unroll
                for (int gi = 0; gi < AD_GROUP; ++gi) sc[u][gi] += __shfl_xor_sync(0xffffffffu, sc[u][gi], o);
#pragma unroll
        for (int gi = 0; gi < AD_GROUP; ++gi) {
            float m_new = m[gi];
#pragma unroll
            for (int u = 0; u < AD_TOK; ++u)
                if (j0 + u <= my_hi) m_new = fmaxf(m_new, sc[u][gi]);
            const float alpha = __expf(m[gi] - m_new);            // exp(-inf) = 0 before the first key
            float lsum = l[gi] * alpha;
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[gi][e] *= alpha;
#pragma unroll
            for (int u = 0; u < AD_TOK; ++u) {
                const float pj = (j0 + u <= my_hi) ? __expf(sc[u][gi] - m_new) : 0.f;
                lsum += pj;
                sc[u][gi] = pj;
            }
            l[gi] = lsum;
            m[gi] = m_new;
        }
#pragma unroll
        for (int u = 0; u < AD_TOK; ++u) {
            float vr[VEC];
            ad_unpack<VEC>(v_raw[u], vr);
#pragma unroll
            for (int gi = 0; gi < AD_GROUP; ++gi)
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[gi][e] = fmaf(sc[u][gi], vr[e], acc[gi][e]);
        }
    };
    // one copy of the loop body (instruction fetch matters at this size): use a turn, then fetch the next
    // (a second set of registers for a turn in flight meanwhile was measured: no faster, the turn is
    // bound by its shuffles, and 190 registers a thread)
#pragma unroll 1
    while (j0 <= my_hi) {
        consume(j0, ka, va);
        j0 += TURN;
        if (j0 <= my_hi) issue(j0, ka, va);
    }

    if (FUSE && owns_new && warp == 0) {
        // the token's own key and value: from the projection's output, not from the cache
        const __nv_bfloat16* k_src = q + (size_t)b * ldq + (size_t)(n_q + kvh) * head_dim;
        const __nv_bfloat16* v_src = k_src + (size_t)n_kv * head_dim;
        AdRaw<VEC> k_raw = ad_load_raw<VEC, FULL>(k_src, lane, head_dim);
        const AdRaw<VEC> v_raw = ad_load_raw<VEC, FULL>(v_src, lane, head_dim);
        float kr[VEC], vr[VEC];
        ad_unpack<VEC>(k_raw, kr);
        ad_unpack<VEC>(v_raw, vr);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, kr[e], 16);
            kr[e] = __bfloat162float(__float2bfloat16_rn(kr[e] * rc[e] + other * rs[e]));   // as the cache will hold it
        }
        if (sub == 0) {
            const size_t row = ((((size_t)pt[p >> page_shift] * n_kv + kvh) << page_shift) + (p & page_mask)) * head_dim;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                k_cache[row + lane * VEC + e] = __float2bfloat16_rn(kr[e]);
                v_cache[row + lane * VEC + e] = __float2bfloat16_rn(vr[e]);
            }
        }
#pragma unroll
        for (int gi = 0; gi < AD_GROUP; ++gi) {
            float sc = 0.f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) sc = fmaf(qv[gi][e], kr[e], sc);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
            const float m_new = fmaxf(m[gi], sc);
            const float alpha = __expf(m[gi] - m_new), pj = __expf(sc - m_new);
            l[gi] = l[gi] * alpha + pj;
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[gi][e] = fmaf(pj, vr[e], acc[gi][e] * alpha);
            m[gi] = m_new;
        }
    }

    // merge the 4 warps in warp order
#pragma unroll
    for (int gi = 0; gi < AD_GROUP; ++gi) {
        if (lane == 0) { sm_m[warp][gi] = m[gi]; sm_l[warp][gi] = l[gi]; }
#pragma unroll
        for (int e = 0; e < VEC; ++e) sm_acc[warp][gi][lane * VEC + e] = acc[gi][e];
    }
    __syncthreads();
    const int width = 32 * VEC;
    // thread e of the block owns element (head gi, dim d) of the merged partial
    for (int e = threadIdx.x; e < n_heads * width; e += (NW * 32)) {
        const int gi = e / width, d = e % width;
        if (d >= head_dim) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sm_m[w][gi]);
        float ll = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = (sm_m[w][gi] == -INFINITY) ? 0.f : __expf(sm_m[w][gi] - mm);
            ll += sm_l[w][gi] * f;
            a += sm_acc[w][gi][d] * f;
        }
        if (n_splits == 1) {
            out[(size_t)b * ldo + (size_t)(h0 + gi) * head_dim + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
        } else {
            float* part = scratch + (((size_t)b * n_q + h0 + gi) * n_splits + split) * (head_dim + 2);
            part[d] = a;
            if (d == 0) { part[head_dim] = mm; part[head_dim + 1] = ll; }
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
        if (is_last) *counter = 0;                               // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // every thread owns elements (head gi, dim d) of the output and goes through the splits itself,
    // in split order, eight at a time so that their loads are in flight together: a split's
    // (max, sum) and its value for d; the factors exp(max_split - max_all) are cheap to recompute
    for (int e = threadIdx.x; e < n_heads * head_dim; e += (NW * 32)) {
        const int gi = e / head_dim, d = e % head_dim;
        const float* base = scratch + ((size_t)b * n_q + h0 + gi) * n_splits * (head_dim + 2);
        float mm = -INFINITY, ll = 0.f, a = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float pm[8], pl[8], pv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool live = s0 + i < n_splits;
                const float* part = base + (size_t)(live ? s0 + i : s0) * (head_dim + 2);
                pm[i] = live ? __ldcg(part + head_dim) : -INFINITY;
                pl[i] = __ldcg(part + head_dim + 1);
                pv[i] = __ldcg(part + d);
            }
            float m_new = mm;
#pragma unroll
            for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, pm[i]);
            const float keep = (mm == -INFINITY) ? 0.f : __expf(mm - m_new);
            ll *= keep; a *= keep;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float f = (pm[i] == -INFINITY) ? 0.f : __expf(pm[i] - m_new);
                ll = fmaf(pl[i], f, ll);
                a = fmaf(pv[i], f, a);
            }
            mm = m_new;
        }
        out[(size_t)b * ldo + (size_t)(h0 + gi) * head_dim + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
    }
}

// Scratch one launch needs: floats for the partial results, ints for the arrival counters.
static inline long long ad_scratch_floats(int n_seqs, int n_q, int head_dim, int n_splits) {
    return (long long)n_seqs * n_q * n_splits * (head_dim + 2);
}

static inline int ad_counters(int n_seqs, int n_q, int n_kv) {
    const int group = n_q / n_kv;
    return n_seqs * n_kv * ((group + AD_GROUP - 1) / AD_GROUP);
}

// Checks the sizes, picks the vector width and launches.  ``counters`` must be zero on entry
// (every launch leaves them zero); scratch and counters may be null when n_splits is 1.
static inline int ad_launch(const void* q, int ldq, const void* k_cache, const void* v_cache, const int* pos,
                            const int* slot, const int* page_table, int max_pages, void* out, int ldo,
                            int n_seqs, int n_q, int n_kv, int head_dim, int page_shift, int window,
                            float scale, int n_splits, float* scratch, int* counters, cudaStream_t stream,
                            bool pdl = false, const float* cos_t = nullptr, const float* sin_t = nullptr) {
    typedef __nv_bfloat16 bf16;
    if (n_seqs <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * AD_MAX_VEC || n_kv <= 0 || n_q % n_kv || n_splits < 1 ||
        n_splits > AD_MAX_SPLITS)
        return SSB_ERR_BAD_SIZE;
    const bool fuse = cos_t != nullptr;
    if (fuse && (!sin_t || head_dim % 32 || (head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256)))
        return SSB_ERR_UNSUPPORTED;
    if (n_splits > 1 && (!scratch || !counters)) return SSB_ERR_BAD_SIZE;
    const int group = n_q / n_kv;
    dim3 grid(n_seqs, n_kv * ((group + AD_GROUP - 1) / AD_GROUP), n_splits);
    const int vec = (head_dim + 31) / 32;
    int rc = 0;
#define SSB_AD_ARGS (const bf16*)q, ldq, (bf16*)k_cache, (bf16*)v_cache, pos, slot, page_table, max_pages, \
        (bf16*)out, ldo, n_q, n_kv, head_dim, page_shift, window, scale, n_splits, scratch, counters, cos_t, sin_t
    // few blocks (small batches): 8 warps each, so that a page of keys is one turn of the block
    const bool wide = (long long)grid.x * grid.y * grid.z <= 600;
#define SSB_AD_W(V, FUSE_, FULL_) \
    (wide ? ssb_launch(attention_decode_kernel<V, FUSE_, FULL_, 8>, grid, dim3(256), 0, stream, pdl, SSB_AD_ARGS) \
          : ssb_launch(attention_decode_kernel<V, FUSE_, FULL_, 4>, grid, dim3(128), 0, stream, pdl, SSB_AD_ARGS))
#define SSB_AD(V) \
    rc = fuse ? SSB_AD_W(V, true, true) : head_dim == 32 * V ? SSB_AD_W(V, false, true) : SSB_AD_W(V, false, false)
    // vector loads need VEC elements aligned: rows are head_dim * 2 bytes apart
    if (vec == 1) SSB_AD(1);
    else if (vec == 2 && head_dim % 2 == 0 && ldq % 2 == 0) SSB_AD(2);
    else if (vec <= 4 && head_dim % 4 == 0 && ldq % 4 == 0) SSB_AD(4);
    else if (vec <= 8 && head_dim % 8 == 0 && ldq % 8 == 0) SSB_AD(8);
    else return SSB_ERR_UNSUPPORTED;
#undef SSB_AD
#undef SSB_AD_W
#undef SSB_AD_ARGS
    return rc ? rc : ssb_launch_status();
}
