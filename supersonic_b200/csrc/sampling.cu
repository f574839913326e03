// Sampling kernels: argmax, and temperature / top-k / top-p sampling of rows of float32 logits
// (one block per row; the sampling rule also on a cluster of 8 blocks per row, which is the one used: the row
// held in the cluster's shared memory when a cut has to be searched for, read in place when not).
//
// Rules follow the reference's samplers:
//   greedy      strict '>' so the lowest index wins ties
//               (crates/runner/src/decode_engine.rs:11162-11172;
//                kernels/prefill_helpers_bridge_cuda.cu:247-287)
//   sampling    logits * (1/T); keep the k largest; max-subtracted softmax; keep the smallest
//               set of most probable tokens whose mass reaches top_p; draw r = u * kept mass and
//               take the first token whose running sum reaches r
//               (crates/runner/src/qwen36_moe_decode.rs:1115-1185)
//   random u    xorshift64 (13, 7, 17), u = (state >> 40) / 2^24
//               (crates/runner/src/qwen36_moe_decode.rs:1085-1105)
// Differences, on purpose: nothing is sorted.  The k-th largest value and the top-p cut are
// found by bisection over the order-preserving integer image of the floats, every token
// tied with a cut is kept, and the running sum walks tokens in index order instead of
// probability order (the distribution is the same).  Each sequence owns its generator
// state, so a draw does not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned float_order_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = 0.f;
    const int n_warps = blockDim.x >> 5;
    for (int w = 0; w < n_warps; ++w) r += red[w];       // same order in every thread
    return r;
}

__device__ __forceinline__ float block_max(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = -INFINITY;
    const int n_warps = blockDim.x >> 5;
    for (int w = 0; w < n_warps; ++w) r = fmaxf(r, red[w]);
    return r;
}

// ---- argmax ----------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out) {
    __shared__ float best_v[SAMPLE_THREADS / 32];
    __shared__ int best_i[SAMPLE_THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }                  // ascending i per thread: first max kept
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;   // all -inf or NaN: token 0, as a host loop would
    }
}

SSB_API int ssb_argmax(const float* logits, long long ld, int n_rows, int vocab, int* out,
                       cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return SSB_ERR_BAD_SIZE;
    argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, out);
    return ssb_launch_status();
}

// ---- negative log-likelihood of given targets (teacher-forced scoring) ------------------------
// nll[r] = max + log(sum_i exp(x_i - max)) - x[target_r] over a row of float32 logits, the
// reference's formula (crates/runner/src/llama31_engine.rs:465-479 on the host in float64;
// kernels/prefill_helpers_bridge_cuda.cu:405-463 on the device from bfloat16 logits).  Sums are
// float32 with a fixed order: per thread ascending, then lanes, then warps.
__global__ void __launch_bounds__(SAMPLE_THREADS)
target_nll_kernel(const float* __restrict__ logits, long long ld, int vocab, const int* __restrict__ targets,
                  float* __restrict__ out) {
    __shared__ float red[SAMPLE_THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += SAMPLE_THREADS) m = fmaxf(m, row[i]);
    m = block_max(m, red);
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += SAMPLE_THREADS) sum += expf(row[i] - m);
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) {
        const int t = targets[blockIdx.x];
        out[blockIdx.x] = (t >= 0 && t < vocab) ? m + logf(sum) - row[t] : NAN;
    }
}

SSB_API int ssb_target_nll(const float* logits, long long ld, int n_rows, int vocab, const int* targets,
                           float* out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return SSB_ERR_BAD_SIZE;
    target_nll_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, targets, out);
    return ssb_launch_status();
}

// ---- temperature / top-k / top-p -------------------------------------------------------
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int vocab, float inv_temperature, int top_k,
              float top_p, const int* __restrict__ slots, unsigned long long* __restrict__ rng_state,
              int* __restrict__ out, float* __restrict__ drawn_u) {
    __shared__ float red[SAMPLE_THREADS / 32];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int found;
    const int tid = threadIdx.x;
    const float* row = logits + (size_t)blockIdx.x * ld;

    // one draw per row, from the sequence's own generator
    float u;
    {
        const int s = slots ? slots[blockIdx.x] : blockIdx.x;
        unsigned long long x = rng_state[s];
        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
        u = (float)(x >> 40) / 16777216.0f;
        __syncthreads();
        if (tid == 0) { rng_state[s] = x; if (drawn_u) drawn_u[blockIdx.x] = u; }
    }

    // cut 1: the k-th largest scaled logit (as an order key); 0 keeps everything
    unsigned cut = 0u;
    if (top_k > 0 && top_k < vocab) {
        unsigned lo = 0u, hi = 0xffffffffu;              // largest t with count(key >= t) >= k
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            float cnt = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS)
                cnt += (float_order_key(row[i] * inv_temperature) >= mid) ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)top_k) lo = mid; else hi = mid - 1u;
        }
        cut = lo;
    }

    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) mx = fmaxf(mx, row[i] * inv_temperature);
    mx = block_max(mx, red);

    float total = 0.f;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float x = row[i] * inv_temperature;
        if (float_order_key(x) >= cut) total += expf(x - mx);
    }
    total = block_sum(total, red);
    if (!(total > 0.f) || isinf(total) || isnan(total)) {          // degenerate row: greedy
        if (tid == 0) found = 0x7fffffff;
        __syncthreads();
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) if (row[i] > bv) { bv = row[i]; bi = i; }
        const float gm = block_max(bv, red);
        if (bv == gm && bi != 0x7fffffff) atomicMin(&found, bi);
        __syncthreads();
        if (tid == 0) out[blockIdx.x] = (found == 0x7fffffff) ? 0 : found;
        return;
    }

    // cut 2: the largest key t with mass(key >= t) >= top_p * total
    if (top_p < 1.0f) {
        const float need = top_p * total;
        unsigned lo = cut, hi = 0xffffffffu;
        while (lo < hi) {
            const unsigned mid = lo + (unsigned)(((unsigned long long)hi - lo + 1ull) >> 1);
            float mass = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float x = row[i] * inv_temperature;
                if (float_order_key(x) >= mid) mass += expf(x - mx);
            }
            mass = block_sum(mass, red);
            if (mass >= need) lo = mid; else hi = mid - 1u;
        }
        cut = lo;
    }

    // draw: contiguous chunk of indices per thread, running sum in index order
    const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(tid * per, vocab), end = min(begin + per, vocab);
    float mine = 0.f;
    for (int i = begin; i < end; ++i) {
        const float x = row[i] * inv_temperature;
        if (float_order_key(x) >= cut) mine += expf(x - mx);
    }
    chunk_sum[tid] = mine;
    if (tid == 0) found = 0x7fffffff;
    __syncthreads();
    float before = 0.f, kept = 0.f;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {            // same order in every thread
        if (t == tid) before = kept;
        kept += chunk_sum[t];
    }
    const float r = u * kept;
    // the intervals [before, before + mine] tile [0, kept], so some thread owns r
    if (mine > 0.f && before <= r && r <= before + mine) {
        float cum = before;
        int last = -1, hit = -1;
        for (int i = begin; i < end; ++i) {
            const float x = row[i] * inv_temperature;
            if (float_order_key(x) >= cut) {
                last = i;
                cum += expf(x - mx);
                if (cum >= r) { hit = i; break; }
            }
        }
        if (hit < 0) hit = last;                          // rounding left r a hair above this chunk's sum
        if (hit >= 0) atomicMin(&found, hit);
    }
    __syncthreads();
    if (tid == 0) out[blockIdx.x] = (found == 0x7fffffff) ? 0 : found;
}

// ---- the same rule on a cluster of blocks ---------------------------------------------------
// One block walking a row of 128k logits 30 to 60 times (a bisection step each) is bound by that
// block's path to L2: 320 us for top-k, 690 us for top-k and top-p.  Here a cluster of 8 blocks
// holds the row, scaled by 1/T, in its distributed shared memory (a slice each, read from global
// memory once); a bisection step sums over the slice and the 8 partial sums meet through shared
// memory of the cluster, in rank order, so every block takes the same decision.  The running sum
// of the draw goes through the slices in rank order: index order, as in the single-block kernel.
constexpr int SC_CTAS = 8;
constexpr int SC_THREADS = 512;

__device__ __forceinline__ unsigned sc_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float sc_remote_f32(const float* local, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

constexpr int SC_WAYS = 3;         // thresholds tried per search step: the range shrinks four times a step (1 and 7 measured slower)

struct ScShared {
    float red[2][SC_WAYS][SC_THREADS / 32];
    float pub[2][SC_WAYS];         // what this block publishes to the cluster
    float chunk_sum[SC_THREADS];
    int found;
};

// Sum (or maximum) over the cluster: every block gets the same value, combined in rank order.
// ``turn`` alternates between two sets of slots (every thread keeps its own copy, they agree by
// construction): a slot is written again only two meetings later, when nobody reads it any more.
template <bool MAX>
__device__ __forceinline__ float sc_all(float v, ScShared& sh, int& turn) {
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = MAX ? fmaxf(v, w) : v + w;
    }
    if ((threadIdx.x & 31) == 0) sh.red[turn][0][threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = MAX ? -INFINITY : 0.f;
        for (int w = 0; w < SC_THREADS / 32; ++w) m = MAX ? fmaxf(m, sh.red[turn][0][w]) : m + sh.red[turn][0][w];
        sh.pub[turn][0] = m;
    }
    sc_cluster_sync();                                   // every block's value is published
    float r = MAX ? -INFINITY : 0.f;
#pragma unroll
    for (unsigned c = 0; c < SC_CTAS; ++c) {
        const float o = sc_remote_f32(&sh.pub[turn][0], c);
        r = MAX ? fmaxf(r, o) : r + o;
    }
    turn ^= 1;
    return r;
}

// The same for SC_WAYS sums at once (one meeting of the cluster for all of them).
__device__ __forceinline__ void sc_all_sums(float (&v)[SC_WAYS], ScShared& sh, int& turn) {
#pragma unroll
    for (int k = 0; k < SC_WAYS; ++k) {
        for (int o = 16; o > 0; o >>= 1) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
        if ((threadIdx.x & 31) == 0) sh.red[turn][k][threadIdx.x >> 5] = v[k];
    }
    __syncthreads();
    if (threadIdx.x < SC_WAYS) {
        float m = 0.f;
        for (int w = 0; w < SC_THREADS / 32; ++w) m += sh.red[turn][threadIdx.x][w];
        sh.pub[turn][threadIdx.x] = m;
    }
    sc_cluster_sync();
#pragma unroll
    for (int k = 0; k < SC_WAYS; ++k) {
        float r = 0.f;
#pragma unroll
        for (unsigned c = 0; c < SC_CTAS; ++c) r += sc_remote_f32(&sh.pub[turn][k], c);
        v[k] = r;
    }
    turn ^= 1;
}

// One step of the search for the largest key t in [lo, hi] with f(t) >= need, f falling in t:
// SC_WAYS thresholds are tried at once (their sums f[0] >= f[1] >= ... are given), and the range
// shrinks to the part between two of them that holds the answer.
__device__ __forceinline__ void sc_thresholds(unsigned lo, unsigned hi, unsigned (&t)[SC_WAYS]) {
    const unsigned long long span = (unsigned long long)hi - lo;
#pragma unroll
    for (int k = 0; k < SC_WAYS; ++k) t[k] = lo + (unsigned)((span * (k + 1) + SC_WAYS) / (SC_WAYS + 1));   // > lo, <= hi, rising
}
__device__ __forceinline__ void sc_narrow(unsigned& lo, unsigned& hi, const unsigned (&t)[SC_WAYS],
                                          const float (&f)[SC_WAYS], float need) {
    int k = SC_WAYS - 1;
    while (k >= 0 && !(f[k] >= need)) --k;               // the highest threshold that still holds
    if (k + 1 < SC_WAYS) hi = t[k + 1] - 1u;
    if (k >= 0) lo = t[k];
}

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long ld, int vocab, float inv_temperature, int top_k,
                      float top_p, const int* __restrict__ slots, unsigned long long* __restrict__ rng_state,
                      int* __restrict__ out, float* __restrict__ drawn_u) {
    extern __shared__ float xs[];                        // this block's slice of the scaled logits
    __shared__ ScShared sh;
    const int tid = threadIdx.x, row_id = blockIdx.y;
    const unsigned rank = sc_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int per_cta = (vocab + SC_CTAS - 1) / SC_CTAS;
    const int lo_i = min((int)rank * per_cta, vocab), hi_i = min(lo_i + per_cta, vocab), n = hi_i - lo_i;
    int turn = 0;
    if (tid == 0) sh.found = 0x7fffffff;
    for (int i = tid; i < n; i += SC_THREADS) xs[i] = row[lo_i + i] * inv_temperature;

    // one draw per row, from the sequence's own generator (every block computes it; the first
    // block writes the new state back after the first meeting of the cluster)
    const int seq = slots ? slots[row_id] : row_id;
    unsigned long long state = rng_state[seq];
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    const float u = (float)(state >> 40) / 16777216.0f;
    __syncthreads();

    float mx = -INFINITY;
    for (int i = tid; i < n; i += SC_THREADS) mx = fmaxf(mx, xs[i]);
    mx = sc_all<true>(mx, sh, turn);
    if (rank == 0 && tid == 0) { rng_state[seq] = state; if (drawn_u) drawn_u[row_id] = u; }

    unsigned cut = 0u;
    if (top_k > 0 && top_k < vocab) {
        unsigned lo = 0u, hi = float_order_key(mx);      // the largest key there is
        while (lo < hi) {
            unsigned t[SC_WAYS];
            sc_thresholds(lo, hi, t);
            float cnt[SC_WAYS] = {};
            for (int i = tid; i < n; i += SC_THREADS) {
                const unsigned key = float_order_key(xs[i]);
#pragma unroll
                for (int k = 0; k < SC_WAYS; ++k) cnt[k] += (key >= t[k]) ? 1.f : 0.f;
            }
            sc_all_sums(cnt, sh, turn);
            sc_narrow(lo, hi, t, cnt, (float)top_k);
        }
        cut = lo;
    }
    float total = 0.f;
    for (int i = tid; i < n; i += SC_THREADS)
        if (float_order_key(xs[i]) >= cut) total += expf(xs[i] - mx);
    total = sc_all<false>(total, sh, turn);
    if (!(total > 0.f) || isinf(total) || isnan(total)) {                   // degenerate row: greedy, lowest index
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = tid; i < n; i += SC_THREADS) if (xs[i] > bv) { bv = xs[i]; bi = lo_i + i; }
        const float gm = sc_all<true>(bv, sh, turn);
        if (bv == gm && bi != 0x7fffffff) atomicMin(&sh.found, bi);
    } else {
        if (top_p < 1.0f) {
            const float need = top_p * total;
            unsigned lo = cut, hi = float_order_key(mx);
            while (lo < hi) {
                unsigned t[SC_WAYS];
                sc_thresholds(lo, hi, t);
                float mass[SC_WAYS] = {};
                for (int i = tid; i < n; i += SC_THREADS) {
                    const unsigned key = float_order_key(xs[i]);
                    if (key >= t[0]) {
                        const float e = expf(xs[i] - mx);
#pragma unroll
                        for (int k = 0; k < SC_WAYS; ++k) mass[k] += (key >= t[k]) ? e : 0.f;
                    }
                }
                sc_all_sums(mass, sh, turn);
                sc_narrow(lo, hi, t, mass, need);
            }
            cut = lo;
        }
        // draw: a contiguous chunk of the slice per thread; positions along the running sum are
        // P(thread) = (sum of the slices before) + (sum of the chunks before), and a thread owns
        // [P(thread), P(next thread)], so the intervals tile [0, kept] without gaps
        const int per = (n + SC_THREADS - 1) / SC_THREADS;
        const int begin = min(tid * per, n), end = min(begin + per, n);
        float mine = 0.f;
        for (int i = begin; i < end; ++i)
            if (float_order_key(xs[i]) >= cut) mine += expf(xs[i] - mx);
        sh.chunk_sum[tid] = mine;
        __syncthreads();
        float before = 0.f, slice_sum = 0.f;
        for (int t = 0; t < SC_THREADS; ++t) {           // same order in every thread
            if (t == tid) before = slice_sum;
            slice_sum += sh.chunk_sum[t];
        }
        if (tid == 0) sh.pub[turn][0] = slice_sum;
        sc_cluster_sync();
        float base = 0.f, kept = 0.f;
        for (unsigned c = 0; c < SC_CTAS; ++c) {
            if (c == rank) base = kept;
            kept += sc_remote_f32(&sh.pub[turn][0], c);
        }
        turn ^= 1;
        const float r = u * kept;
        const float p_lo = base + before;
        const float p_hi = (tid == SC_THREADS - 1) ? base + slice_sum : base + (before + mine);
        if (mine > 0.f && p_lo <= r && r <= p_hi) {
            float cum = p_lo;
            int last = -1, hit = -1;
            for (int i = begin; i < end; ++i)
                if (float_order_key(xs[i]) >= cut) {
                    last = i;
                    cum += expf(xs[i] - mx);
                    if (cum >= r) { hit = i; break; }
                }
            if (hit < 0) hit = last;                      // rounding left r a hair above this chunk's sum
            if (hit >= 0) atomicMin(&sh.found, lo_i + hit);
        }
    }
    // the lowest index found in any block
    sc_cluster_sync();
    if (rank == 0 && tid == 0) {
        int best = 0x7fffffff;
        for (unsigned c = 0; c < SC_CTAS; ++c) {
            unsigned addr = (unsigned)__cvta_generic_to_shared(&sh.found), remote;
            int v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(c));
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
            best = min(best, v);
        }
        out[row_id] = (best == 0x7fffffff) ? 0 : best;
    }
    sc_cluster_sync();                                   // no block leaves while its shared memory may be read
}

// ---- temperature alone: the row is read, not held --------------------------------------------
// Without a top-k or top-p cut nothing is searched for, so nothing needs the row in shared memory:
// two passes over the slice (maximum; sums of exponentials), two meetings of the cluster, and the
// one warp whose stretch of the running sum holds r = u * total looks at its 128 logits again.
// With no slice to hold, all 8 blocks of every row of a batch of 64 are resident at once (with
// 64 KB slices three blocks share an SM and 512 blocks come in two waves: 101 us; this form 23 us;
// one row: 26 and 12 us).
// The running sum goes in index order: a block takes its slice in stretches of 2,048 logits,
// a warp 128 of them, a lane 4; sums meet in that order (stretches through a scan over their sums).
constexpr int ST_EL = 4;                                 // logits in a row per lane
constexpr int ST_TILE = SC_THREADS * ST_EL;              // a stretch
constexpr int ST_MAX_IT = 32;                            // stretches per slice: one per lane of the warp that scans them
constexpr int ST_WARPS = SC_THREADS / 32;

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
sample_stream_kernel(const float* __restrict__ logits, long long ld, int vocab, float inv_temperature,
                     const int* __restrict__ slots, unsigned long long* __restrict__ rng_state,
                     int* __restrict__ out, float* __restrict__ drawn_u) {
    __shared__ ScShared sh;                              // chunk_sum holds [stretch][warp] here
    __shared__ float it_before[ST_MAX_IT];               // sum of the stretches before a stretch
    __shared__ float it_sum[ST_MAX_IT];
    __shared__ int sel_it, sel_warp;
    __shared__ float sel_before;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, row_id = blockIdx.y;
    const unsigned rank = sc_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int per_cta = (vocab + SC_CTAS - 1) / SC_CTAS;
    const int lo_i = min((int)rank * per_cta, vocab), hi_i = min(lo_i + per_cta, vocab), n = hi_i - lo_i;
    const int n_it = (n + ST_TILE - 1) / ST_TILE;
    int turn = 0;
    if (tid == 0) sh.found = 0x7fffffff;

    const int seq = slots ? slots[row_id] : row_id;
    unsigned long long state = rng_state[seq];
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    const float u = (float)(state >> 40) / 16777216.0f;

    float mx = -INFINITY;
    for (int it = 0; it < n_it; ++it) {
        const int i0 = (it * SC_THREADS + tid) * ST_EL;
#pragma unroll
        for (int e = 0; e < ST_EL; ++e)
            if (i0 + e < n) mx = fmaxf(mx, row[lo_i + i0 + e] * inv_temperature);
    }
    mx = sc_all<true>(mx, sh, turn);
    if (rank == 0 && tid == 0) { rng_state[seq] = state; if (drawn_u) drawn_u[row_id] = u; }

    // exponentials of lane's 4 logits of a stretch (0 beyond the slice)
    auto weights = [&](int it, float (&w)[ST_EL]) {
        const int i0 = (it * SC_THREADS + tid) * ST_EL;
#pragma unroll
        for (int e = 0; e < ST_EL; ++e) w[e] = (i0 + e < n) ? expf(row[lo_i + i0 + e] * inv_temperature - mx) : 0.f;
    };
    for (int it = 0; it < n_it; ++it) {
        float w[ST_EL];
        weights(it, w);
        float v = (w[0] + w[1]) + (w[2] + w[3]);
        // lanes in order: an inclusive scan, whose last lane holds the warp's sum as the draw will walk it
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += t;
        }
        if (lane == 31) sh.chunk_sum[it * ST_WARPS + warp] = v;
    }
    __syncthreads();
    float slice_sum = 0.f;
    if (warp == 0) {
        // lane = stretch: its warps in order, then the stretches by an inclusive scan
        float v = 0.f;
        if (lane < n_it)
            for (int w = 0; w < ST_WARPS; ++w) v += sh.chunk_sum[lane * ST_WARPS + w];
        float incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        it_before[lane] = incl - v;
        it_sum[lane] = v;
        slice_sum = __shfl_sync(0xffffffffu, incl, 31);
        if (lane == 0) sh.pub[turn][0] = slice_sum;
    }
    sc_cluster_sync();
    float base = 0.f, kept = 0.f;
    for (unsigned c = 0; c < SC_CTAS; ++c) {
        if (c == rank) base = kept;
        kept += sc_remote_f32(&sh.pub[turn][0], c);
    }
    const float mine = sc_remote_f32(&sh.pub[turn][0], rank);
    turn ^= 1;
    if (!(kept > 0.f) || isinf(kept) || isnan(kept)) {                       // degenerate row: greedy, lowest index
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int it = 0; it < n_it; ++it) {
            const int i0 = (it * SC_THREADS + tid) * ST_EL;
            for (int e = 0; e < ST_EL; ++e)
                if (i0 + e < n) { const float x = row[lo_i + i0 + e] * inv_temperature; if (x > bv) { bv = x; bi = lo_i + i0 + e; } }
        }
        const float gm = sc_all<true>(bv, sh, turn);
        if (bv == gm && bi != 0x7fffffff) atomicMin(&sh.found, bi);
    } else {
        const float r = u * kept;
        const bool owner = mine > 0.f && base <= r && r <= base + mine;      // the slices tile [0, kept]
        if (owner && warp == 0) {
            // the last stretch with any weight that starts at or before r, then the last such warp of it
            // (the first stretch with weight starts at base, which is not above r: there is one)
            const unsigned at = __ballot_sync(0xffffffffu, lane < n_it && it_sum[lane] > 0.f && base + it_before[lane] <= r);
            const int it = at ? 31 - __clz(at) : 0;
            float before = base + it_before[it];
            float run = before;
            for (int w = 0; w < lane && w < ST_WARPS; ++w) run += sh.chunk_sum[it * ST_WARPS + w];
            const unsigned aw = __ballot_sync(0xffffffffu, lane < ST_WARPS && sh.chunk_sum[it * ST_WARPS + min(lane, ST_WARPS - 1)] > 0.f && run <= r);
            const int w_sel = aw ? 31 - __clz(aw) : 0;
            before = __shfl_sync(0xffffffffu, run, w_sel);
            if (lane == 0) { sel_it = it; sel_warp = w_sel; sel_before = before; }
        }
        __syncthreads();
        if (owner && warp == sel_warp) {
            float w[ST_EL];
            weights(sel_it, w);
            const float v = (w[0] + w[1]) + (w[2] + w[3]);
            float incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const float start = sel_before + (incl - v);
            const int i0 = (sel_it * SC_THREADS + tid) * ST_EL;
            const unsigned al = __ballot_sync(0xffffffffu, v > 0.f && start <= r);
            if (al && lane == 31 - __clz(al)) {
                float cum = start;
                int last = -1, hit = -1;
#pragma unroll
                for (int e = 0; e < ST_EL; ++e)
                    if (hit < 0 && w[e] > 0.f) {
                        last = i0 + e;
                        cum += w[e];
                        if (cum >= r) hit = i0 + e;
                    }
                if (hit < 0) hit = last;                 // rounding left r a hair above this lane's sum
                if (hit >= 0) atomicMin(&sh.found, lo_i + hit);
            }
        }
    }
    sc_cluster_sync();
    if (rank == 0 && tid == 0) {
        int best = 0x7fffffff;
        for (unsigned c = 0; c < SC_CTAS; ++c) {
            unsigned addr = (unsigned)__cvta_generic_to_shared(&sh.found), remote;
            int v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(c));
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
            best = min(best, v);
        }
        out[row_id] = (best == 0x7fffffff) ? 0 : best;
    }
    sc_cluster_sync();                                   // no block leaves while its shared memory may be read
}

SSB_API int ssb_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature,
                       int top_k, float top_p, const int* slots, unsigned long long* rng_state, int* out,
                       float* drawn_u, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || vocab >= 0x40000000 || !(temperature > 0.f)) return SSB_ERR_BAD_SIZE;
    // temperature alone: nothing to search, the row stays where it is
    if ((top_k <= 0 || top_k >= vocab) && !(top_p < 1.0f) && n_rows <= 65535 &&
        (vocab + SC_CTAS - 1) / SC_CTAS <= ST_MAX_IT * ST_TILE) {
        sample_stream_kernel<<<dim3(SC_CTAS, n_rows), SC_THREADS, 0, stream>>>(
            logits, ld, vocab, 1.0f / temperature, slots, rng_state, out, drawn_u);
        return ssb_launch_status();
    }
    // a cluster of 8 blocks per row where the row's slices fit shared memory (vocabularies up to 400k)
    const size_t slice = (size_t)((vocab + SC_CTAS - 1) / SC_CTAS) * sizeof(float);
    if (slice <= 200 * 1024 && n_rows <= 65535) {
        static size_t configured = 0;
        if (slice > 48 * 1024 && slice > configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slice);
            if (e != cudaSuccess) return (int)e;
            configured = slice;
        }
        sample_cluster_kernel<<<dim3(SC_CTAS, n_rows), SC_THREADS, slice, stream>>>(
            logits, ld, vocab, 1.0f / temperature, top_k, top_p, slots, rng_state, out, drawn_u);
        return ssb_launch_status();
    }
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, 1.0f / temperature, top_k,
                                                         top_p, slots, rng_state, out, drawn_u);
    return ssb_launch_status();
}
