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
// found over the order-preserving integer image of the floats (a byte at a time on the cluster,
// by bisection in the one-block kernel), every token tied with a cut is kept, and the running
// sum walks tokens in index order instead of probability order (the distribution is the same).
// Each sequence owns its generator state, so a draw does not depend on what else is in the batch.
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
// One block walking a row of 128k logits 30 to 60 times (a search step each) is bound by that
// block's path to L2: 320 us for top-k, 690 us for top-k and top-p.  Here a cluster of 8 blocks
// shares the row (a slice each) and meets through the cluster's shared memory, always combining
// in rank order, so every block takes the same decisions.  The running sum of the draw goes through
// the slices in rank order and through a slice in index order: in stretches of 2,048 logits, of which
// a warp takes 128 and a lane 4; sums meet in that order (the stretches through a scan over their sums).
constexpr int SC_CTAS = 8;
constexpr int SC_THREADS = 512;
constexpr int SC_WARPS = SC_THREADS / 32;
constexpr int ST_EL = 4;                                 // logits in a row per lane
constexpr int ST_TILE = SC_THREADS * ST_EL;              // a stretch
constexpr int ST_MAX_IT = 32;                            // stretches per slice: one per lane of the warp that scans them

__device__ __forceinline__ unsigned sc_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned sc_remote_addr(const void* local, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ float sc_remote_f32(const float* local, unsigned rank) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(sc_remote_addr(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ unsigned sc_remote_u32(const unsigned* local, unsigned rank) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(sc_remote_addr(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ int sc_remote_s32(const int* local, unsigned rank) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(sc_remote_addr(local, rank)) : "memory");
    return v;
}

struct ScShared {
    float red[2][SC_WARPS];
    float pub[2];                  // what this block publishes to the cluster
    float part[ST_MAX_IT * SC_WARPS];   // sums of the draw: [stretch][warp]
    float it_before[ST_MAX_IT], it_sum[ST_MAX_IT];
    float sel_before;
    int sel_it, sel_warp;
    int found;
};

// Maximum over the cluster: every block gets the same value.  ``turn`` alternates between two sets of
// slots (every thread keeps its own copy, they agree by construction): a slot is written again only
// two meetings later, when nobody reads it any more.
__device__ __forceinline__ float sc_max(float v, ScShared& sh, int& turn) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh.red[turn][threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = -INFINITY;
        for (int w = 0; w < SC_WARPS; ++w) m = fmaxf(m, sh.red[turn][w]);
        sh.pub[turn] = m;
    }
    sc_cluster_sync();                                   // every block's value is published
    float r = -INFINITY;
#pragma unroll
    for (unsigned c = 0; c < SC_CTAS; ++c) r = fmaxf(r, sc_remote_f32(&sh.pub[turn], c));
    turn ^= 1;
    return r;
}

// The draw and the end of a row's kernel.  weights(it, w) gives this lane's 4 weights of stretch it
// (0 for what is cut or lies beyond the slice); argmax_of_mine() gives this thread's largest scaled logit
// and its index, for a row with nothing to draw from (no weight, or a sum that is not finite), which
// takes its largest logit, lowest index first.
template <typename Weights, typename Largest>
__device__ __forceinline__ void sc_draw(ScShared& sh, int& turn, unsigned rank, int n, int n_it, int lo_i, float u,
                                        int* __restrict__ out_row, Weights weights, Largest largest_of_mine) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int it = 0; it < n_it; ++it) {
        float w[ST_EL];
        weights(it, w);
        float v = (w[0] + w[1]) + (w[2] + w[3]);
        // lanes in order: an inclusive scan, whose last lane holds the warp's sum as the draw will walk it
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float q = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += q;
        }
        if (lane == 31) sh.part[it * SC_WARPS + warp] = v;
    }
    __syncthreads();
    if (warp == 0) {
        // lane = stretch: its warps in order, then the stretches by an inclusive scan
        float v = 0.f;
        if (lane < n_it)
            for (int w = 0; w < SC_WARPS; ++w) v += sh.part[lane * SC_WARPS + w];
        float incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float q = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += q;
        }
        sh.it_before[lane] = incl - v;
        sh.it_sum[lane] = v;
        if (lane == 31) sh.pub[turn] = incl;
    }
    sc_cluster_sync();
    float base = 0.f, kept = 0.f;
    for (unsigned c = 0; c < SC_CTAS; ++c) {
        if (c == rank) base = kept;
        kept += sc_remote_f32(&sh.pub[turn], c);
    }
    const float mine = sc_remote_f32(&sh.pub[turn], rank);
    turn ^= 1;
    if (!(kept > 0.f) || isinf(kept) || isnan(kept)) {
        float bv; int bi;
        largest_of_mine(bv, bi);
        const float gm = sc_max(bv, sh, turn);
        if (bv == gm && bi != 0x7fffffff) atomicMin(&sh.found, bi);
    } else {
        const float r = u * kept;
        const bool owner = mine > 0.f && base <= r && r <= base + mine;      // the slices tile [0, kept]
        if (owner && warp == 0) {
            // the last stretch with any weight that starts at or before r, then the last such warp of it
            // (the first stretch with weight starts at base, which is not above r: there is one)
            const unsigned at = __ballot_sync(0xffffffffu, lane < n_it && sh.it_sum[lane] > 0.f && base + sh.it_before[lane] <= r);
            const int it = at ? 31 - __clz(at) : 0;
            float run = base + sh.it_before[it];
            for (int w = 0; w < lane && w < SC_WARPS; ++w) run += sh.part[it * SC_WARPS + w];
            const unsigned aw = __ballot_sync(0xffffffffu, lane < SC_WARPS && sh.part[it * SC_WARPS + min(lane, SC_WARPS - 1)] > 0.f && run <= r);
            const int w_sel = aw ? 31 - __clz(aw) : 0;
            const float before = __shfl_sync(0xffffffffu, run, w_sel);
            if (lane == 0) { sh.sel_it = it; sh.sel_warp = w_sel; sh.sel_before = before; }
        }
        __syncthreads();
        if (owner && warp == sh.sel_warp) {
            float w[ST_EL];
            weights(sh.sel_it, w);
            const float v = (w[0] + w[1]) + (w[2] + w[3]);
            float incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float q = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += q;
            }
            const float start = sh.sel_before + (incl - v);
            const int i0 = (sh.sel_it * SC_THREADS + tid) * ST_EL;
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
    // the lowest index found in any block
    sc_cluster_sync();
    if (rank == 0 && tid == 0) {
        int best = 0x7fffffff;
        for (unsigned c = 0; c < SC_CTAS; ++c) best = min(best, sc_remote_s32(&sh.found, c));
        *out_row = (best == 0x7fffffff) ? 0 : best;
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
__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
sample_stream_kernel(const float* __restrict__ logits, long long ld, int vocab, float inv_temperature,
                     const int* __restrict__ slots, unsigned long long* __restrict__ rng_state,
                     int* __restrict__ out, float* __restrict__ drawn_u) {
    __shared__ ScShared sh;
    const int tid = threadIdx.x, row_id = blockIdx.y;
    const unsigned rank = sc_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int per_cta = (vocab + SC_CTAS - 1) / SC_CTAS;
    const int lo_i = min((int)rank * per_cta, vocab), hi_i = min(lo_i + per_cta, vocab), n = hi_i - lo_i;
    const int n_it = (n + ST_TILE - 1) / ST_TILE;
    int turn = 0;
    if (tid == 0) sh.found = 0x7fffffff;

    // one draw per row, from the sequence's own generator (every block computes it; the first
    // block writes the new state back after the first meeting of the cluster)
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
    mx = sc_max(mx, sh, turn);
    if (rank == 0 && tid == 0) { rng_state[seq] = state; if (drawn_u) drawn_u[row_id] = u; }

    auto weights = [&](int it, float (&w)[ST_EL]) {
        const int i0 = (it * SC_THREADS + tid) * ST_EL;
#pragma unroll
        for (int e = 0; e < ST_EL; ++e) w[e] = (i0 + e < n) ? expf(row[lo_i + i0 + e] * inv_temperature - mx) : 0.f;
    };
    auto largest = [&](float& bv, int& bi) {
        bv = -INFINITY; bi = 0x7fffffff;
        for (int i = tid; i < n; i += SC_THREADS) {
            const float x = row[lo_i + i] * inv_temperature;
            if (x > bv) { bv = x; bi = lo_i + i; }       // ascending i per thread: first maximum kept
        }
    };
    sc_draw(sh, turn, rank, n, n_it, lo_i, u, out + row_id, weights, largest);
}

// ---- with a cut: the slice in shared memory, the cuts by radix selection ------------------------
// The k-th largest scaled logit and the top-p cut are found a byte at a time, from the top: every
// block counts its slice's keys (for top-p: adds its weights) into 256 bins of the byte among the keys
// that share the bytes found so far, the cluster's bins are added up in rank order, and the bin in
// which the count (the mass) from the top reaches what is needed gives the next byte: four meetings
// of the cluster per cut, where a search that halves or quarters a range of keys takes 16 to 32
// (64 rows with top-k 40 and top-p 0.9: 330 us that way).  Weights are added as integers (their
// value times 2^40): the sum in a bin then does not depend on the order in which a block's threads
// reach it, and a draw is the same in every run.
struct RxShared {
    unsigned hist[2][3][256];      // a bin's sum in three pieces of 14 bits' weight each (plain 32-bit adds in shared memory)
    unsigned long long warp_sum[8];
    unsigned long long need, need_left;
    int bin;
};

// Adds into a bin: plain 32-bit adds in shared memory, which the hardware takes one after the other when
// lanes meet on a bin (a 64-bit add there is a compare-and-swap loop: four times the time of the whole
// search, measured).  A weight's 40-bit integer goes in three pieces of 14 bits' weight; a slice has at most
// 2^16 elements, so a piece's sum stays below 2^30.
template <bool COUNT>
__device__ __forceinline__ void rx_add(unsigned (*hist)[256], bool takes_part, unsigned bin, unsigned long long q) {
    if (!takes_part) return;
    if (COUNT) {
        atomicAdd(&hist[0][bin], 1u);
    } else {
        atomicAdd(&hist[0][bin], (unsigned)(q & 0x3fffull));
        atomicAdd(&hist[1][bin], (unsigned)((q >> 14) & 0x3fffull));
        atomicAdd(&hist[2][bin], (unsigned)(q >> 28));
    }
}

// One byte of a cut.  Every thread has added its elements into rx.hist[buf] before.  Returns the bin b
// with S(b) >= need > S(b + 1), S(b) being what bins b.. hold over the whole cluster, and lowers need by
// S(b + 1).  top_fraction >= 0: need is first set to that fraction of everything counted (at least 1).
template <bool COUNT>
__device__ __forceinline__ int rx_byte(RxShared& rx, int buf, unsigned long long& need, float top_fraction) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __syncthreads();
    sc_cluster_sync();                                   // every block's bins are complete
    unsigned long long g = 0, v = 0;
    if (tid < 256) {
#pragma unroll
        for (unsigned c = 0; c < SC_CTAS; ++c) {
            g += (unsigned long long)sc_remote_u32(&rx.hist[buf][0][tid], c);
            if (!COUNT)
                g += ((unsigned long long)sc_remote_u32(&rx.hist[buf][1][tid], c) << 14) +
                     ((unsigned long long)sc_remote_u32(&rx.hist[buf][2][tid], c) << 28);
        }
        v = g;                                           // v = what this warp's bins from this one up hold
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long q = __shfl_down_sync(0xffffffffu, v, o);
            if (lane + o < 32) v += q;
        }
        if (lane == 0) rx.warp_sum[warp] = v;
    }
    __syncthreads();
    if (tid < 256) {
        for (int w = warp + 1; w < 8; ++w) v += rx.warp_sum[w];
        if (top_fraction >= 0.f && tid == 0) {
            unsigned long long nd = (unsigned long long)((double)top_fraction * (double)v);
            rx.need = nd > 0 ? nd : 1;
        }
    }
    __syncthreads();
    if (top_fraction >= 0.f) need = rx.need;
    if (tid < 256 && v >= need && v - g < need) { rx.bin = tid; rx.need_left = need - (v - g); }
    __syncthreads();
    need = rx.need_left;
    return rx.bin;
}

__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long ld, int vocab, float inv_temperature, int top_k,
                      float top_p, const int* __restrict__ slots, unsigned long long* __restrict__ rng_state,
                      int* __restrict__ out, float* __restrict__ drawn_u) {
    extern __shared__ unsigned xs[];                     // this block's slice: keys of the scaled logits, later weights
    __shared__ ScShared sh;
    __shared__ RxShared rx;
    const int tid = threadIdx.x, row_id = blockIdx.y;
    const unsigned rank = sc_rank();
    const float* row = logits + (size_t)row_id * ld;
    const int per_cta = (vocab + SC_CTAS - 1) / SC_CTAS;
    const int lo_i = min((int)rank * per_cta, vocab), hi_i = min(lo_i + per_cta, vocab), n = hi_i - lo_i;
    const int n_it = (n + ST_TILE - 1) / ST_TILE;
    int turn = 0;
    if (tid == 0) { sh.found = 0x7fffffff; rx.bin = 0; rx.need_left = 0; }   // a row without any weight finds no bin

    const int seq = slots ? slots[row_id] : row_id;
    unsigned long long state = rng_state[seq];
    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
    const float u = (float)(state >> 40) / 16777216.0f;

    float mx = -INFINITY;
    for (int i = tid; i < n; i += SC_THREADS) {
        const float x = row[lo_i + i] * inv_temperature;
        xs[i] = float_order_key(x);
        mx = fmaxf(mx, x);
    }
    mx = sc_max(mx, sh, turn);
    if (rank == 0 && tid == 0) { rng_state[seq] = state; if (drawn_u) drawn_u[row_id] = u; }

    int buf = 0;
    unsigned cut = 0u;                                   // keys below it are not kept; 0 keeps everything
    if (top_k > 0 && top_k < vocab) {
        unsigned prefix = 0u, mask = 0u;
        unsigned long long need = (unsigned long long)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += SC_THREADS) rx.hist[buf][0][b] = 0u;
            __syncthreads();
            for (int i0 = 0; i0 < n; i0 += SC_THREADS) {
                const int i = i0 + tid;
                const unsigned key = i < n ? xs[i] : 0u;
                rx_add<true>(rx.hist[buf], i < n && (key & mask) == prefix, (key >> shift) & 255u, 1ull);
            }
            const int b = rx_byte<true>(rx, buf, need, -1.f);
            prefix |= (unsigned)b << shift;
            mask |= 255u << shift;
            buf ^= 1;
        }
        cut = prefix;                                    // the key of the k-th largest: everything tied with it is kept
    }
    // weights in place of the keys: exp(x - max) of what the top-k cut keeps, else 0.  As bit patterns
    // non-negative floats are ordered like their values, so the top-p cut is searched over the bits.
    for (int i = tid; i < n; i += SC_THREADS) {
        const unsigned key = xs[i];
        const float x = __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
        const float w = (key >= cut) ? expf(x - mx) : 0.f;
        xs[i] = (w > 0.f && w <= 1.f) ? __float_as_uint(w) : 0u;            // not a number (an infinite maximum): no weight
    }
    unsigned w_cut = 1u;                                 // weights (as bits) below it are not kept: 1 drops only zeros
    if (top_p < 1.0f) {
        unsigned prefix = 0u, mask = 0u;
        unsigned long long need = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 3 * 256; b += SC_THREADS) rx.hist[buf][0][b] = 0u;
            __syncthreads();
            for (int i0 = 0; i0 < n; i0 += SC_THREADS) {
                const int i = i0 + tid;
                const unsigned bits = i < n ? xs[i] : 0u;
                rx_add<false>(rx.hist[buf], bits != 0u && (bits & mask) == prefix, (bits >> shift) & 255u,
                       (unsigned long long)(__uint_as_float(bits) * 1099511627776.f));
            }
            const int b = rx_byte<false>(rx, buf, need, shift == 24 ? fmaxf(top_p, 0.f) : -1.f);
            prefix |= (unsigned)b << shift;
            mask |= 255u << shift;
            buf ^= 1;
        }
        w_cut = prefix > 1u ? prefix : 1u;
    }
    __syncthreads();
    auto weights = [&](int it, float (&w)[ST_EL]) {
        const int i0 = (it * SC_THREADS + tid) * ST_EL;
#pragma unroll
        for (int e = 0; e < ST_EL; ++e) {
            const unsigned bits = (i0 + e < n) ? xs[i0 + e] : 0u;
            w[e] = bits >= w_cut ? __uint_as_float(bits) : 0.f;
        }
    };
    auto largest = [&](float& bv, int& bi) {
        bv = -INFINITY; bi = 0x7fffffff;
        for (int i = tid; i < n; i += SC_THREADS) {
            const float x = row[lo_i + i] * inv_temperature;
            if (x > bv) { bv = x; bi = lo_i + i; }
        }
    };
    sc_draw(sh, turn, rank, n, n_it, lo_i, u, out + row_id, weights, largest);
}

SSB_API int ssb_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature,
                       int top_k, float top_p, const int* slots, unsigned long long* rng_state, int* out,
                       float* drawn_u, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || vocab >= 0x40000000 || !(temperature > 0.f)) return SSB_ERR_BAD_SIZE;
    const int per_cta = (vocab + SC_CTAS - 1) / SC_CTAS;
    const size_t slice = (size_t)per_cta * sizeof(float);
    // a cluster of 8 blocks per row while a slice has at most 32 stretches (vocabularies up to 524,288)
    if (n_rows <= 65535 && per_cta <= ST_MAX_IT * ST_TILE) {
        // temperature alone: nothing to search, the row stays where it is
        if ((top_k <= 0 || top_k >= vocab) && !(top_p < 1.0f)) {
            sample_stream_kernel<<<dim3(SC_CTAS, n_rows), SC_THREADS, 0, stream>>>(
                logits, ld, vocab, 1.0f / temperature, slots, rng_state, out, drawn_u);
            return ssb_launch_status();
        }
        if (slice <= 200 * 1024) {                       // the slices fit shared memory (vocabularies up to 400k)
            static size_t configured = 0;
            if (slice > 40 * 1024 && slice > configured) {
                cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slice);
                if (e != cudaSuccess) return (int)e;
                configured = slice;
            }
            sample_cluster_kernel<<<dim3(SC_CTAS, n_rows), SC_THREADS, slice, stream>>>(
                logits, ld, vocab, 1.0f / temperature, top_k, top_p, slots, rng_state, out, drawn_u);
            return ssb_launch_status();
        }
    }
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, 1.0f / temperature, top_k,
                                                         top_p, slots, rng_state, out, drawn_u);
    return ssb_launch_status();
}
