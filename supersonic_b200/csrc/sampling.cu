// Sampling kernels: argmax, and temperature / top-k / top-p sampling, one block per row of
// float32 logits.
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

SSB_API int ssb_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature,
                       int top_k, float top_p, const int* slots, unsigned long long* rng_state, int* out,
                       float* drawn_u, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || vocab >= 0x40000000 || !(temperature > 0.f)) return SSB_ERR_BAD_SIZE;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, 1.0f / temperature, top_k,
                                                         top_p, slots, rng_state, out, drawn_u);
    return ssb_launch_status();
}
