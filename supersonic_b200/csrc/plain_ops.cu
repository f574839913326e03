// Plain kernels: one simple kernel per operation, all arithmetic in IEEE float32
// (no fast-math in this file), a fixed order of summation that depends only on
// the element's own position, never on what else is in the batch.
//
// They are the whole float32 path of the engine and the reference beside each
// fast kernel.  Templated on the storage type so that the same code also runs
// with bfloat16 storage.  Formulas as the reference computes them:
//   embedding   kernels/full_attention_cuda.cuh:2012-2034
//   rmsnorm     kernels/full_attention_cuda.cuh:2826-2873
//   matmul      kernels/full_attention_4b_cuda.cuh:2671-2743 (out[m,n] = sum_k a[m,k] w[n,k])
//   rope        kernels/prefill_helpers_cuda.cuh:80-111 (half-split pairs)
//   kv append   kernels/certified_kv_bridge_cuda.cu:32-51
//   attention   kernels/full_attention_cuda.cuh:360-474, 476-576
//   swiglu      kernels/full_attention_cuda.cuh:1995-2010
//   argmax      kernels/prefill_helpers_bridge_cuda.cu:247-287 (lowest index wins ties)
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :], written into the float32 residual stream
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {          // the host refuses such ids; never read out of range
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ssb_to_float(src[c]);
}

SSB_API int ssb_embed(const int* ids, const void* table, int table_dtype, float* out, int n_tokens,
                      int hidden, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (table_dtype == SSB_F32)
        embed_kernel<float><<<n_tokens, 256, 0, stream>>>(ids, (const float*)table, out, hidden, vocab);
    else if (table_dtype == SSB_BF16)
        embed_kernel<bf16><<<n_tokens, 256, 0, stream>>>(ids, (const bf16*)table, out, hidden, vocab);
    else
        return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// rmsnorm over rows of the float32 residual stream; optional row gather
// ---------------------------------------------------------------------------------------
template <typename TO, typename TW>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const TW* __restrict__ w, float eps, TO* __restrict__ out, int hidden) {
    __shared__ float red[256];
    const int r = blockIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
    float part = 0.f;
    for (int c = threadIdx.x; c < hidden; c += 256) {
        const float v = src[c];
        part = fmaf(v, v, part);
    }
    red[threadIdx.x] = part;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    const float inv = 1.0f / sqrtf(red[0] / (float)hidden + eps);
    TO* dst = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += 256)
        dst[c] = ssb_from_float<TO>(src[c] * inv * ssb_to_float(w[c]));
}

SSB_API int ssb_rmsnorm(const float* x, const int* rows, const void* w, int w_dtype, float eps,
                        void* out, int out_dtype, int n_rows, int hidden, int pdl, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    int rc = 0;
#define SSB_RMS(TO, TW) \
    rc = ssb_launch(rmsnorm_kernel<TO, TW>, dim3(n_rows), dim3(256), 0, stream, pdl != 0, x, rows, (const TW*)w, eps, \
                    (TO*)out, hidden)
    if (out_dtype == SSB_F32 && w_dtype == SSB_F32) SSB_RMS(float, float);
    else if (out_dtype == SSB_F32 && w_dtype == SSB_BF16) SSB_RMS(float, bf16);
    else if (out_dtype == SSB_BF16 && w_dtype == SSB_F32) SSB_RMS(bf16, float);
    else if (out_dtype == SSB_BF16 && w_dtype == SSB_BF16) SSB_RMS(bf16, bf16);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_RMS
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// C[m, n] (+)= sum_k A[m, k] * W[n, k]; 64x64 tile, 16-wide k steps.  float32 throughout, in a
// fixed order: the 16 products of a k step are summed with FMAs, and the steps' sums are added
// with compensation (Kahan), so that the rounding error of a long row (14,336 terms in a
// feed-forward) stays at a few units in the last place instead of growing with its length.
// ---------------------------------------------------------------------------------------
template <typename TA, typename TC, bool ACCUMULATE>
__global__ void __launch_bounds__(256)
gemm_nt_plain_kernel(const TA* __restrict__ A, int lda, const TA* __restrict__ W, int ldw,
                     TC* __restrict__ C, int ldc, int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4], lost[4][4];          // running sums and what their last additions rounded away
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; lost[i][j] = 0.f; }

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;         // 0..1023
            const int r = idx / BK, c = idx % BK;
            const int k = k0 + c;
            const int m = m0 + r, n = n0 + r;
            As[c][r] = (m < M && k < K) ? ssb_to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[c][r] = (n < N && k < K) ? ssb_to_float(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float y = __fsub_rn(part[i][j], lost[i][j]);       // explicit roundings: nothing is re-associated
                const float t = __fadd_rn(acc[i][j], y);
                lost[i][j] = __fsub_rn(__fsub_rn(t, acc[i][j]), y);
                acc[i][j] = t;
            }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TC* dst = C + (size_t)m * ldc + n;
            if (ACCUMULATE) *dst = ssb_from_float<TC>(ssb_to_float(*dst) + acc[i][j]);
            else *dst = ssb_from_float<TC>(acc[i][j]);
        }
    }
}

SSB_API int ssb_gemm_nt_plain(const void* A, int lda, const void* W, int ldw, int in_dtype, void* C,
                              int ldc, int out_dtype, int M, int N, int K, int accumulate,
                              cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return SSB_ERR_BAD_SIZE;
    if (accumulate && out_dtype != SSB_F32) return SSB_ERR_BAD_DTYPE;
    dim3 grid((N + 63) / 64, (M + 63) / 64);
#define SSB_GEMM(TA, TC, ACC) \
    gemm_nt_plain_kernel<TA, TC, ACC><<<grid, 256, 0, stream>>>( \
        (const TA*)A, lda, (const TA*)W, ldw, (TC*)C, ldc, M, N, K)
    if (in_dtype == SSB_F32 && out_dtype == SSB_F32) {
        if (accumulate) SSB_GEMM(float, float, true); else SSB_GEMM(float, float, false);
    } else if (in_dtype == SSB_BF16 && out_dtype == SSB_F32) {
        if (accumulate) SSB_GEMM(bf16, float, true); else SSB_GEMM(bf16, float, false);
    } else if (in_dtype == SSB_BF16 && out_dtype == SSB_BF16) {
        SSB_GEMM(bf16, bf16, false);
    } else {
        return SSB_ERR_BAD_DTYPE;
    }
#undef SSB_GEMM
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// rotary position encoding on q (in place) and k, then k and v into the paged cache
// qkv row layout: [q heads | k heads | v heads], each head_dim wide
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, int table_positions,
                                   const int* __restrict__ pos, const int* __restrict__ slot,
                                   const int* __restrict__ page_table, int max_pages,
                                   T* __restrict__ k_cache, T* __restrict__ v_cache, int n_q, int n_kv,
                                   int head_dim, int rotary_dim, int page_shift, int write_cache) {
    const int t = blockIdx.x;
    const int s = slot[t];
    if (s < 0) return;                                   // padding row
    const int p = pos[t];
    const int half = rotary_dim / 2;
    T* row = qkv + (size_t)t * ld;
    const bool have_table = (cos_t != nullptr) && p < table_positions;
    const float* c_row = have_table ? cos_t + (size_t)p * half : nullptr;
    const float* s_row = have_table ? sin_t + (size_t)p * half : nullptr;
    const int n_rot_heads = write_cache ? n_q + n_kv : n_q;
    // rotate q heads (and k heads), pairs (i, i + half) of the first rotary_dim elements
    for (int e = threadIdx.x; e < n_rot_heads * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        T* x = row + (size_t)h * head_dim;
        const float c = have_table ? c_row[i] : 1.f, sn = have_table ? s_row[i] : 0.f;
        const float x1 = ssb_to_float(x[i]), x2 = ssb_to_float(x[i + half]);
        x[i] = ssb_from_float<T>(x1 * c - x2 * sn);
        x[i + half] = ssb_from_float<T>(x1 * sn + x2 * c);
    }
    if (!write_cache) return;
    __syncthreads();
    const T* k_src = row + (size_t)n_q * head_dim;
    const T* v_src = k_src + (size_t)n_kv * head_dim;
    for (int e = threadIdx.x; e < n_kv * head_dim; e += blockDim.x) {
        const int h = e / head_dim, d = e % head_dim;
        const size_t off = ssb_cache_row(page_table, max_pages, s, p, page_shift, n_kv, h, head_dim) + d;
        k_cache[off] = k_src[e];
        v_cache[off] = v_src[e];
    }
}

SSB_API int ssb_rope_append(void* qkv, int ld, int dtype, const float* cos_t, const float* sin_t,
                            int table_positions, const int* pos, const int* slot,
                            const int* page_table, int max_pages, void* k_cache, void* v_cache,
                            int n_tokens, int n_q, int n_kv, int head_dim, int rotary_dim,
                            int page_shift, int write_cache, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim % 2 || rotary_dim > head_dim || rotary_dim < 0) return SSB_ERR_BAD_SIZE;
    if (dtype == SSB_F32)
        rope_append_kernel<float><<<n_tokens, 256, 0, stream>>>(
            (float*)qkv, ld, cos_t, sin_t, table_positions, pos, slot, page_table, max_pages,
            (float*)k_cache, (float*)v_cache, n_q, n_kv, head_dim, rotary_dim, page_shift, write_cache);
    else if (dtype == SSB_BF16)
        rope_append_kernel<bf16><<<n_tokens, 256, 0, stream>>>(
            (bf16*)qkv, ld, cos_t, sin_t, table_positions, pos, slot, page_table, max_pages,
            (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv, head_dim, rotary_dim, page_shift, write_cache);
    else
        return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// attention of each token over its sequence's cached keys: one block per (token, head).
// Keys are visited in chunks of 128 starting at the first visible key, so the order of
// every sum depends on the token's own position and window only.
// ---------------------------------------------------------------------------------------
constexpr int ATT_THREADS = 128;
constexpr int ATT_MAX_HEAD_DIM = 512;

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
    red[threadIdx.x] = v;
    __syncthreads();
    for (int s = ATT_THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + s]);
        __syncthreads();
    }
    const float r = red[0];
    __syncthreads();
    return r;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
    red[threadIdx.x] = v;
    __syncthreads();
    for (int s = ATT_THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    const float r = red[0];
    __syncthreads();
    return r;
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_plain_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, const int* __restrict__ pos,
                       const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages,
                       T* __restrict__ out, int ldo, int n_q, int n_kv, int head_dim, int page_shift,
                       int window, float scale) {
    __shared__ float q_s[ATT_MAX_HEAD_DIM];
    __shared__ float p_s[ATT_THREADS];
    __shared__ float red[ATT_THREADS];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    T* o = out + (size_t)t * ldo + (size_t)h * head_dim;
    const int s = slot[t];
    if (s < 0) {
        for (int d = tid; d < head_dim; d += ATT_THREADS) o[d] = ssb_from_float<T>(0.f);
        return;
    }
    const int p = pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int kvh = h / (n_q / n_kv);
    const T* qp = q + (size_t)t * ldq + (size_t)h * head_dim;
    for (int d = tid; d < head_dim; d += ATT_THREADS) q_s[d] = ssb_to_float(qp[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_HEAD_DIM / ATT_THREADS];
#pragma unroll
    for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) acc[i] = 0.f;

    for (int base = lo; base <= p; base += ATT_THREADS) {
        const int j = base + tid;
        float sc = -INFINITY;
        if (j <= p) {
            const T* kr = k_cache + ssb_cache_row(page_table, max_pages, s, j, page_shift, n_kv, kvh, head_dim);
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[d], ssb_to_float(kr[d]), dot);
            sc = dot * scale;
        }
        const float cm = block_reduce_max(sc, red);
        const float m_new = fmaxf(m, cm);
        const float pj = (j <= p) ? expf(sc - m_new) : 0.f;
        p_s[tid] = pj;
        const float cs = block_reduce_sum(pj, red);      // also orders p_s writes before reads
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + cs;
        const int n_in = min(ATT_THREADS, p - base + 1);
#pragma unroll
        for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) {
            const int d = tid + i * ATT_THREADS;
            if (d < head_dim) {
                float a = acc[i] * alpha;
                for (int jj = 0; jj < n_in; ++jj) {
                    const T* vr = v_cache + ssb_cache_row(page_table, max_pages, s, base + jj, page_shift,
                                                          n_kv, kvh, head_dim);
                    a = fmaf(p_s[jj], ssb_to_float(vr[d]), a);
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < ATT_MAX_HEAD_DIM / ATT_THREADS; ++i) {
        const int d = tid + i * ATT_THREADS;
        if (d < head_dim) o[d] = ssb_from_float<T>(l > 0.f ? acc[i] / l : 0.f);
    }
}

SSB_API int ssb_attention_plain(const void* q, int ldq, int dtype, const void* k_cache,
                                const void* v_cache, const int* pos, const int* slot,
                                const int* page_table, int max_pages, void* out, int ldo, int n_tokens,
                                int n_q, int n_kv, int head_dim, int page_shift, int window, float scale,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim > ATT_MAX_HEAD_DIM || head_dim <= 0 || n_kv <= 0 || n_q % n_kv) return SSB_ERR_BAD_SIZE;
    dim3 grid(n_tokens, n_q);
    if (dtype == SSB_F32)
        attention_plain_kernel<float><<<grid, ATT_THREADS, 0, stream>>>(
            (const float*)q, ldq, (const float*)k_cache, (const float*)v_cache, pos, slot, page_table,
            max_pages, (float*)out, ldo, n_q, n_kv, head_dim, page_shift, window, scale);
    else if (dtype == SSB_BF16)
        attention_plain_kernel<bf16><<<grid, ATT_THREADS, 0, stream>>>(
            (const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, pos, slot, page_table,
            max_pages, (bf16*)out, ldo, n_q, n_kv, head_dim, page_shift, window, scale);
    else
        return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// swiglu: z[t, c] = silu(gate[t, c]) * up[t, c].  Gate and up are the two halves of a row, or
// (interleaved) come as [8 gate | 8 up] per 16 columns
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, int ld, T* __restrict__ z, int ldz, int inter,
                              size_t total, int interleaved) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int c = (int)(idx % inter);
    const int cg = interleaved ? (c / 8) * 16 + (c % 8) : c;
    const int cu = interleaved ? cg + 8 : inter + c;
    const float g = ssb_to_float(gu[t * ld + cg]);
    const float u = ssb_to_float(gu[t * ld + cu]);
    z[t * ldz + c] = ssb_from_float<T>(g / (1.0f + expf(-g)) * u);
}

SSB_API int ssb_swiglu(const void* gate_up, int ld, void* z, int ldz, int dtype, int n_tokens, int inter,
                       int interleaved, cudaStream_t stream) {
    if (interleaved && inter % 8) return SSB_ERR_BAD_SIZE;
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == SSB_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, ld, (float*)z, ldz, inter, total, interleaved);
    else if (dtype == SSB_BF16)
        swiglu_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)gate_up, ld, (bf16*)z, ldz, inter, total, interleaved);
    else
        return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// out (float32) += x
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void add_into_kernel(float* __restrict__ out, const T* __restrict__ x, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += ssb_to_float(x[i]);
}

SSB_API int ssb_add_into(float* out, const void* x, int x_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (x_dtype == SSB_F32) add_into_kernel<float><<<blocks, 256, 0, stream>>>(out, (const float*)x, (size_t)n);
    else if (x_dtype == SSB_BF16) add_into_kernel<bf16><<<blocks, 256, 0, stream>>>(out, (const bf16*)x, (size_t)n);
    else return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}
