// Element-wise kernels with 16-byte accesses for bfloat16 activations:
// RMSNorm of the float32 residual stream (16-byte loads, the row kept in registers between the sum
// of squares and the scaling) and rotary encoding + paged cache append (bfloat16 pairs, 16-byte
// copies of the values, one page lookup per token and kv head).  Same arithmetic and the same
// roundings as the plain kernels in plain_ops.cu, which remain their reference and the fallback
// for sizes these refuse.  Formulas: kernels/full_attention_cuda.cuh:2826-2873 (rmsnorm),
// kernels/prefill_helpers_cuda.cuh:80-111 (rope), kernels/certified_kv_bridge_cuda.cu:32-51 (append).
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

// ---- rmsnorm: one block per row, hidden <= 4 * 256 * RV floats ------------------------------
constexpr int RN_THREADS = 256;

template <int RV, typename TW>            // RV float4 per thread
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows, const TW* __restrict__ w, float eps,
                   bf16* __restrict__ out, int hidden) {
    __shared__ float red[RN_THREADS / 32];
    ssb_pdl_launch_dependents();
    const int r = blockIdx.x;
    const int n4 = hidden / 4;
    // The norm's weights are written by no kernel of a step: they are in registers before the dependency
    // wait, so that after it only the row itself has to come (one trip to L2 on the critical path, not two).
    float wv[RV][4];
#pragma unroll
    for (int i = 0; i < RV; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
#pragma unroll
        for (int k = 0; k < 4; ++k) wv[i][k] = c < n4 ? ssb_to_float(w[4 * c + k]) : 0.f;
    }
    ssb_pdl_wait();
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden);
    float4 v[RV];
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < RV; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
        v[i] = c < n4 ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        part = fmaf(v[i].x, v[i].x, part); part = fmaf(v[i].y, v[i].y, part);
        part = fmaf(v[i].z, v[i].z, part); part = fmaf(v[i].w, v[i].w, part);
    }
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < RN_THREADS / 32; ++i) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    uint2* dst = reinterpret_cast<uint2*>(out + (size_t)r * hidden);
#pragma unroll
    for (int i = 0; i < RV; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
        if (c >= n4) continue;
        __nv_bfloat162 a = __floats2bfloat162_rn(v[i].x * inv * wv[i][0], v[i].y * inv * wv[i][1]);
        __nv_bfloat162 b = __floats2bfloat162_rn(v[i].z * inv * wv[i][2], v[i].w * inv * wv[i][3]);
        uint2 p;
        p.x = *reinterpret_cast<uint32_t*>(&a);
        p.y = *reinterpret_cast<uint32_t*>(&b);
        dst[c] = p;
    }
}

SSB_API int ssb_rmsnorm_vec(const float* x, const int* rows, const void* w, int w_dtype, float eps, void* out,
                            int n_rows, int hidden, int pdl, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden % 4 || hidden > 4 * RN_THREADS * 8 || (((uintptr_t)x | (uintptr_t)out) & 15)) return SSB_ERR_BAD_SIZE;
    const int rv = (hidden / 4 + RN_THREADS - 1) / RN_THREADS;
    int rc = 0;
#define SSB_RV(RV_) \
    rc = w_dtype == SSB_F32 \
        ? ssb_launch(rmsnorm_vec_kernel<RV_, float>, dim3(n_rows), dim3(RN_THREADS), 0, stream, pdl != 0, x, rows, (const float*)w, eps, (bf16*)out, hidden) \
        : ssb_launch(rmsnorm_vec_kernel<RV_, bf16>, dim3(n_rows), dim3(RN_THREADS), 0, stream, pdl != 0, x, rows, (const bf16*)w, eps, (bf16*)out, hidden)
    if (rv <= 1) SSB_RV(1); else if (rv <= 2) SSB_RV(2); else if (rv <= 4) SSB_RV(4); else SSB_RV(8);
#undef SSB_RV
    return rc ? rc : ssb_launch_status();
}

// ---- round a float32 sum to bfloat16 and clear it ---------------------------------------------
// A projection whose K range is split over blocks that add with float atomics leaves float32 sums
// in a scratch that was zero before; this writes them out as bfloat16 and zeroes the scratch for
// the next projection that uses it.  8 elements a thread.
__global__ void __launch_bounds__(256)
round_and_clear_kernel(float* __restrict__ sums, bf16* __restrict__ out, int ldo, int n_rows, int n_cols) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int per_row = n_cols / 8;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_rows * per_row) return;
    const int r = (int)(i / per_row), c = (int)(i % per_row) * 8;
    float4* src = reinterpret_cast<float4*>(sums + (size_t)r * n_cols + c);
    const float4 a = src[0], b = src[1];
    src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 v;
    v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
    v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = v;
}

// sums: float32 [n_rows, n_cols] contiguous (left zero); out: bfloat16 [n_rows, n_cols], row stride ldo.
SSB_API int ssb_round_and_clear(float* sums, void* out, int ldo, int n_rows, int n_cols, int pdl, cudaStream_t stream) {
    if (n_rows <= 0 || n_cols <= 0) return 0;
    if (n_cols % 8 || ldo % 8 || (((uintptr_t)sums | (uintptr_t)out) & 15)) return SSB_ERR_BAD_SIZE;
    const long long n = (long long)n_rows * (n_cols / 8);
    const int rc = ssb_launch(round_and_clear_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, pdl != 0,
                              sums, (bf16*)out, ldo, n_rows, n_cols);
    return rc ? rc : ssb_launch_status();
}

// ---- rope + append: one block per token ------------------------------------------------------
template <int DUMMY>
__global__ void __launch_bounds__(256)
rope_append_vec_kernel(bf16* __restrict__ qkv, int ld, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ page_table,
                       int max_pages, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int n_q, int n_kv,
                       int head_dim, int page_shift) {
    const int t = blockIdx.x;
    const int s = slot[t];
    if (s < 0) return;
    const int p = pos[t];
    const int half = head_dim / 2, hp = half / 2;               // pairs of adjacent elements per half
    bf16* row = qkv + (size_t)t * ld;
    const float2* c_row = reinterpret_cast<const float2*>(cos_t + (size_t)p * half);
    const float2* s_row = reinterpret_cast<const float2*>(sin_t + (size_t)p * half);
    const int page = page_table[(size_t)s * max_pages + (p >> page_shift)];
    const size_t tok_base = ((size_t)page * n_kv) << page_shift;
    const int in_page = p & ((1 << page_shift) - 1);
    // rotate q heads in place; rotate k heads in place and into the cache
    for (int e = threadIdx.x; e < (n_q + n_kv) * hp; e += blockDim.x) {
        const int h = e / hp, i2 = e % hp;
        __nv_bfloat162* x = reinterpret_cast<__nv_bfloat162*>(row + (size_t)h * head_dim);
        const float2 a = __bfloat1622float2(x[i2]), b = __bfloat1622float2(x[i2 + hp]);
        const float2 c = c_row[i2], sn = s_row[i2];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y);
        x[i2] = lo;
        x[i2 + hp] = hi;
        if (h >= n_q) {
            __nv_bfloat162* kc = reinterpret_cast<__nv_bfloat162*>(
                k_cache + ((tok_base + ((size_t)(h - n_q) << page_shift)) + in_page) * head_dim);
            kc[i2] = lo;
            kc[i2 + hp] = hi;
        }
    }
    // values: 16-byte copies
    const int v8 = head_dim / 8;
    const uint4* v_src = reinterpret_cast<const uint4*>(row + (size_t)(n_q + n_kv) * head_dim);
    for (int e = threadIdx.x; e < n_kv * v8; e += blockDim.x) {
        const int h = e / v8, j = e % v8;
        uint4* vc = reinterpret_cast<uint4*>(v_cache + ((tok_base + ((size_t)h << page_shift)) + in_page) * head_dim);
        vc[j] = v_src[e];
    }
}

// Full-width rotation (rotary_dim == head_dim), head_dim a multiple of 8, rows 16-byte aligned.
SSB_API int ssb_rope_append_vec(void* qkv, int ld, const float* cos_t, const float* sin_t, int table_positions,
                                const int* pos, const int* slot, const int* page_table, int max_pages,
                                void* k_cache, void* v_cache, int n_tokens, int n_q, int n_kv, int head_dim,
                                int page_shift, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim % 8 || ld % 8 || !cos_t || !sin_t || table_positions <= 0) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15)
        return SSB_ERR_BAD_SIZE;
    rope_append_vec_kernel<0><<<n_tokens, 256, 0, stream>>>((bf16*)qkv, ld, cos_t, sin_t, pos, slot, page_table, max_pages,
                                                            (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv, head_dim, page_shift);
    return ssb_launch_status();
}
