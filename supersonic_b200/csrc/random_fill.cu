// Seeded random weights, element by element: value i of a tensor depends on (seed, tensor name,
// i) alone, so a tensor is the same whether it is made whole or in pieces, on the device or on
// the host, today or by another build.  The reference has no random weights (it always loads a
// checkpoint: crates/runner/src/llama31_engine.rs:170-287); this is the library's own.
//
// The draw uses integer arithmetic only until its last two steps, so that the host version
// (weights/random_fill.py) gives the same bits:
//   key     = mix(seed ^ fnv1a64(name))                                  (host, once per tensor)
//   z_j     = mix(key + (3 i + j + 1) * 0x9E3779B97F4A7C15),  j = 0, 1, 2
//   S       = sum of the twelve 16-bit fields of z_0, z_1, z_2
//   n       = (2 S - 12 * 65535) / 131072     a sum of twelve uniforms, mean 0, variance 1 - 2^-32
//   value   = mean + std * n                   two correctly rounded double operations
// then rounded to float32 and, for bfloat16 tensors, once more to nearest even.
#include "common.cuh"

__host__ __device__ __forceinline__ unsigned long long rf_mix(unsigned long long z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ int rf_fields(unsigned long long z) {
    return (int)(z & 0xFFFF) + (int)((z >> 16) & 0xFFFF) + (int)((z >> 32) & 0xFFFF) + (int)(z >> 48);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long first, long long count,
                                   unsigned long long key, double mean, double std) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += stride) {
        const unsigned long long i = (unsigned long long)(first + e);
        int s = 0;
#pragma unroll
        for (int j = 0; j < 3; ++j) s += rf_fields(rf_mix(key + (3ull * i + j + 1ull) * 0x9E3779B97F4A7C15ull));
        const double n = (double)(2 * s - 12 * 65535) * (1.0 / 131072.0);
        const double v = __dadd_rn(mean, __dmul_rn(std, n));       // no fused multiply-add: the host has none
        out[e] = ssb_from_float<T>(__double2float_rn(v));
    }
}

// out[0 .. count) = elements first .. first + count - 1 of the tensor whose key is `key`.
SSB_API int ssb_random_fill(void* out, int dtype, long long first, long long count, unsigned long long key,
                            double mean, double std, cudaStream_t stream) {
    if (count <= 0) return 0;
    const int threads = 256;
    const long long want = (count + threads - 1) / threads;
    const int blocks = (int)(want < 65536 ? want : 65536);
    if (dtype == SSB_F32)
        random_fill_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, first, count, key, mean, std);
    else if (dtype == SSB_BF16)
        random_fill_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, first, count, key,
                                                                         mean, std);
    else
        return SSB_ERR_BAD_DTYPE;
    return ssb_launch_status();
}
