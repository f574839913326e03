// Projections of up to 128 rows (decode steps, short prompts) on tcgen05: out[b, n] = sum_k x[b, k] W[n, k], with the
// weights as the M side of the MMA.  A block owns 128 rows of W and a range of K; 128 x 64 tiles
// of W (16 KB of useful bytes a stage) and the matching columns of x arrive through TMA into an
// four-stage ring; one thread issues tcgen05.mma (M 128, N = rows rounded up to 16/32/64/128); the
// accumulator [W row, batch row] sits in tensor memory.  When K is split over several blocks
// (few row tiles: the small projections), a store or SwiGLU output goes through scratch: each
// block writes its partial tile and the block that arrives last for the tile adds them in split
// order (same result every time); an add into the float32 residual is done the same way when the
// caller gives scratch, else by every block with float atomics (cheaper; the order of the shares,
// and so the last bits, then vary between runs).
// Epilogues: store, add into the float32 residual, SwiGLU over [8 gate | 8 up] rows.
//
// The general GEMM (gemm_tc.cu) has the tokens on the M side: with 64 tokens it re-reads the
// activations for every 64 columns of W and fills few SMs; here the weights stream once and the
// small operand is the one that repeats.  Replaces the reference's cuBLAS GEMV per projection
// (kernels/full_attention_bridge_4b_cuda.cu:4768-4813), which it runs one sequence at a time.
//
// Every mbarrier wait is bounded (tc_helpers.cuh): on a timeout the block records a code in the
// caller's error word, lets its copies land, frees its tensor memory and returns.
#include "common.cuh"
#include "tc_helpers.cuh"

typedef __nv_bfloat16 bf16;

constexpr int GV_BM = 128;                // rows of W per block
// stages of the ring: as many as let two blocks share an SM (no second wave for 149..296 blocks):
// 18 KB a stage at up to 16 batch rows, 20 KB at 32, 24 KB at 64, 32 KB at 128
__host__ __device__ constexpr int gv_stages(int bnb) { return bnb <= 16 ? 6 : (bnb <= 32 ? 5 : (bnb <= 64 ? 4 : 3)); }
constexpr int GV_MAX_ROWS = 128;
constexpr unsigned GV_ROT = 5;            // k-blocks by which neighbouring row tiles start apart (see the producer)
constexpr int GV_THREADS = 192;           // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

template <int BNB>                        // batch rows per tile: 16, 32, 64 or 128
__global__ void __launch_bounds__(GV_THREADS, 2)
gemv_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               void* __restrict__ out, int ldo, int out_is_f32, int n_rows, int N, int K, int mode, int splits,
               float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ error_word) {
    constexpr int GV_STAGES = gv_stages(BNB);
    constexpr uint32_t W_BYTES = GV_BM * TC_BK * 2, X_BYTES = BNB * TC_BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = BNB < 32 ? 32 : BNB;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + GV_STAGES * STAGE_BYTES);    // full[S], empty[S], acc_full
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * GV_STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);       // [0]: a role gave up; [1]: stays zero
    int* is_last = (int*)(tmem_slot + 3);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * GV_BM;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int kb_per = (k_blocks + splits - 1) / splits;
    const int kb0 = split * kb_per, kb1 = min(k_blocks, kb0 + kb_per);
    const int my_blocks = max(0, kb1 - kb0);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + GV_STAGES), acc_full = smem_u32(bars + 2 * GV_STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < GV_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(acc_full, 1);
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        *is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ssb_pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // The weights are written by no kernel of a step: the ring's first tiles of W are asked
            // for before the dependency wait, so that they stream in while the predecessor still runs
            // (the block is resident by then, through programmatic dependent launch).  Only x has to
            // wait; a stage's barrier completes when both of its tiles have landed.
            // Blocks walk their k-blocks from different starting points (and wrap): the tiles of x are the
            // same for every block, and blocks that run in step would all ask L2 for the same few lines at once
            // (8B gate/up: 38.0 to 35.9 us at 8 rows, 40.7 to 39.3 at 64; a step gains about half a per cent).
            const int rot = my_blocks > 0 ? (int)(((unsigned)tile * GV_ROT) % (unsigned)my_blocks) : 0;
            auto kb_of = [&](int i) { const int j = i + rot; return kb0 + (j >= my_blocks ? j - my_blocks : j); };
            // the weights pass through L2 once a step: they are the first to leave it again
            const uint64_t w_policy = ssb_policy_evict_first();
            const int pre = min(my_blocks, GV_STAGES);
            for (int i = 0; i < pre; ++i) {                  // the ring is empty: no wait for a free stage
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                tma_load_2d_hint(smem_u32(smem + i * STAGE_BYTES), &map_w, full0 + 8 * i, kb_of(i) * TC_BK, n0, w_policy);
            }
            ssb_pdl_wait();                                  // x is the predecessor's output
            for (int i = 0; i < pre; ++i)
                tma_load_2d(smem_u32(smem + i * STAGE_BYTES) + W_BYTES, &map_x, full0 + 8 * i, kb_of(i) * TC_BK, 0);
            int issued = pre;
            for (int i = pre; i < my_blocks; ++i) {
                const int s = i % GV_STAGES;
                const uint32_t phase = (i / GV_STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_PRODUCER); break;
                }
                const uint32_t w_dst = smem_u32(smem + s * STAGE_BYTES), x_dst = w_dst + W_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d_hint(w_dst, &map_w, full0 + 8 * s, kb_of(i) * TC_BK, n0, w_policy);
                tma_load_2d(x_dst, &map_x, full0 + 8 * s, kb_of(i) * TC_BK, 0);
                issued = i + 1;
            }
            if (*abort_flag)
                for (int i = max(0, issued - GV_STAGES); i < issued; ++i)
                    mbar_wait(full0 + 8 * (i % GV_STAGES), (i / GV_STAGES) & 1, abort_flag + 1);
        }
    } else if (warp == 1) {
        if (lane == 0 && my_blocks > 0) {
            // D float32, A and B bfloat16, both K-major, N = BNB, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNB >> 3) << 17) | ((uint32_t)(GV_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < my_blocks && ok; ++i) {
                const int s = i % GV_STAGES;
                const uint32_t phase = (i / GV_STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, phase, abort_flag)) {
                    *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_MMA); ok = false; break;
                }
                tc_fence_after();
                const uint32_t w_addr = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t dw = smem_desc(w_addr), dx = smem_desc(w_addr + W_BYTES);
                static_assert(TC_BK == 64, "four k-steps a k-block");
                tc_mma_x4(tmem, dw, dx, idesc, i ? 1u : 0u);
                tc_commit(empty0 + 8 * s);
            }
            if (ok) tc_commit(acc_full);
        }
    } else {
        // epilogue: thread = one row of W (tensor-memory lane); the BNB batch columns are taken CW at a
        // time so that a pass's sums fit the registers
        constexpr int CW = BNB < 64 ? BNB : 64;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // row within the tile
        const int n = n0 + r;
        float v[CW];
        ssb_pdl_wait();                                      // out and the scratch may still be the predecessor's
        bool ok = true;
        if (my_blocks > 0) {
            ok = mbar_wait(acc_full, 0, abort_flag);
            if (!ok) { *abort_flag = 1; atomicCAS(error_word, 0, TC_ERR_EPILOGUE); }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps agree on the outcome
        ok = abort_flag[0] == 0;
        if (ok && my_blocks > 0) tc_fence_after();
        // this block's sums of columns c0 .. c0 + CW - 1 (zeros for a block without k-blocks)
        auto own_sums = [&](int c0) {
            if (my_blocks > 0) {
#pragma unroll
                for (int c = 0; c < (CW + 31) / 32; ++c) {
                    uint32_t raw[32];
                    tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c0 + c * 32, raw);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c * 32 + j < CW) v[c * 32 + j] = __uint_as_float(raw[j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CW; ++j) v[j] = 0.f;
            }
        };
        // Adding into the float32 residual with K split over blocks and no scratch: each block adds its
        // share straight in (red.global.add.f32).  The order in which shares meet varies from run to
        // run, so the last bits of the residual may; everything else uses the ordered fix-up below.
        // With scratch given, an add is ordered too: the last block of the tile adds the sum of the shares.
        const bool atomic_add = splits > 1 && mode == TC_ACCUMULATE && partials == nullptr;
        const bool through_scratch = splits > 1 && !atomic_add;
        if (ok && through_scratch) {
            // partial tile to scratch; the block that arrives last adds all of them in split order
            float* mine = partials + (((size_t)tile * splits + split) * GV_BM + r) * BNB;
            for (int c0 = 0; c0 < BNB; c0 += CW) {
                own_sums(c0);
#pragma unroll
                for (int j = 0; j < CW; j += 4)
                    *reinterpret_cast<float4*>(mine + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
            if (warp == 2 && lane == 0) {
                const int arrived = atomicAdd(counters + tile, 1);
                *is_last = (arrived == splits - 1);
                if (*is_last) counters[tile] = 0;            // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = *is_last != 0;
            if (ok) __threadfence();
        }
        if (ok) {
            for (int c0 = 0; c0 < BNB; c0 += CW) {
                if (through_scratch) {
#pragma unroll
                    for (int j = 0; j < CW; ++j) v[j] = 0.f;
                    for (int sp = 0; sp < splits; ++sp) {
                        const float* p = partials + (((size_t)tile * splits + sp) * GV_BM + r) * BNB + c0;
#pragma unroll
                        for (int j = 0; j < CW; j += 4) {
                            const float4 t4 = __ldcg(reinterpret_cast<const float4*>(p + j));
                            v[j] += t4.x; v[j + 1] += t4.y; v[j + 2] += t4.z; v[j + 3] += t4.w;
                        }
                    }
                } else {
                    own_sums(c0);
                }
                if (mode == TC_SWIGLU) {
                    // rows come as [8 gate | 8 up] per 16: the up value of gate row r sits 8 lanes further
                    const bool is_gate = (r & 15) < 8;
                    const int n_out = n0 / 2 + (r >> 4) * 8 + (r & 7);
                    // sixteen columns at a time, each step for all of them before the next: shuffle,
                    // activation and store of one column are a chain of dependent instructions, and taken
                    // column by column the 64 columns of a full tile took 9 us
#pragma unroll
                    for (int j0 = 0; j0 < CW; j0 += 16) {
                        float up[16], act[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) up[j] = __shfl_down_sync(0xffffffffu, v[j0 + j], 8);
#pragma unroll
                        for (int j = 0; j < 16; ++j) act[j] = __fdividef(v[j0 + j], 1.0f + __expf(-v[j0 + j])) * up[j];
                        if (is_gate && n + 8 < N) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c0 + j0 + j < n_rows)
                                    ((bf16*)out)[(size_t)(c0 + j0 + j) * ldo + n_out] = __float2bfloat16_rn(act[j]);
                        }
                    }
                } else if (n < N) {
#pragma unroll
                    for (int j = 0; j < CW; ++j) {
                        if (c0 + j >= n_rows) break;
                        const size_t o = (size_t)(c0 + j) * ldo + n;
                        if (atomic_add) { if (my_blocks > 0) atomicAdd((float*)out + o, v[j]); }
                        else if (mode == TC_ACCUMULATE) ((float*)out)[o] += v[j];
                        else if (out_is_f32) ((float*)out)[o] = v[j];
                        else ((bf16*)out)[o] = __float2bfloat16_rn(v[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int BNB>
static int launch_gv(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int ldo, int out_is_f32, int n_rows,
                     int N, int K, int mode, int splits, float* partials, int* counters, int* error_word, bool pdl,
                     cudaStream_t stream) {
    constexpr int GV_STAGES = gv_stages(BNB);
    constexpr size_t smem = GV_STAGES * (GV_BM + BNB) * TC_BK * 2 + (2 * GV_STAGES + 1) * 8 + 32 + 1024;
    auto kern = gemv_tc_kernel<BNB>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int rc = ssb_launch(kern, dim3((N + GV_BM - 1) / GV_BM, splits), dim3(GV_THREADS), smem, stream, pdl, mw, mx,
                              out, ldo, out_is_f32, n_rows, N, K, mode, splits, partials, counters, error_word);
    return rc ? rc : ssb_launch_status();
}

static inline int gv_bnb(int n_rows) { return n_rows <= 16 ? 16 : (n_rows <= 32 ? 32 : (n_rows <= 64 ? 64 : 128)); }
SSB_API int ssb_gemv_tc_max_rows() { return GV_MAX_ROWS; }

// Scratch for a launch with splits > 1: floats for the partial tiles, ints (zeroed once) for the counters.
SSB_API long long ssb_gemv_tc_scratch_floats(int n_rows, int N, int splits) {
    const int bnb = gv_bnb(n_rows);
    return splits > 1 ? (long long)((N + GV_BM - 1) / GV_BM) * splits * GV_BM * bnb : 0;
}
SSB_API int ssb_gemv_tc_counters(int N) { return (N + GV_BM - 1) / GV_BM; }

// x: bfloat16 [n_rows <= 128, K]; W: bfloat16 [N, K]; modes as ssb_gemm_tc.  splits: blocks that
// share the K range of a row tile (1 = none).
SSB_API int ssb_gemv_tc(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int out_dtype,
                        int n_rows, int N, int K, int mode, int splits, float* partials, int* counters,
                        int* error_word, int pdl, cudaStream_t stream) {
    if (n_rows <= 0 || N <= 0) return 0;
    if (n_rows > GV_MAX_ROWS || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || !error_word || splits < 1) return SSB_ERR_BAD_SIZE;
    if (((uintptr_t)x | (uintptr_t)W | (uintptr_t)partials) & 15) return SSB_ERR_BAD_SIZE;
    if (splits > 1 && (mode != TC_ACCUMULATE || partials) && (!partials || !counters)) return SSB_ERR_BAD_SIZE;
    if (splits > (K + TC_BK - 1) / TC_BK) return SSB_ERR_BAD_SIZE;
    if (mode == TC_ACCUMULATE && out_dtype != SSB_F32) return SSB_ERR_BAD_DTYPE;
    if (mode == TC_SWIGLU && (out_dtype != SSB_BF16 || N % 16)) return SSB_ERR_BAD_SIZE;
    const int bnb = gv_bnb(n_rows);
    CUtensorMap mw, mx;
    int rc = make_map(&mw, W, N, K, ldw, GV_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, n_rows, K, ldx, bnb);
    if (rc) return rc;
    const int f32o = out_dtype == SSB_F32;
    if (bnb == 16) return launch_gv<16>(mw, mx, out, ldo, f32o, n_rows, N, K, mode, splits, partials, counters, error_word, pdl != 0, stream);
    if (bnb == 32) return launch_gv<32>(mw, mx, out, ldo, f32o, n_rows, N, K, mode, splits, partials, counters, error_word, pdl != 0, stream);
    if (bnb == 64) return launch_gv<64>(mw, mx, out, ldo, f32o, n_rows, N, K, mode, splits, partials, counters, error_word, pdl != 0, stream);
    return launch_gv<128>(mw, mx, out, ldo, f32o, n_rows, N, K, mode, splits, partials, counters, error_word, pdl != 0, stream);
}
