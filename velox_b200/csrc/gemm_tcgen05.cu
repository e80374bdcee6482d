// C[M,N] = A[M,K] * W[N,K]^T (+ bias) in bfloat16 on the fifth-generation tensor
// cores: tcgen05.mma with the accumulator in tensor memory, operands brought into
// shared memory by TMA.
//
// Blocks are persistent (one per SM); each takes 128 x BN tiles of C (BN = 128 or
// 256) in turn and has six warps, which work on different tiles at once: while the
// epilogue warps write tile i from one half of the tensor memory, the tensor core
// already accumulates tile i + 1 in the other half, fed by a ring of stages that
// runs on across tiles:
//   warp 0   producer: one thread waits for a free stage and issues two tiled TMA
//            loads (cp.async.bulk.tensor.2d, 128-byte swizzle): a 128 x 64 tile of A
//            and a BN x 64 tile of W, completion counted on the stage's "full"
//            mbarrier;
//   warp 1   allocates 2 x BN columns of tensor memory; one thread waits for a full
//            stage, issues four tcgen05.mma (M 128, N BN, K 16 each) whose operands
//            are shared-memory descriptors of the swizzled tiles, and commits them to
//            the stage's "empty" mbarrier, so the stage is free when the tensor core
//            has read it; after a tile's last k block it commits to that
//            accumulator's "full" mbarrier, and before it reuses an accumulator it
//            waits for its "empty" mbarrier;
//   warps 2-5  epilogue: each reads its 32 lanes (rows) of the accumulator with
//            tcgen05.ld, 32 columns at a time, adds the bias, rounds to bfloat16 and
//            stores; or, gated, takes act(gate) * up of column tiles laid out as 8
//            gate columns followed by their 8 up columns, in float32, and stores
//            half as many columns; then they arrive on the accumulator's "empty"
//            mbarrier.
// Rows past M and columns past N are zero-filled by TMA on the way in and masked on
// the way out; K may end inside a k block (zero-filled too).
//
// Every wait on an mbarrier is bounded.  If one runs out the block records a code
// in the caller's error word, the other roles run out of their own bounded waits,
// and the block frees its tensor memory and returns.
//
// Sizes: K a multiple of 8, rows of A, W and C 16-byte aligned, N a multiple of 16.
#include "tcgen05_gemm.cuh"

template <int BN, int STAGES, bool GATED>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, bf16* __restrict__ C, int M, int N, int K, int ldc, int act,
                    int* __restrict__ error) {
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int failed;
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    // the swizzled tiles must start on 1024-byte boundaries
    unsigned char* tiles = (unsigned char*)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    // Tiles are numbered with the row tile running fastest, so that blocks working
    // at the same time share a tile of W and walk over the rows of A (which stays
    // in L2): W is read from memory once.  Block b takes tiles b, b + grid, ...
    const int mtiles = (M + TC_BM - 1) / TC_BM, ntiles = (N + BN - 1) / BN;
    const int total_tiles = mtiles * ntiles;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc_mbar_init(tc_smem_u32(&full_bar[s]), 1);
            tc_mbar_init(tc_smem_u32(&empty_bar[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(tc_smem_u32(&acc_full[i]), 1);
            tc_mbar_init(tc_smem_u32(&acc_empty[i]), 4);   // one arrival per epilogue warp
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: two accumulators of BN columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem_u32(&tmem_base_s)), "r"((unsigned)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---- producer: one continuous stream of stages over all of this block's tiles ----
        if (lane == 0) {
            int it = 0;
            for (int ti = 0; ti < my_tiles && !failed; ++ti) {
                const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
                const int m0 = (tile % mtiles) * TC_BM, n0 = (tile / mtiles) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES &&
                        !tc_mbar_wait(tc_smem_u32(&empty_bar[s]), (unsigned)(((it / STAGES) - 1) & 1))) {
                        failed = 1;
                        atomicExch(error, TC_ERR_PRODUCER);
                        break;
                    }
                    const unsigned bar = tc_smem_u32(&full_bar[s]);
                    tc_mbar_expect_tx(bar, STAGE_BYTES);
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    tc_tma_load_2d(tc_smem_u32(st), &map_a, kb * TC_BK, m0, bar);
                    tc_tma_load_2d(tc_smem_u32(st + A_BYTES), &map_w, kb * TC_BK, n0, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor core: tile ti accumulates into buffer ti & 1 ----
        if (lane == 0) {
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = BN, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) |
                                   ((unsigned)(TC_BM >> 4) << 24);
            int it = 0;
            for (int ti = 0; ti < my_tiles && !failed; ++ti) {
                const int buf = ti & 1;
                // the epilogue must have emptied this buffer (it last held tile ti - 2)
                if (ti >= 2 && !tc_mbar_wait(tc_smem_u32(&acc_empty[buf]), (unsigned)(((ti >> 1) - 1) & 1))) {
                    failed = 1;
                    atomicExch(error, TC_ERR_MMA);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)(buf * BN);
                bool ok = true;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc_mbar_wait(tc_smem_u32(&full_bar[s]), (unsigned)((it / STAGES) & 1))) {
                        failed = 1;
                        atomicExch(error, TC_ERR_MMA);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned a_addr = tc_smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    const unsigned long long adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)   // 32 bytes further along K inside the swizzle atom
                        tc_mma(tmem_d, adesc + (unsigned long long)(k4 * 2), bdesc + (unsigned long long)(k4 * 2),
                               idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                    tc_commit(tc_smem_u32(&empty_bar[s]));   // the stage is free once these have read it
                }
                if (!ok) break;
                tc_commit(tc_smem_u32(&acc_full[buf]));      // the accumulator is complete once all have finished
            }
        }
    } else {
        // ---- epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of tensor memory ----
        const int quarter = warp & 3;
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int buf = ti & 1;
            const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
            const int m0 = (tile % mtiles) * TC_BM, n0 = (tile / mtiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            bool ok = tc_mbar_wait(tc_smem_u32(&acc_full[buf]), (unsigned)((ti >> 1) & 1));
            if (!ok && lane == 0) { failed = 1; atomicExch(error, TC_ERR_EPILOGUE); }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned tmem_acc = tmem_base + (unsigned)(buf * BN) + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= N) break;   // (uniform) columns past N hold zeros
                unsigned r[32];
                tc_ld32(tmem_acc + (unsigned)c0, r);
                if (row >= M) continue;
                if (!GATED) {
                    bf16* dst = C + (size_t)row * ldc + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n0 + c0 + j >= N) break;
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[i] = __uint_as_float(r[j + i]);
                            if (bias) v[i] += bias[n0 + c0 + j + i];
                        }
                        uint4 pk;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                        *reinterpret_cast<uint4*>(dst + j) = pk;
                    }
                } else {
                    bf16* dst = C + (size_t)row * ldc + ((n0 + c0) >> 1);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {   // two tiles of 8 gates + 8 ups
                        if (n0 + c0 + t * 16 >= N) break;
                        uint4 pk;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float g0 = __uint_as_float(r[t * 16 + 2 * i]), g1 = __uint_as_float(r[t * 16 + 2 * i + 1]);
                            const float u0 = __uint_as_float(r[t * 16 + 8 + 2 * i]), u1 = __uint_as_float(r[t * 16 + 9 + 2 * i]);
                            h[i] = __floats2bfloat162_rn(activation(g0, act) * u0, activation(g1, act) * u1);
                        }
                        *reinterpret_cast<uint4*>(dst + t * 8) = pk;
                    }
                }
            }
            // the buffer may be overwritten once all four epilogue warps have read it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem_u32(&acc_empty[buf])) : "memory");
        }
    }
    // everybody meets before the tensor memory goes back (every wait above was bounded)
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)(2 * BN)) : "memory");
    }
}

// ---- host side ----
template <int BN, int STAGES, bool GATED>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, bf16* C, int M, int N, int K,
                     int ldc, int act, int* error, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(gemm_tcgen05_kernel<BN, STAGES, GATED>, smem, configured)) return rc;
    // persistent: one block per SM (its shared memory fills one), fewer if there are fewer tiles
    static int sm_counts[VX_MAX_DEVICES];
    const int sms = vx_sm_count(sm_counts);
    const int tiles = ((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
    dim3 grid(tiles < sms ? tiles : sms);
    VX_LAUNCH_K(VX_K_GEMM, (gemm_tcgen05_kernel<BN, STAGES, GATED>), grid, TC_THREADS, smem, stream, ma, mw, bias, C, M,
                N, K, ldc, act, error);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// gated: 0 plain, C is [M, N]; 1: W's rows come in tiles of 8 gate rows followed by
// their 8 up rows and C is [M, N/2] = act(gate) * up.  `error` is a device int that
// a block sets (TC_ERR_*) if one of its bounded waits runs out; the caller zeroes it
// and reads it when it wants to know.  `wide` picks 128 x 256 tiles (else 128 x 128).
extern "C" int vx_gemm_tcgen05(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int lda,
                               int ldw, int ldc, int gated, int act, int wide, int* error, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VX_OK;
    if (K <= 0 || (K & 7) || (N & 15) || !error) return VX_ERR_SHAPE;
    if ((lda & 7) || (ldw & 7) || (ldc & 7) || lda < K || ldw < K) return VX_ERR_ALIGN;
    if ((((uintptr_t)A) | ((uintptr_t)W) | ((uintptr_t)C)) & 15) return VX_ERR_ALIGN;
    if (gated && (bias || act < 0 || act > 3)) return VX_ERR_SHAPE;
    if (ldc < (gated ? N / 2 : N)) return VX_ERR_SHAPE;
    CUtensorMap ma, mw;
    const int bn = wide ? 256 : 128;
    if (!tc_make_map(&ma, A, M, K, lda, TC_BM) || !tc_make_map(&mw, W, N, K, ldw, bn)) return VX_ERR_DRIVER;
    bf16* c = (bf16*)C;
    if (wide)
        return gated ? tc_launch<256, 4, true>(ma, mw, bias, c, M, N, K, ldc, act, error, stream)
                     : tc_launch<256, 4, false>(ma, mw, bias, c, M, N, K, ldc, act, error, stream);
    return gated ? tc_launch<128, 6, true>(ma, mw, bias, c, M, N, K, ldc, act, error, stream)
                 : tc_launch<128, 6, false>(ma, mw, bias, c, M, N, K, ldc, act, error, stream);
}
