// C[M,N] = A[M,K] * W[N,K]^T (+ bias) in bfloat16 with two blocks on one tile:
// tcgen05.mma.cta_group::2 forms a 256 x 256 tile of C on the tensor cores of a
// pair of SMs (a cluster of two blocks).  Block r of the pair brings rows
// m0 + 128 r .. + 127 of A and rows n0 + 128 r .. + 127 of W into its own shared
// memory (plain TMA loads, each block its own; nothing is multicast), the tensor
// cores of both SMs read both halves of W, and each block's tensor memory holds
// the 128 x 256 accumulator of its rows.  Against one block per 128 x 256 tile
// every SM reads half as many bytes of W from shared memory per multiply-add,
// which is what limits the single-block kernel.
//
// Clusters are persistent (one per pair of SMs) and take tiles in turn, the row
// tile running fastest.  In each block:
//   warp 0   producer: one thread waits for a free stage of its own block and
//            issues its two loads; their bytes are counted on the "full" mbarrier
//            of the leading block (rank 0), which expects both blocks' bytes;
//   warp 1   allocates all 512 columns of tensor memory (both blocks, the same
//            warp); in the leading block one thread waits for a full stage, issues
//            four products (M 256, N 256, K 16) and commits them to the stage's
//            "empty" mbarrier in both blocks; after a tile's last k block it
//            commits to the accumulator's "full" mbarrier in both blocks;
//   warps 2-5  epilogue of the block's own 128 rows (tcgen05.ld, bias or gated
//            activation, bfloat16 stores), then an arrival on the leading block's
//            accumulator "empty" mbarrier (eight arrivals free it).
// Two accumulators of 256 columns alternate, so a tile's epilogue runs under the
// next tile's products.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in the
// caller's error word, the other roles and the other block run out of their own
// bounded waits, both blocks meet at the cluster's barrier, free their tensor
// memory and return.
//
// Sizes: K a multiple of 8, rows of A, W and C 16-byte aligned, N a multiple of 16.
#include "tcgen05_gemm.cuh"

#define TP_BN 256
#define TP_HALF 128   // rows of W a block loads
#define TP_ERR_PRODUCER 4
#define TP_ERR_MMA 5
#define TP_ERR_EPILOGUE 6

__device__ __forceinline__ unsigned tp_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of `addr` in the block of rank `rank`.
__device__ __forceinline__ unsigned tp_map_to_rank(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void tp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A tiled load into this block's shared memory whose bytes are counted on an mbarrier
// that may live in the other block of the pair (`bar`: an address in the cluster's window).
__device__ __forceinline__ void tp_tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tp_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                       unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// One arrival, when the products issued so far have completed, on the mbarrier at this
// offset in both blocks of the pair.
__device__ __forceinline__ void tp_commit_both(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tp_arrive_remote(unsigned bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

template <int STAGES, bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const float* __restrict__ bias, bf16* __restrict__ C, int M, int N, int K, int ldc, int act,
                         int* __restrict__ error) {
    extern __shared__ unsigned char tp_smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int failed;
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, W_BYTES = TP_HALF * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    unsigned char* tiles = (unsigned char*)(((uintptr_t)tp_smem_raw + 1023) & ~(uintptr_t)1023);
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = tp_cluster_rank();
    const int nkb = (K + TC_BK - 1) / TC_BK;
    const int mtiles = (M + 2 * TC_BM - 1) / (2 * TC_BM), ntiles = (N + TP_BN - 1) / TP_BN;
    const int total_tiles = mtiles * ntiles;
    const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
    const int my_tiles = (total_tiles - pair + pairs - 1) / pairs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc_mbar_init(tc_smem_u32(&full_bar[s]), 1);    // the leading block's producer (with both blocks' bytes)
            tc_mbar_init(tc_smem_u32(&empty_bar[s]), 1);   // the commit of the products that read the stage
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(tc_smem_u32(&acc_full[i]), 1);
            tc_mbar_init(tc_smem_u32(&acc_empty[i]), 8);   // one arrival per epilogue warp of both blocks
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: two accumulators of 256 columns x 128 lanes in each block
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem_u32(&tmem_base_s)), "r"((unsigned)(2 * TP_BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    tp_cluster_sync();   // the other block's mbarriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---- producer (both blocks): this block's halves of every stage ----
        if (lane == 0) {
            int it = 0;
            for (int ti = 0; ti < my_tiles && !failed; ++ti) {
                const int tile = pair + ti * pairs;
                const int m0 = (tile % mtiles) * (2 * TC_BM) + (int)rank * TC_BM;
                const int n0 = (tile / mtiles) * TP_BN + (int)rank * TP_HALF;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES &&
                        !tc_mbar_wait(tc_smem_u32(&empty_bar[s]), (unsigned)(((it / STAGES) - 1) & 1))) {
                        failed = 1;
                        atomicExch(error, TP_ERR_PRODUCER);
                        break;
                    }
                    if (rank == 0) tc_mbar_expect_tx(tc_smem_u32(&full_bar[s]), 2 * STAGE_BYTES);
                    const unsigned bar = tp_map_to_rank(tc_smem_u32(&full_bar[s]), 0);
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    tp_tma_load_2d(tc_smem_u32(st), &map_a, kb * TC_BK, m0, bar);
                    tp_tma_load_2d(tc_smem_u32(st + A_BYTES), &map_w, kb * TC_BK, n0, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor cores of the pair, driven by the leading block ----
        if (lane == 0 && rank == 0) {
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = 256, M = 256
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TP_BN >> 3) << 17) |
                                   ((unsigned)((2 * TC_BM) >> 4) << 24);
            int it = 0;
            for (int ti = 0; ti < my_tiles && !failed; ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !tc_mbar_wait(tc_smem_u32(&acc_empty[buf]), (unsigned)(((ti >> 1) - 1) & 1))) {
                    failed = 1;
                    atomicExch(error, TP_ERR_MMA);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)(buf * TP_BN);
                bool ok = true;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!tc_mbar_wait(tc_smem_u32(&full_bar[s]), (unsigned)((it / STAGES) & 1))) {
                        failed = 1;
                        atomicExch(error, TP_ERR_MMA);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned a_addr = tc_smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    const unsigned long long adesc = tc_smem_desc(a_addr), bdesc = tc_smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        tp_mma(tmem_d, adesc + (unsigned long long)(k4 * 2), bdesc + (unsigned long long)(k4 * 2),
                               idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                    tp_commit_both(tc_smem_u32(&empty_bar[s]));
                }
                if (!ok) break;
                tp_commit_both(tc_smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---- epilogue (both blocks): warp w reads lanes 32 * (w % 4) .. + 31 of its block's tensor memory ----
        const int quarter = warp & 3;
        const unsigned lead_empty[2] = {tp_map_to_rank(tc_smem_u32(&acc_empty[0]), 0),
                                        tp_map_to_rank(tc_smem_u32(&acc_empty[1]), 0)};
        for (int ti = 0; ti < my_tiles; ++ti) {
            const int buf = ti & 1;
            const int tile = pair + ti * pairs;
            const int m0 = (tile % mtiles) * (2 * TC_BM) + (int)rank * TC_BM, n0 = (tile / mtiles) * TP_BN;
            const int row = m0 + quarter * 32 + lane;
            bool ok = tc_mbar_wait(tc_smem_u32(&acc_full[buf]), (unsigned)((ti >> 1) & 1));
            if (!ok && lane == 0) { failed = 1; atomicExch(error, TP_ERR_EPILOGUE); }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned tmem_acc = tmem_base + (unsigned)(buf * TP_BN) + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < TP_BN; c0 += 32) {
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
            // the buffer may be overwritten once the epilogue warps of both blocks have read it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) tp_arrive_remote(lead_empty[buf]);
        }
    }
    // Both blocks meet before the tensor memory goes back: the leading block's products read the
    // other block's shared memory and arrive on its mbarriers (every wait above was bounded).
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    tp_cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((unsigned)(2 * TP_BN)) : "memory");
    }
}

template <int STAGES, bool GATED>
static int tp_launch(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, bf16* C, int M, int N, int K,
                     int ldc, int act, int* error, cudaStream_t stream) {
    const size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + TP_HALF * TC_BK * 2) + 1024;
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(gemm_tcgen05_pair_kernel<STAGES, GATED>, smem, configured)) return rc;
    // persistent: one cluster per pair of SMs, fewer if there are fewer tiles
    static int sm_counts[VX_MAX_DEVICES];
    const int pairs_max = vx_sm_count(sm_counts) / 2;
    const int tiles = ((M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + TP_BN - 1) / TP_BN);
    dim3 grid(2 * (tiles < pairs_max ? tiles : pairs_max));
    // (plain stream order: the cluster's size is fixed at compile time and the launch carries no attribute)
    gemm_tcgen05_pair_kernel<STAGES, GATED><<<grid, TC_THREADS, smem, stream>>>(ma, mw, bias, C, M, N, K, ldc, act, error);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// The same contract as vx_gemm_tcgen05, on 256 x 256 tiles formed by pairs of blocks.
extern "C" int vx_gemm_tcgen05_pair(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                                    int lda, int ldw, int ldc, int gated, int act, int* error, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VX_OK;
    if (K <= 0 || (K & 7) || (N & 15) || !error) return VX_ERR_SHAPE;
    if ((lda & 7) || (ldw & 7) || (ldc & 7) || lda < K || ldw < K) return VX_ERR_ALIGN;
    if ((((uintptr_t)A) | ((uintptr_t)W) | ((uintptr_t)C)) & 15) return VX_ERR_ALIGN;
    if (gated && (bias || act < 0 || act > 3)) return VX_ERR_SHAPE;
    if (ldc < (gated ? N / 2 : N)) return VX_ERR_SHAPE;
    CUtensorMap ma, mw;
    if (!tc_make_map(&ma, A, M, K, lda, TC_BM) || !tc_make_map(&mw, W, N, K, ldw, TP_HALF)) return VX_ERR_DRIVER;
    bf16* c = (bf16*)C;
    return gated ? tp_launch<6, true>(ma, mw, bias, c, M, N, K, ldc, act, error, stream)
                 : tp_launch<6, false>(ma, mw, bias, c, M, N, K, ldc, act, error, stream);
}
