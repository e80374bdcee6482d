// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands by TMA), bfloat16, head
// size 128.
//
// grid (pairs of query tiles x kv heads x runs, 1, request), one block per SM at a
// time, numbered longest first.  A block takes TWO query tiles of 128 rows of one
// request, each 128 / G consecutive new tokens for each of the G query heads of one
// kv head (G from 1 to 8; 128 / G rounded down to a multiple of 8, so that every head's rows
// start on a boundary of the shared-memory swizzle), so the heads of a group and both tiles share every
// key/value tile.  It walks over the request's keys in tiles of 128.
//
//   warps 0-3, 4-7  softmax of query tile 0 and of query tile 1: a thread owns one
//               row (one lane of tensor memory) and holds its 128 scores in
//               registers.  It masks by select (causal: key <= the row's position;
//               window: key >= position + 1 - W), takes 2^(s - m) against a
//               reference m that comes from the row's earlier tiles (its own
//               maximum only for a row's first keys, a masked tile, or when the
//               tile's sum shows that the scores have outgrown the reference),
//               keeps m and the row's sum in float32 (base 2), writes the
//               probabilities back over the scores as packed bfloat16, and rescales
//               its row of O when the reference moves (by more than 2^8).  At the end
//               it divides O by the sum and stores its row.
//   warp 8      tensor core: one thread issues, for each key tile and each query
//               tile q, O_q += P_q V (A operand straight from tensor memory, V as the
//               MN-major B operand) and then S_q = Q_q K^T of the NEXT key tile over
//               the probabilities just used (the tensor core takes its instructions
//               in order), so that one query tile's softmax runs under the other's
//               products;
//   warps 9-11  producers: keys (warp 9) and values (warp 10), page by page with
//               tiled TMA loads (128-byte swizzle), one 16-key x 64-column box per
//               lane, into two shared-memory buffers each; the two query tiles once
//               (warp 11).
// Registers move from warps 8-11 to the softmax warps (setmaxnreg).  In the steady
// state the tensor core sets the pace: 32 products of 128 x 128 x 16 per key tile
// take about 3,450 cycles, of which a softmax thread is busy for 1,830.
//
// Keys past the request's last key and below its window are masked; the values of a
// tile that reaches past the last key are cleared in shared memory first, because a
// never-written slot may hold NaN and 0 * NaN is NaN in the tensor core.
//
// Every wait on an mbarrier is bounded.  If one runs out the block records a code
// in the caller's error word, the other roles run out of their own bounded waits,
// and the block frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

#define PT_ROWS 128
#define PT_KEYS 128
#define PT_D 128
#define PT_QTILES 2                  // query tiles a block works on
#define PT_THREADS 384
#define PT_MMA_WARP 8                // warps 0-3: softmax of query tile 0, 4-7: of tile 1, 8: tensor core, 9-11: producers
#define PT_SPIN_LIMIT (1 << 24)
#define PT_LOG2E 1.4426950408889634f
#define PT_HALF_BYTES (128 * 128)   // 128 rows x 64 columns of bf16: one swizzled half of a tile
#define PT_TILE_BYTES (2 * PT_HALF_BYTES)
#define PT_RESCALE_THRESHOLD 8.0f
#define PT_SUM_LIMIT 16777216.f    // 2^24: a tile's sum of probabilities beyond which its own maximum is taken

__device__ __forceinline__ unsigned pt_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pt_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void pt_mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pt_mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool pt_mbar_wait(unsigned bar, unsigned parity) {
    for (int i = 0; i < PT_SPIN_LIMIT; ++i) {
        unsigned ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void pt_tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory descriptors, 128-byte swizzle, version 1.  K-major (Q and K: rows
// 128 bytes apart, groups of 8 rows 1024 bytes apart); MN-major (V: the 64-column
// halves 16 KB apart = leading offset, groups of 8 keys 1024 bytes apart).
__device__ __forceinline__ unsigned long long pt_desc_kmajor(unsigned addr) {
    return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | ((unsigned long long)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ unsigned long long pt_desc_mnmajor(unsigned addr) {
    return (unsigned long long)((addr >> 4) & 0x3FFF) | ((unsigned long long)(PT_HALF_BYTES >> 4) << 16) |
           ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void pt_mma_ss(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void pt_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for x <= 8 on the multiply-add pipes: x = n + f with n the nearest integer,
// 2^f by a cubic on [-0.5, 0.5] (relative error 1.4e-4, thirty times below the
// rounding of a probability to bfloat16), 2^n by an add to the exponent bits.  The
// special-function unit makes 16 exponentials a cycle per SM, which is as long as
// the tile's tensor-core work; every PT_POLY_EVERY-th exponential can go this way
// instead.  With eight softmax warps every fourth one did (8,192 tokens: 644 -> 613
// us); with sixteen the unit's latency hides behind the other warps and the cubic's
// nine instructions cost more than they save (8,192 tokens: 653 us with every
// fourth, 626 with every eighth, 600 with none), so none does by default.
#ifndef PT_POLY_EVERY
#define PT_POLY_EVERY 1024
#endif
__device__ __forceinline__ float pt_ex2_poly(float x) {
    x = fmaxf(x, -126.f);
    const float t = x + 12582912.f;          // 1.5 * 2^23: the sum's low mantissa bits hold n
    const float f = x - (t - 12582912.f);
    float p = fmaf(f, 0.055029310f, 0.24225681f);
    p = fmaf(p, f, 0.69325304f);
    p = fmaf(p, f, 0.99995136f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ void pt_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void pt_ld32_issue(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void pt_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void pt_ld32(unsigned taddr, unsigned (&r)[32]) {
    pt_ld32_issue(taddr, r);
    pt_wait_ld();
}
__device__ __forceinline__ void pt_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void pt_st16(unsigned taddr, const unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Tokens of a query tile: each of the G query heads of a kv head has as many rows of the tile's 128, a multiple of 8.
__device__ __host__ __forceinline__ int pt_toks_per_tile(int share) { return (PT_ROWS / share) & ~7; }

// A short portion on top of many cached keys has few query blocks (a 64-token portion at 4 query heads
// per kv head: one) but many key tiles for each to walk alone.  Its key tiles are then cut into `splits`
// runs that as many blocks take; each writes its unnormalised output and (reference, sum) per row, and
// the join kernel below adds the runs in order.  The number of runs depends on the request's own portion
// and keys only, never on what else is in the step.
__device__ __host__ __forceinline__ int pt_splits_of(int n_new, int kv_len, int toks_per_tile, int Hk, int max_splits,
                                                     int sms) {
    const int q_blocks = (n_new + PT_QTILES * toks_per_tile - 1) / (PT_QTILES * toks_per_tile);
    const int key_tiles = (kv_len + PT_KEYS - 1) / PT_KEYS;
    const int fill = sms / (q_blocks * Hk);  // no more runs than give every SM one block: a second wave would wait for the first
    if (fill < 2 || key_tiles < 8) return 1; // blocks enough for the SMs already, or nothing to cut
    int s = key_tiles / 4;                   // four key tiles a run at least
    s = s < fill ? s : fill;
    return s < max_splits ? s : max_splits;
}

// barriers of a block
struct PtBarriers {
    unsigned long long q_full[PT_QTILES];
    unsigned long long k_full[2], k_empty[2], v_full[2], v_empty[2];
    unsigned long long s_full[PT_QTILES], p_ready[PT_QTILES], pv_done[PT_QTILES];
};

__global__ void __launch_bounds__(PT_THREADS, 1)
paged_prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                  const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                                  int max_blocks, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ kv_offsets, const int* __restrict__ seq_list,
                                  bf16* __restrict__ out, int out_row_stride,
                                  float scale_log2, int window, int H, int Hk, int S, int share,
                                  float* __restrict__ part_o, float* __restrict__ part_ml, int max_splits, int sms,
                                  int* __restrict__ error) {
    extern __shared__ unsigned char pt_smem_raw[];
    __shared__ __align__(8) PtBarriers bars;
    __shared__ unsigned tmem_base_s;
    __shared__ int failed;
    unsigned char* smem = (unsigned char*)(((uintptr_t)pt_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;                                   // 2 x 32 KB
    unsigned char* k_s = smem + 2 * PT_TILE_BYTES;               // 2 x 32 KB
    unsigned char* v_s = smem + 4 * PT_TILE_BYTES;               // 2 x 32 KB
    if (threadIdx.x == 0) {   // (the maps' first use would otherwise wait for them: 1 % at 2,048 tokens)
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
    }
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are handed out in the order of blockIdx.x: the longest first (the last tokens of a prompt), over
    // all kv heads, so that the short ones fill the gaps at the end (with the kv head in blockIdx.y a head's
    // short blocks would come before the next head's long ones: 2,048 tokens took 50 instead of 34 us by the
    // same arithmetic).
    const int split = (int)blockIdx.x % max_splits;
    const int hk = ((int)blockIdx.x / max_splits) % Hk;
    const int qb = (int)gridDim.x / (max_splits * Hk) - 1 - (int)blockIdx.x / (max_splits * Hk);
    const int seq = seq_list ? seq_list[blockIdx.z] : (int)blockIdx.z;
    const int toks_per_tile = pt_toks_per_tile(share);
    const int row_base = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - row_base;
    const int t_base = qb * PT_QTILES * toks_per_tile;
    if (t_base >= n_new) return;   // (before anything is allocated)
    const int off = kv_offsets[seq];
    const int kv_total = off + n_new;
    const int splits = pt_splits_of(n_new, kv_total, toks_per_tile, Hk, max_splits, sms);
    if (split >= splits) return;
    const int* bt = block_table + (size_t)seq * max_blocks;
    // The two query tiles of the block: their tokens, the keys they see, the key tiles of those.
    int t0[PT_QTILES], live[PT_QTILES], tile_a[PT_QTILES], tile_b[PT_QTILES];
    int kv_lo_all = 0, kv_hi_all = 0, lo = 0, hi = 0;
#pragma unroll
    for (int q = 0; q < PT_QTILES; ++q) {
        t0[q] = t_base + q * toks_per_tile;
        live[q] = max(0, min(toks_per_tile, n_new - t0[q]));
        tile_a[q] = tile_b[q] = 0;
        if (live[q] > 0) {
            const int kv_hi = off + t0[q] + live[q];   // one past the last visible key of the tile
            const int kv_lo = window > 0 ? max(0, off + t0[q] + 1 - window) : 0;
            tile_a[q] = kv_lo / PT_KEYS;
            tile_b[q] = (kv_hi + PT_KEYS - 1) / PT_KEYS;
            if (q == 0) kv_lo_all = kv_lo;
            kv_hi_all = kv_hi;
        }
    }
    lo = tile_a[0];
    hi = live[1] > 0 ? tile_b[1] : tile_b[0];
    if (splits > 1) {
        // this block's run of the block's key tiles
        const int per = (hi - lo + splits - 1) / splits;
        lo += split * per;
        hi = min(lo + per, hi);
    }
    bool any = false;
#pragma unroll
    for (int q = 0; q < PT_QTILES; ++q) {
        tile_a[q] = max(tile_a[q], lo);
        tile_b[q] = live[q] > 0 ? min(tile_b[q], hi) : tile_a[q];
        if (tile_b[q] <= tile_a[q]) tile_a[q] = tile_b[q] = 0;   // nothing of this run for this query tile
        any = any || tile_b[q] > tile_a[q];
    }
    if (splits > 1) {
        // a query tile without a key in this run (early tokens of a portion see fewer keys) weighs nothing
#pragma unroll
        for (int q = 0; q < PT_QTILES; ++q) {
            if (live[q] > 0 && tile_b[q] == tile_a[q] && threadIdx.x < PT_ROWS) {
                const int r = threadIdx.x;
                const int hi_ = r / toks_per_tile, tok = r - hi_ * toks_per_tile;
                if (hi_ < share && tok < live[q]) {
                    const size_t p = ((size_t)(row_base + t0[q] + tok) * H + (hk * share + hi_)) * max_splits + split;
                    part_ml[2 * p] = -INFINITY;
                    part_ml[2 * p + 1] = 0.f;
                }
            }
        }
    }
    if (!any) return;
    {   // the tiles that are loaded: from the first tile any query tile wants to the last
        int first = hi, last = lo;
#pragma unroll
        for (int q = 0; q < PT_QTILES; ++q)
            if (tile_b[q] > tile_a[q]) { first = min(first, tile_a[q]); last = max(last, tile_b[q]); }
        lo = first;
        hi = last;
    }
    const int ntiles = hi - lo;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            pt_mbar_init(pt_smem_u32(&bars.k_full[i]), 1);
            pt_mbar_init(pt_smem_u32(&bars.k_empty[i]), 1);
            pt_mbar_init(pt_smem_u32(&bars.v_full[i]), 1);
            pt_mbar_init(pt_smem_u32(&bars.v_empty[i]), 1);
        }
        for (int q = 0; q < PT_QTILES; ++q) {
            pt_mbar_init(pt_smem_u32(&bars.q_full[q]), 1);
            pt_mbar_init(pt_smem_u32(&bars.s_full[q]), 1);
            pt_mbar_init(pt_smem_u32(&bars.p_ready[q]), 4);   // one arrival per softmax warp of the tile
            pt_mbar_init(pt_smem_u32(&bars.pv_done[q]), 1);
        }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == PT_MMA_WARP) {  // tensor memory: scores/probabilities of tiles 0 and 1, outputs of tiles 0 and 1 (128 columns each)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(pt_smem_u32(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (share * toks_per_tile < PT_ROWS && threadIdx.x < PT_QTILES * PT_ROWS) {
        // rows of the query tiles that belong to no head are never loaded: cleared, so that their scores are finite
        const int r = threadIdx.x & (PT_ROWS - 1), qq = threadIdx.x >> 7;
        if (r >= share * toks_per_tile) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<uint4*>(q_s + qq * PT_TILE_BYTES + (i >> 3) * PT_HALF_BYTES + r * 128 + (i & 7) * 16) =
                    make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_s;
    // Registers go from the group of the tensor-core and producer warps to the two groups of softmax warps,
    // whose threads hold a row of 128 scores each.  The block's pool is what it was launched with, 384 x 168
    // registers, and 256 x 216 + 128 x 72 is exactly that: a request beyond the pool would wait for ever.
    // (With 208 and 88 the softmax threads spill five registers and the kernel is 1.5-3 % slower.)
    if (warp >= PT_MMA_WARP) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    if (warp == PT_MMA_WARP + 1 || warp == PT_MMA_WARP + 2) {
        // ---------------- producers of keys (one warp) and values (the other) ----------------
        // A tile is 16 boxes of 16 keys x 64 columns (a page holds 16 keys or a multiple), one box
        // per lane; keys and values wait for their own buffers (a key buffer is free as soon as
        // the scores of both query tiles are formed, long before the value buffer of the same tile).
        const int which = warp - (PT_MMA_WARP + 1);           // keys / values
        const int g = (lane & 15) >> 1, half = lane & 1;
        const CUtensorMap* map = which ? &map_v : &map_k;
        for (int i = 0; i < ntiles && !failed; ++i) {
            const int b = i & 1;
            const int key_base = (lo + i) * PT_KEYS;
            // Groups of 16 keys outside [kv_lo, kv_hi) repeat the nearest group inside: they
            // are masked anyway, and their pages may not be this request's.
            int key = key_base + g * 16;
            key = max(min(key, (kv_hi_all - 1) & ~15), kv_lo_all & ~15);
            const int page = bt[key / S];   // (asked for before the wait below)
            const unsigned full = pt_smem_u32(which ? &bars.v_full[b] : &bars.k_full[b]);
            bool ok = true;
            if (lane == 0) {
                if (i >= 2)
                    ok = pt_mbar_wait(pt_smem_u32(which ? &bars.v_empty[b] : &bars.k_empty[b]),
                                      (unsigned)(((i >> 1) - 1) & 1));
                if (!ok) {
                    failed = 1;
                    atomicExch(error, 11);
                } else {
                    pt_mbar_expect_tx(full, PT_TILE_BYTES);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < 16) {
                const int y = (page * Hk + hk) * S + (key % S);
                unsigned char* dst = (which ? v_s : k_s) + b * PT_TILE_BYTES;
                pt_tma_load_2d(pt_smem_u32(dst + half * PT_HALF_BYTES + g * 16 * 128), map, half * 64, y, full);
            }
        }
    } else if (warp == PT_MMA_WARP + 3) {
        // ---------------- producer of the queries: for each shared head, its tokens' two 64-column halves ----------------
#pragma unroll
        for (int q = 0; q < PT_QTILES; ++q) {
            if (tile_b[q] == tile_a[q]) continue;
            if (lane == 0) pt_mbar_expect_tx(pt_smem_u32(&bars.q_full[q]), (unsigned)(2 * share * toks_per_tile * 128));   // (the heads' rows, two halves)
            __syncwarp();
            if (lane < 2 * share) {
                const int hi_ = lane >> 1, half = lane & 1;
                pt_tma_load_2d(pt_smem_u32(q_s + q * PT_TILE_BYTES + half * PT_HALF_BYTES + hi_ * toks_per_tile * 128), &map_q,
                               (hk * share + hi_) * PT_D + half * 64, row_base + t0[q], pt_smem_u32(&bars.q_full[q]));
            }
        }
    } else {
        // ---------------- tensor core ----------------
        if (lane == 0) {
            // S = Q K^T: float32 out, bf16 A and B, both K-major, N = 128 keys, M = 128 rows
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PT_KEYS >> 3) << 17) |
                                     ((unsigned)(PT_ROWS >> 4) << 24);
            // O += P V: A from tensor memory, B = V MN-major (bit 16), N = 128 (head size)
            const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(PT_D >> 3) << 17) |
                                     ((unsigned)(PT_ROWS >> 4) << 24);
            auto issue_s = [&](int q, int t) {   // scores of query tile q on key tile t, over the tile's scores/probabilities
                const unsigned qa = pt_smem_u32(q_s + q * PT_TILE_BYTES), ka = pt_smem_u32(k_s + ((t - lo) & 1) * PT_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < PT_D / 16; ++k) {
                    const unsigned o = (unsigned)((k >> 2) * PT_HALF_BYTES + (k & 3) * 32);
                    pt_mma_ss(tmem_base + (unsigned)(q * 128), pt_desc_kmajor(qa + o), pt_desc_kmajor(ka + o), idesc_s,
                              k > 0 ? 1u : 0u);
                }
                pt_commit(pt_smem_u32(&bars.s_full[q]));
            };
            bool ok = true;
            // the first key tile's scores
            ok = pt_mbar_wait(pt_smem_u32(&bars.k_full[0]), 0);
#pragma unroll
            for (int q = 0; q < PT_QTILES; ++q) {
                if (tile_b[q] > tile_a[q]) {
                    ok = ok && pt_mbar_wait(pt_smem_u32(&bars.q_full[q]), 0);   // (once: the queries stay)
                    if (ok && tile_a[q] == lo) {
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        issue_s(q, lo);
                    }
                }
            }
            if (ok) pt_commit(pt_smem_u32(&bars.k_empty[0]));
            for (int t = lo; t < hi && ok; ++t) {
                const int u = t - lo, b = u & 1;
                bool have_v = false, have_k = false;
#pragma unroll
                for (int q = 0; q < PT_QTILES; ++q) {
                    if (t >= tile_a[q] && t < tile_b[q]) {
                        // O_q += P_q V: the probabilities of this tile, the values
                        if (!have_v) { ok = ok && pt_mbar_wait(pt_smem_u32(&bars.v_full[b]), (unsigned)((u >> 1) & 1)); have_v = true; }
                        const int n = t - tile_a[q];
                        ok = ok && pt_mbar_wait(pt_smem_u32(&bars.p_ready[q]), (unsigned)(n & 1));
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        const unsigned va = pt_smem_u32(v_s + b * PT_TILE_BYTES);
#pragma unroll
                        for (int k = 0; k < PT_KEYS / 16; ++k)   // 16 keys a step: 8 columns of packed P, 2 KB of V
                            pt_mma_ts(tmem_base + (unsigned)(256 + q * 128), tmem_base + (unsigned)(q * 128 + k * 8),
                                      pt_desc_mnmajor(va + (unsigned)(k * 2048)), idesc_o, (n > 0 || k > 0) ? 1u : 0u);
                        pt_commit(pt_smem_u32(&bars.pv_done[q]));
                    }
                    if (t + 1 >= tile_a[q] && t + 1 < tile_b[q]) {
                        // the next scores of this query tile go where its probabilities were: the tensor core
                        // takes its instructions in order, so P V above has read them before
                        if (!have_k) { ok = ok && pt_mbar_wait(pt_smem_u32(&bars.k_full[b ^ 1]), (unsigned)(((u + 1) >> 1) & 1)); have_k = true; }
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        issue_s(q, t + 1);
                    }
                }
                if (!ok) break;
                pt_commit(pt_smem_u32(&bars.v_empty[b]));
                if (t + 1 < hi) pt_commit(pt_smem_u32(&bars.k_empty[b ^ 1]));
            }
            if (!ok) { failed = 1; atomicExch(error, 12); }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
        // ---------------- softmax and epilogue: warps 0-3 query tile 0, warps 4-7 query tile 1; a thread owns a row ----------------
        const int q = warp >> 2;
        const int my_t0 = q ? t0[1] : t0[0], my_live = q ? live[1] : live[0];
        const int my_a = q ? tile_a[1] : tile_a[0], my_b = q ? tile_b[1] : tile_b[0];
        const int quarter = warp & 3;                            // the warp's quarter of tensor memory's lanes
        const int r = quarter * 32 + lane;                       // row of the tile = lane of tensor memory
        // (with 3, 5, 6 or 7 heads a kv head the tile's last rows belong to no head: they act as rows beyond the portion)
        const int hi_raw = r / toks_per_tile;
        const int hi_ = hi_raw < share ? hi_raw : 0, tok = hi_raw < share ? r - hi_raw * toks_per_tile : toks_per_tile;
        // (rows beyond the portion's last token act as the last token: they are computed and not stored)
        const int pos = min(off + my_t0 + tok, kv_total - 1);
        const int lo_key = window > 0 ? pos + 1 - window : 0;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned s_addr = tmem_base + (unsigned)(q * 128) + lane_addr;
        const unsigned o_addr = tmem_base + (unsigned)(256 + q * 128) + lane_addr;
        const int my_tiles = my_b - my_a;
        float m_used = -INFINITY, l = 0.f;
        const int warp_min_pos = __reduce_min_sync(0xffffffffu, pos), warp_max_lo = __reduce_max_sync(0xffffffffu, lo_key);
        bool ok = true;
        for (int n = 0; n < my_tiles; ++n) {
            const int t = my_a + n;
            const int key_base = t * PT_KEYS;
            ok = pt_mbar_wait(pt_smem_u32(&bars.s_full[q]), (unsigned)(n & 1));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // the row's 128 scores are read once and stay in registers for both passes
            unsigned v[PT_KEYS];
#pragma unroll
            for (int c = 0; c < 4; ++c) pt_ld32_issue(s_addr + (unsigned)(c * 32), *reinterpret_cast<unsigned(*)[32]>(&v[c * 32]));
            pt_wait_ld();
            // A tile that every row of the warp sees whole needs no masking at all.
            const bool whole = key_base + PT_KEYS - 1 <= warp_min_pos && key_base >= warp_max_lo;
            if (!whole) {
#pragma unroll
                for (int j = 0; j < PT_KEYS; ++j) {
                    const int key = key_base + j;
                    if (!(key <= pos && key >= lo_key)) v[j] = 0xff800000u;   // -inf
                }
            }
            // The reference of the exponentials comes from the row's earlier tiles whenever it can: softmax does
            // not care what it is relative to, and bfloat16 probabilities and float32 sums are as exact at 2^20
            // as at 1.  The tile's own maximum (a pass over the 128 scores) is taken only for a row's first keys,
            // for a masked tile, or when the tile's sum shows that its scores have outgrown the reference
            // (a sum of 2^24 or more, infinity included); then the reference moves and O is rescaled, as it is
            // when the maximum has grown by more than the threshold 2^8.
            bool with_max = __any_sync(0xffffffffu, !whole || m_used == -INFINITY);
            float tile_sum = 0.f;
#pragma unroll 1
            for (int attempt = 0; attempt < 2 && ok; ++attempt) {
                if (with_max) {
                    // the maximum, in eight chains of three-input maxima
                    float m8[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) m8[c] = -INFINITY;
#pragma unroll
                    for (int j = 0; j < PT_KEYS; j += 2)
                        asm("max.f32 %0, %0, %1, %2;\n" : "+f"(m8[(j >> 1) & 7]) : "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])));
                    float mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
                    mx *= scale_log2;   // (the scale is positive)
                    float alpha = 1.f;
                    const bool move = mx > m_used + PT_RESCALE_THRESHOLD;
                    if (move) {
                        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
                        m_used = mx;
                        l *= alpha;
                    }
                    if (n > 0 && __any_sync(0xffffffffu, move)) {
                        // O is rescaled in the rows that moved; P V of the previous tile must be complete
                        ok = pt_mbar_wait(pt_smem_u32(&bars.pv_done[q]), (unsigned)((n - 1) & 1));
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            unsigned acc[32];
                            pt_ld32(o_addr + (unsigned)(c * 32), acc);
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * alpha);
                            pt_st32(o_addr + (unsigned)(c * 32), acc);
                        }
                    }
                }
                // probabilities, written back over the scores as packed bfloat16
                // (m_used is -inf only while the row has seen no key; every score is -inf then and 2^-inf = 0)
                const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
                const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(neg_m, neg_m);
                float2 sum2[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) sum2[c] = make_float2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    unsigned pk[32];
#pragma unroll
                    for (int j = 0; j < 64; j += 2) {
                        const int jj = c * 64 + j;
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[jj]), __uint_as_float(v[jj + 1])), sc2, nm2);
                        float2 p;
                        p.x = (jj % PT_POLY_EVERY == PT_POLY_EVERY - 1) ? pt_ex2_poly(x.x) : pt_ex2(x.x);
                        p.y = ((jj + 1) % PT_POLY_EVERY == PT_POLY_EVERY - 1) ? pt_ex2_poly(x.y) : pt_ex2(x.y);
                        sum2[(j >> 1) & 3] = __fadd2_rn(sum2[(j >> 1) & 3], p);
                        const __nv_bfloat162 h = __floats2bfloat162_rn(p.x, p.y);
                        pk[j >> 1] = *reinterpret_cast<const unsigned*>(&h);
                    }
                    pt_st32(s_addr + (unsigned)(c * 32), pk);
                }
                const float2 s01 = __fadd2_rn(sum2[0], sum2[1]), s23 = __fadd2_rn(sum2[2], sum2[3]);
                tile_sum = (s01.x + s01.y) + (s23.x + s23.y);
                if (with_max || !__any_sync(0xffffffffu, !(tile_sum < PT_SUM_LIMIT))) break;
                with_max = true;   // once more, relative to this tile's maximum
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            if (!ok) break;
            l += tile_sum;
            if ((t + 1) * PT_KEYS > kv_total && (q == 0 || !(t >= tile_a[0] && t < tile_b[0]))) {
                // the tile reaches past the request's last key: the lowest query tile that works on it clears
                // those value rows (both halves); the tensor core takes the tiles' products in this order
                const int u = t - lo, b = u & 1;
                ok = pt_mbar_wait(pt_smem_u32(&bars.v_full[b]), (unsigned)((u >> 1) & 1));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                unsigned char* vt = v_s + b * PT_TILE_BYTES;
                const int first = max(kv_total - t * PT_KEYS, 0);
                for (int idx = quarter * 32 + lane; idx < (PT_KEYS - first) * 16; idx += PT_ROWS) {
                    const int row = first + (idx >> 4), c16 = idx & 15;
                    *reinterpret_cast<uint4*>(vt + (c16 >> 3) * PT_HALF_BYTES + row * 128 + (c16 & 7) * 16) =
                        make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) pt_mbar_arrive(pt_smem_u32(&bars.p_ready[q]));
        }
        if (ok && my_tiles > 0) {
            ok = pt_mbar_wait(pt_smem_u32(&bars.pv_done[q]), (unsigned)((my_tiles - 1) & 1));
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) {
            if (lane == 0) { failed = 1; atomicExch(error, 13); }
        } else if (my_tiles > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = 1.f / l;
            const bool is_live = tok < my_live;
            bf16* dst = out + (size_t)(row_base + my_t0 + tok) * out_row_stride + (size_t)(hk * share + hi_) * PT_D;
            const size_t p = ((size_t)(row_base + my_t0 + tok) * H + (hk * share + hi_)) * max_splits + split;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                unsigned acc[32];
                pt_ld32(o_addr + (unsigned)(c * 32), acc);
                if (is_live && splits > 1) {
                    // one run of several: the unnormalised output and what it is relative to, for the join
                    float* po = part_o + p * PT_D + c * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(po + j) = make_float4(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]),
                                                                         __uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
                } else if (is_live) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 pk;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int q2 = 0; q2 < 4; ++q2)
                            h[q2] = __floats2bfloat162_rn(__uint_as_float(acc[j + 2 * q2]) * inv,
                                                          __uint_as_float(acc[j + 2 * q2 + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + j) = pk;
                    }
                }
            }
            if (is_live && splits > 1) {
                part_ml[2 * p] = m_used;
                part_ml[2 * p + 1] = l;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == PT_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Adds the runs of the query tiles that were cut (see pt_splits_of): grid (32 x query tiles, kv head,
// request), a block for four rows of a query tile, a warp per row, the runs in order.
__global__ void __launch_bounds__(128)
paged_prefill_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int max_splits, int sms,
                          const int* __restrict__ cu_seqlens, const int* __restrict__ kv_offsets,
                          const int* __restrict__ seq_list, bf16* __restrict__ out, int out_row_stride, int H, int Hk,
                          int share) {
    pdl_wait();
    pdl_trigger();
    const int qt = blockIdx.x >> 5, hk = blockIdx.y;
    const int seq = seq_list ? seq_list[blockIdx.z] : (int)blockIdx.z;
    const int toks_per_tile = pt_toks_per_tile(share);
    const int row_base = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - row_base;
    const int t0 = qt * toks_per_tile;
    if (t0 >= n_new) return;
    const int splits = pt_splits_of(n_new, kv_offsets[seq] + n_new, toks_per_tile, Hk, max_splits, sms);
    if (splits <= 1) return;   // written whole by the kernel above
    const int toks_live = min(toks_per_tile, n_new - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        const int r = ((int)(blockIdx.x & 31) << 2) + warp;
        const int hi = r / toks_per_tile, tok = r - hi * toks_per_tile;
        if (hi >= share || tok >= toks_live) return;
        const int row = row_base + t0 + tok, h = hk * share + hi;
        const size_t p0 = ((size_t)row * H + h) * max_splits;
        float M = -INFINITY;
        for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, part_ml[2 * (p0 + s2)]);
        float L = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s2 = 0; s2 < splits; ++s2) {
            const float m = part_ml[2 * (p0 + s2)];
            if (m == -INFINITY) continue;   // (a run without a visible key: its output was not written)
            const float wgt = exp2f(m - M);
            L += wgt * part_ml[2 * (p0 + s2) + 1];
            const float4 v = *reinterpret_cast<const float4*>(part_o + (p0 + s2) * PT_D + lane * 4);
            o.x += wgt * v.x; o.y += wgt * v.y; o.z += wgt * v.z; o.w += wgt * v.w;
        }
        const float inv = 1.f / L;
        __nv_bfloat162 a = __floats2bfloat162_rn(o.x * inv, o.y * inv), b = __floats2bfloat162_rn(o.z * inv, o.w * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<const unsigned*>(&a);
        pk.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(out + (size_t)row * out_row_stride + (size_t)h * PT_D + lane * 4) = pk;
    }
}

// ---- host side ----
typedef CUresult (*pt_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static pt_encode_fn pt_encoder() {
    static pt_encode_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (pt_encode_fn)p;
    }
    return fn;
}

// a [rows, cols] bfloat16 matrix with row stride ld (elements), read in boxes of box_rows x 64
static bool pt_make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    pt_encode_fn enc = pt_encoder();
    if (!enc) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Request i brings the token rows [cu_seqlens[i], cu_seqlens[i+1]) of q (`tokens` rows
// in all, row stride q_row_stride, query head h at columns h * 128) at positions
// kv_offsets[i] onward; pools are [pages, Hk, S, 128].  `error`: a device int a block
// sets if one of its bounded waits runs out.  With `seq_list` (device, `requests`
// entries) only the requests it names are worked on.  `max_splits` > 1 lets requests
// with few query tiles and many keys cut their key tiles into up to so many runs
// (pt_splits_of decides per request); `scratch` then holds tokens * H * max_splits *
// (D + 2) floats.
extern "C" int vx_paged_prefill_attention_tc(const void* q, int q_row_stride, int tokens, const void* k_pool,
                                             const void* v_pool, int pages, const int* block_table, int max_blocks,
                                             const int* cu_seqlens, const int* kv_offsets, const int* seq_list, void* out,
                                             int out_row_stride, float scale, int window, int requests, int max_new,
                                             int H, int Hk, int D, int S, float* scratch, int max_splits, int* error,
                                             cudaStream_t stream) {
    if (requests <= 0 || max_new <= 0 || tokens <= 0) return VX_OK;
    if (D != PT_D || H <= 0 || Hk <= 0 || H % Hk || S <= 0 || S % 16 || window < 0 || !error) return VX_ERR_SHAPE;
    const int G = H / Hk;
    if (G > 8) return VX_ERR_SHAPE;
    if ((q_row_stride & 7) || (((uintptr_t)q) & 15) || (out_row_stride & 7) || (((uintptr_t)out) & 15) ||
        ((((uintptr_t)k_pool) | ((uintptr_t)v_pool)) & 15))
        return VX_ERR_ALIGN;
    if (Hk > 65535 || requests > 65535) return VX_ERR_LIMIT;
    if (max_splits < 1 || max_splits > 64 || (max_splits > 1 && !scratch)) return VX_ERR_SHAPE;
    const int toks_per_tile = pt_toks_per_tile(G);
    CUtensorMap mq, mk, mv;
    if (!pt_make_map(&mq, q, tokens, H * D, q_row_stride, toks_per_tile) ||
        !pt_make_map(&mk, k_pool, (long long)pages * Hk * S, D, D, 16) ||
        !pt_make_map(&mv, v_pool, (long long)pages * Hk * S, D, D, 16))
        return VX_ERR_DRIVER;
    const size_t smem = 6 * (size_t)PT_TILE_BYTES + 1024;
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(paged_prefill_attention_tc_kernel, smem, configured)) return rc;
    const int q_tiles = (max_new + toks_per_tile - 1) / toks_per_tile;
    static int sm_counts[VX_MAX_DEVICES];
    const int sms = vx_sm_count(sm_counts);
    // scratch of the cut query tiles: outputs [tokens, H, max_splits, D], then (reference, sum) [tokens, H, max_splits, 2]
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)tokens * H * max_splits * D : nullptr;
    const int q_blocks = (q_tiles + PT_QTILES - 1) / PT_QTILES;
    dim3 grid(q_blocks * Hk * max_splits, 1, requests);
    VX_LAUNCH_K(VX_K_ATTENTION, paged_prefill_attention_tc_kernel, grid, PT_THREADS, smem, stream, mq, mk, mv,
                block_table, max_blocks, cu_seqlens, kv_offsets, seq_list, (bf16*)out, out_row_stride, scale * PT_LOG2E, window, H,
                Hk, S, G, part_o, part_ml, max_splits, sms, error);
    VX_LAUNCH_CHECK();
    if (max_splits > 1) {
        dim3 jgrid(q_tiles * 32, Hk, requests);
        VX_LAUNCH_K(VX_K_JOIN, paged_prefill_join_kernel, jgrid, 128, 0, stream, (const float*)part_o, (const float*)part_ml,
                    max_splits, sms, cu_seqlens, kv_offsets, seq_list, (bf16*)out, out_row_stride, H, Hk, G);
        VX_LAUNCH_CHECK();
    }
    return VX_OK;
}
