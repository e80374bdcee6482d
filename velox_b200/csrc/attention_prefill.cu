// Paged causal attention for prompt portions, bfloat16, on the tensor cores.
//
// grid (query tile, kv head, request); 8 warps.  A block takes 128 query rows of one
// request: 128 / G consecutive new tokens times the G query heads of one kv head
// (so the heads of a group share each key/value tile; 128 tokens of one head when G
// is no power of two), 16 rows per warp, kept in registers as tensor-core A
// operands, and walks over the request's keys in tiles of 64: the keys that earlier steps left in the pages, then the portion's own
// keys up to the diagonal.  K and V tiles are gathered page by page with cp.async
// into double-buffered shared memory ([64 keys][D], 16-byte chunks XOR-swizzled so
// that ldmatrix reads hit distinct banks) and shared by the eight warps.  Each warp
// forms S = Q K^T for a tile's 64 keys with mma.sync.m16n8k16 (bf16 in, float32
// out), masks (causal: key <= the row's position; window: key >= position + 1 - W;
// by select, so a never-written slot cannot leak), keeps running maximum and sum
// per row in float32 (online softmax, base 2) and adds P V into float32
// accumulators.  Rows past the request's new tokens are computed and not stored.
//
// A request that brings one token (a decoded token in a mixed step) is a tile with
// one live row: correct, and cheap enough beside the prompt portions it rides with.
//
// Sizes: head size 64 or 128; page size a multiple of 16 that divides 64 or is a
// multiple of 64; any head counts with H % Hk == 0; an optional window.  Other
// sizes are refused (the caller then uses the general kernel).
#include "common.cuh"
#include "mma_helpers.cuh"

#define PF_WARPS 4
#define PF_BM 64
#define PF_BN 64
#define PF_LOG2E 1.4426950408889634f

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32)
paged_prefill_attention_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pool,
                               const bf16* __restrict__ v_pool, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ cu_seqlens,
                               const int* __restrict__ kv_offsets, const int* __restrict__ seq_list,
                               bf16* __restrict__ out, int out_row_stride,
                               float scale_log2, int window, int H, int Hk, int S, int share_log2) {
    extern __shared__ __align__(128) unsigned char pf_smem[];
    constexpr int CHUNKS_PER_ROW = D / 8;
    constexpr int TILE_BYTES = PF_BN * D * 2;
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the longest tiles (the last tokens of a prompt) are handed out first
    // (the list of requests is part of the step's description, copied before the step's kernels)
    const int qt = gridDim.x - 1 - blockIdx.x, seq = seq_list ? seq_list[blockIdx.z] : (int)blockIdx.z;
    const int share = 1 << share_log2;                  // query heads of one kv head that share this tile
    const int toks_per_tile = PF_BM >> share_log2;
    const int row_base = cu_seqlens[seq];
    const int n_new = cu_seqlens[seq + 1] - row_base;
    const int t0 = qt * toks_per_tile;                  // first new token of the tile
    if (t0 >= n_new) return;
    const int off = kv_offsets[seq];
    // with sharing, blockIdx.y is the kv head and row r is (token r / share, head hk * share + r % share);
    // without, blockIdx.y is the query head
    const int hk = share > 1 ? blockIdx.y : blockIdx.y / (H / Hk);
    const int head0 = share > 1 ? hk * share : blockIdx.y;
    const int* bt = block_table + (size_t)seq * max_blocks;
    const int toks_live = min(toks_per_tile, n_new - t0);
    const int kv_hi = off + t0 + toks_live;             // one past the last visible key of the tile
    const int kv_lo = window > 0 ? max(0, off + t0 + 1 - window) : 0;
    const int tile_lo = kv_lo / PF_BN, tile_hi = (kv_hi + PF_BN - 1) / PF_BN;

    unsigned char* q_s = pf_smem;                        // [128][D], swizzled
    unsigned char* kv_s = pf_smem + PF_BM * D * 2;       // 2 stages x (K tile, V tile)

    // ---- queries into shared memory, then into registers ----
    for (int c = threadIdx.x; c < PF_BM * CHUNKS_PER_ROW; c += PF_WARPS * 32) {
        const int r = c / CHUNKS_PER_ROW, cc = c % CHUNKS_PER_ROW;
        const int tr = min(t0 + (r >> share_log2), n_new - 1);   // rows past the end repeat the last token
        const int hd = head0 + (r & (share - 1));
        cp_async16(q_s + r * (D * 2) + ((cc ^ (r & 7)) << 4),
                   q + (size_t)(row_base + tr) * q_row_stride + (size_t)hd * D + cc * 8);
    }
    cp_async_commit();

    auto issue = [&](int tile, int stage) {
        unsigned char* ks = kv_s + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* vs = ks + TILE_BYTES;
        for (int c = threadIdx.x; c < PF_BN * CHUNKS_PER_ROW; c += PF_WARPS * 32) {
            const int r = c / CHUNKS_PER_ROW, cc = c % CHUNKS_PER_ROW;
            int key = tile * PF_BN + r;
            // Slots outside [kv_lo, kv_hi) repeat the nearest key inside: they are masked
            // anyway, and a page below a window may already have been given back.
            key = max(min(key, kv_hi - 1), kv_lo);
            const int page = bt[key / S];
            const size_t src = (((size_t)page * Hk + hk) * S + (key % S)) * D + cc * 8;
            const int dst = r * (D * 2) + ((cc ^ (r & 7)) << 4);
            cp_async16(ks + dst, k_pool + src);
            cp_async16(vs + dst, v_pool + src);
        }
    };
    issue(tile_lo, 0);
    cp_async_commit();

    cp_async_wait<1>();   // the queries have landed (the first K/V tile may still be on its way)
    __syncthreads();
    unsigned qf[D / 16][4];
    {
        // A fragment of rows warp*16 .. +15: matrices (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        const int mi = lane >> 3;
        const int r = warp * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int cc = 2 * kk + (mi >> 1);
            ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], q_s + r * (D * 2) + ((cc ^ (r & 7)) << 4));
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // absolute positions of the two rows this thread holds, and of the warp's rows
    const int r0 = warp * 16 + (lane >> 2);
    const int pos0 = off + t0 + (r0 >> share_log2), pos1 = off + t0 + ((r0 + 8) >> share_log2);
    const int lo0 = window > 0 ? pos0 + 1 - window : 0, lo1 = window > 0 ? pos1 + 1 - window : 0;
    const int warp_hi = off + t0 + ((warp * 16 + 15) >> share_log2) + 1;   // one past the warp's last position
    const int warp_lo = window > 0 ? off + t0 + ((warp * 16) >> share_log2) + 1 - window : 0;

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        if (tile + 1 < tile_hi) issue(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* ks = kv_s + (size_t)stage * 2 * TILE_BYTES;
        const unsigned char* vs = ks + TILE_BYTES;
        const int key_base = tile * PF_BN;
        if (key_base < warp_hi && key_base + PF_BN > warp_lo) {   // warp-uniform: some key of the tile is visible
            // S = Q K^T for the tile's 64 keys, 16 at a time; groups no row of the warp sees are skipped
            float sc[PF_BN / 16][2][4];
            bool vis[PF_BN / 16];
#pragma unroll
            for (int kg = 0; kg < PF_BN / 16; ++kg) {
                const int key0 = key_base + kg * 16;
                vis[kg] = key0 < warp_hi && key0 + 16 > warp_lo;
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[kg][0][c] = sc[kg][1][c] = 0.f;
            }
            if (vis[0] && vis[1] && vis[2] && vis[3]) {
                // the common tile, wholly visible to the warp: k steps outermost, so that the
                // eight accumulators of a step are independent and their multiply-accumulates overlap
                const int mi = lane >> 3;
                const int rr = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int cc = 2 * kk + (mi & 1);
#pragma unroll
                    for (int kg = 0; kg < PF_BN / 16; ++kg) {
                        const int r = kg * 16 + rr;
                        unsigned b00, b01, b10, b11;
                        ldmatrix_x4(b00, b01, b10, b11, ks + r * (D * 2) + ((cc ^ (r & 7)) << 4));
                        mma_bf16(sc[kg][0], qf[kk], b00, b01);
                        mma_bf16(sc[kg][1], qf[kk], b10, b11);
                    }
                }
            } else {
                // a tile on the diagonal or at a window's edge: group by group, skipping the hidden ones
                const int mi = lane >> 3;
                const int rr = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
                for (int kg = 0; kg < PF_BN / 16; ++kg) {
                    if (!vis[kg]) continue;
                    const int r = kg * 16 + rr;
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const int cc = 2 * kk + (mi & 1);
                        unsigned b00, b01, b10, b11;
                        ldmatrix_x4(b00, b01, b10, b11, ks + r * (D * 2) + ((cc ^ (r & 7)) << 4));
                        mma_bf16(sc[kg][0], qf[kk], b00, b01);
                        mma_bf16(sc[kg][1], qf[kk], b10, b11);
                    }
                }
            }
            // scale, mask, one softmax update for the whole tile
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int pos = hrow ? pos1 : pos0, lo = hrow ? lo1 : lo0;
                float mx = -INFINITY;
#pragma unroll
                for (int kg = 0; kg < PF_BN / 16; ++kg)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int key = key_base + kg * 16 + nt * 8 + ((lane & 3) << 1) + c;
                            const bool ok = vis[kg] && key <= pos && key >= lo;
                            float& v = sc[kg][nt][2 * hrow + c];
                            v = ok ? v * scale_log2 : -INFINITY;
                            mx = fmaxf(mx, v);
                        }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[hrow], mx);
                const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m[hrow] - m_new);
                float ps = 0.f;
#pragma unroll
                for (int kg = 0; kg < PF_BN / 16; ++kg)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            float& v = sc[kg][nt][2 * hrow + c];
                            v = (m_new == -INFINITY) ? 0.f : exp2f(v - m_new);
                            ps += v;
                        }
                l[hrow] = l[hrow] * alpha + ps;
                m[hrow] = m_new;
#pragma unroll
                for (int i2 = 0; i2 < D / 8; ++i2) {
                    o[i2][2 * hrow] *= alpha;
                    o[i2][2 * hrow + 1] *= alpha;
                }
            }
            // O += P V
#pragma unroll
            for (int kg = 0; kg < PF_BN / 16; ++kg) {
                if (!vis[kg]) continue;
                unsigned pa[4];
                pa[0] = pack_bf16(sc[kg][0][0], sc[kg][0][1]);
                pa[1] = pack_bf16(sc[kg][0][2], sc[kg][0][3]);
                pa[2] = pack_bf16(sc[kg][1][0], sc[kg][1][1]);
                pa[3] = pack_bf16(sc[kg][1][2], sc[kg][1][3]);
                const int mi = lane >> 3;
                const int r = kg * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int nt = 0; nt < D / 8; nt += 2) {
                    const int cc = nt + (mi >> 1);
                    unsigned v00, v01, v10, v11;
                    ldmatrix_x4_trans(v00, v01, v10, v11, vs + r * (D * 2) + ((cc ^ (r & 7)) << 4));
                    mma_bf16(o[nt], pa, v00, v01);
                    mma_bf16(o[nt + 1], pa, v10, v11);
                }
            }
        }
        __syncthreads();   // every warp is done with this stage before it is filled again
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 1);
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 2);
        const int r = r0 + 8 * hrow;
        const int tok = r >> share_log2;
        if (tok >= toks_live) continue;
        const int hd = head0 + (r & (share - 1));
        const float inv = 1.f / l[hrow];
        bf16* dst = out + (size_t)(row_base + t0 + tok) * out_row_stride + (size_t)hd * D + ((lane & 3) << 1);
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                __floats2bfloat162_rn(o[nt][2 * hrow] * inv, o[nt][2 * hrow + 1] * inv);
    }
}

template <int D>
static int launch_prefill(const bf16* q, int q_row_stride, const bf16* k_pool, const bf16* v_pool,
                          const int* block_table, int max_blocks, const int* cu_seqlens, const int* kv_offsets,
                          const int* seq_list, bf16* out, int out_row_stride, float scale, int window, int requests,
                          int max_new, int H, int Hk, int S, cudaStream_t stream) {
    const size_t smem = (size_t)PF_BM * D * 2 + 2 * 2 * (size_t)PF_BN * D * 2;
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(paged_prefill_attention_kernel<D>, smem, configured)) return rc;
    // Query heads of one kv head share a tile (and so its key/value traffic) when
    // their number is a power of two up to 16; otherwise every head has its own tiles.
    const int G = H / Hk;
    int share_log2 = 0;
    if (G > 1 && G <= 16 && (G & (G - 1)) == 0)
        while ((1 << share_log2) < G) ++share_log2;
    const int toks_per_tile = PF_BM >> share_log2;
    dim3 grid((max_new + toks_per_tile - 1) / toks_per_tile, share_log2 ? Hk : H, requests);
    VX_LAUNCH_K(VX_K_ATTENTION, (paged_prefill_attention_kernel<D>), grid, PF_WARPS * 32, smem, stream, q,
                q_row_stride, k_pool, v_pool, block_table, max_blocks, cu_seqlens, kv_offsets, seq_list, out,
                out_row_stride, scale * PF_LOG2E, window, H, Hk, S, share_log2);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// Request i brings the token rows [cu_seqlens[i], cu_seqlens[i+1]) at positions
// kv_offsets[i], kv_offsets[i] + 1, ...; its keys and values (these new ones
// included) are in the pools.  `max_new` bounds the tokens of any request.  With
// `seq_list` (device, `requests` entries) only the requests it names are worked on:
// a mixed step gives its single decoded tokens to the decode kernel instead.
extern "C" int vx_paged_prefill_attention(const void* q, int q_row_stride, const void* k_pool,
                                          const void* v_pool, const int* block_table, int max_blocks,
                                          const int* cu_seqlens, const int* kv_offsets, const int* seq_list, void* out,
                                          int out_row_stride, float scale, int window, int requests,
                                          int max_new, int H, int Hk, int D, int S, cudaStream_t stream) {
    if (requests <= 0 || max_new <= 0) return VX_OK;
    if (H <= 0 || Hk <= 0 || H % Hk || S <= 0 || S % 16 || window < 0) return VX_ERR_SHAPE;
    if (H > 65535 || requests > 65535) return VX_ERR_LIMIT;
    if ((q_row_stride & 7) || (((uintptr_t)q) & 15) || (out_row_stride & 1) || (((uintptr_t)out) & 3))
        return VX_ERR_ALIGN;
    if (D == 128)
        return launch_prefill<128>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                                   block_table, max_blocks, cu_seqlens, kv_offsets, seq_list, (bf16*)out, out_row_stride,
                                   scale, window, requests, max_new, H, Hk, S, stream);
    if (D == 64)
        return launch_prefill<64>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                                  block_table, max_blocks, cu_seqlens, kv_offsets, seq_list, (bf16*)out, out_row_stride,
                                  scale, window, requests, max_new, H, Hk, S, stream);
    return VX_ERR_SHAPE;
}
