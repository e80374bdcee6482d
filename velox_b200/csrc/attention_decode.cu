// Paged attention for decoded tokens (one query per request), bfloat16, with the
// key/value range of a request split into pieces of fixed size that are worked on
// independently and joined by a second, small kernel.
//
// The unit of work is a WARP: it takes `piece_tiles` tiles of 16 keys of one kv
// head of one request and ALL the query heads of that kv head (the group), so
// every key and value is read from memory once; the group's queries fill the rows
// of one 16-row tensor-core tile.  The warp streams its tiles through a cp.async
// pipeline of its own in shared memory (no barrier between warps anywhere in the
// kernel), computes S = Q K^T and O += P V with mma.sync.m16n8k16 (bf16 in,
// float32 out) and keeps a running maximum, sum and accumulator per query row in
// float32 (online softmax, base 2).  A request whose whole range is one piece gets
// its output written at once; otherwise each warp writes its unnormalised
// accumulator and (max, sum) to scratch, and the join kernel (one block per
// request and head) adds the pieces in piece order.
//
// Piece boundaries depend only on the request's own key range (fixed number of
// keys per piece), never on the batch, so a request's output does not depend on
// what else is in the step.
//
// How the pieces are spread over blocks changes nothing in what a warp computes, so
// it is chosen per launch.  The pieces of the step are numbered (request, kv head,
// piece); a block of W warps takes W consecutive numbers.  What bounds the kernel is
// how many tiles are in flight against the memory's latency, so the shapes are made
// to fill the SMs' shared memory:
//   - up to 4 pieces per SM: blocks of 4 warps with 6 stages (5 tiles in flight per
//     warp), one block an SM (batch 8 at 1,900 keys: a step of 6 layers 0.770
//     instead of 0.819 ms with 3 stages);
//   - up to 5 or 6 pieces per SM: one wave of blocks of 5 warps with 5 stages or 6
//     warps with 4, so that every SM holds the same number of pieces, give or take
//     one (batch 5 and 6 at 4,000 keys: 2 and 3 % faster steps);
//   - more: blocks of 4 warps with 3 stages, two blocks an SM.  One wave of 7 warps
//     with 4 stages (224 KB, which leaves no room on the SM for a block of the
//     kernel before or after) made a step at batch 8 and 4,000 keys 14 % slower.
//
// Launched programmatically (see common.cuh) a warp asks for its first tiles before it
// waits for the kernel before it, unless they reach the request's newest position: the
// only thing that kernel may write into the pools is the key and value at position
// kv_len - 1 of each request (which is what writing the step's new tokens does).
//
// Sizes: head size 64 or 128; page size a multiple of 16; group size up to 16;
// any number of heads; an optional window.  Other sizes are refused (the caller
// then uses the general kernel).
#include "common.cuh"
#include "mma_helpers.cuh"

#define LOG2E 1.4426950408889634f

// Shared memory of a block: per warp, DEC_STAGES (3 to 6) stages of a K tile and a V tile
// [16 keys][D] bf16, 16-byte chunks of a row XOR-swizzled with the row index so
// that ldmatrix reads hit distinct banks.
template <int D, int DEC_STAGES, int DEC_WARPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_attention_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pool,
                              const bf16* __restrict__ v_pool, const int* __restrict__ block_table,
                              int max_blocks, const int* __restrict__ token_rows,
                              const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                              float* __restrict__ part_o, float* __restrict__ part_ml, int max_pieces,
                              bf16* __restrict__ out, int out_row_stride, float scale_log2, int window,
                              int H, int Hk, int S, int piece_tiles, int requests, int early_ok) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = 16 * D * 2;
    constexpr int CHUNKS_PER_ROW = D / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int number = (int)blockIdx.x * DEC_WARPS + warp, per_request = Hk * max_pieces;
    if (number >= requests * per_request) return;  // (no barrier follows: a warp may leave alone)
    const int b = number / per_request, hk = (number % per_request) / max_pieces, piece = number % max_pieces;
    const int G = H / Hk;
    // The step's description was copied to the device before any kernel of the
    // step ran, so it may be read before the wait on earlier kernels.
    const int row_tok = token_rows ? token_rows[b] : b;
    const int seq = seq_of_token[row_tok];
    const int kv_len = positions[row_tok] + 1;
    const int start = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int tile_first = start >> 4;
    const int tile_last = (kv_len + 15) >> 4;  // exclusive
    // (a caller whose max_pieces is too small for this request loses keys, but nothing is
    // read or written outside the scratch)
    const int npieces = min((tile_last - tile_first + piece_tiles - 1) / piece_tiles, max_pieces);
    if (piece >= npieces) return;
    const int tile_begin = tile_first + piece * piece_tiles;
    const int count = min(piece_tiles, tile_last - tile_begin);
    const int* bt = block_table + (size_t)seq * max_blocks;
    // lane j holds the page of the warp's j-th tile
    int my_page = 0;
    if (lane < count) my_page = bt[((tile_begin + lane) << 4) / S];

    unsigned char* my_smem = smem_raw + (size_t)warp * DEC_STAGES * 2 * TILE_BYTES;
    // The tiles asked for first hold keys and values of earlier steps, unless they reach the
    // request's newest position (which the kernel before this one has just written, or is
    // still writing): only then do they have to wait for that kernel.
    // (`early_ok` is 0 when a request brings several tokens in this step: then the kernel before this
    // one has written more than the newest position, and nothing is asked for before the wait)
    const bool early = early_ok && ((tile_begin + DEC_STAGES - 1) << 4) <= kv_len - 1;

    auto issue = [&](int j) {
        const int key0 = (tile_begin + j) << 4;
        const int page = __shfl_sync(0xffffffffu, my_page, j);
        const size_t base = (((size_t)page * Hk + hk) * S + (key0 % S)) * D;
        unsigned char* ks = my_smem + (size_t)(j % DEC_STAGES) * 2 * TILE_BYTES;
        unsigned char* vs = ks + TILE_BYTES;
        const unsigned char* kg = reinterpret_cast<const unsigned char*>(k_pool + base);
        const unsigned char* vg = reinterpret_cast<const unsigned char*>(v_pool + base);
#pragma unroll
        for (int i = 0; i < (16 * CHUNKS_PER_ROW) / 32; ++i) {
            const int c = lane + 32 * i;
            const int r = c / CHUNKS_PER_ROW, cc = c % CHUNKS_PER_ROW;
            const int dst = r * (D * 2) + ((cc ^ (r & 7)) << 4);
            cp_async16(ks + dst, kg + (size_t)c * 16);
            cp_async16(vs + dst, vg + (size_t)c * 16);
        }
    };
    if (early) {
#pragma unroll
        for (int s = 0; s < DEC_STAGES - 1; ++s) {
            if (s < count) issue(s);
            cp_async_commit();
        }
    }
    pdl_wait();
    pdl_trigger();
    if (!early) {
#pragma unroll
        for (int s = 0; s < DEC_STAGES - 1; ++s) {
            if (s < count) issue(s);
            cp_async_commit();
        }
    }

    // queries of the group: rows of the A operand, kept in registers
    unsigned qf[D / 16][4];
    {
        const int r0 = lane >> 2, r1 = r0 + 8;
        const bf16* q0 = q + (size_t)row_tok * q_row_stride + (size_t)(hk * G + r0) * D;
        const bf16* q1 = q + (size_t)row_tok * q_row_stride + (size_t)(hk * G + r1) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int c = kk * 16 + (lane & 3) * 2;
            qf[kk][0] = r0 < G ? *reinterpret_cast<const unsigned*>(q0 + c) : 0u;
            qf[kk][1] = r1 < G ? *reinterpret_cast<const unsigned*>(q1 + c) : 0u;
            qf[kk][2] = r0 < G ? *reinterpret_cast<const unsigned*>(q0 + c + 8) : 0u;
            qf[kk][3] = r1 < G ? *reinterpret_cast<const unsigned*>(q1 + c + 8) : 0u;
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < count; ++i) {
        if (i + DEC_STAGES - 1 < count) issue(i + DEC_STAGES - 1);
        cp_async_commit();
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const int key0 = (tile_begin + i) << 4;
        unsigned char* ks = my_smem + (size_t)(i % DEC_STAGES) * 2 * TILE_BYTES;
        unsigned char* vs = ks + TILE_BYTES;
        if (key0 + 16 > kv_len) {
            // Rows past the last key were never written (they may hold anything,
            // NaN included): their probabilities are zero, but 0 * NaN is NaN in
            // the tensor core, so the value rows are cleared.
            for (int c = lane; c < 16 * CHUNKS_PER_ROW; c += 32) {
                const int r = c / CHUNKS_PER_ROW;
                if (key0 + r >= kv_len) *reinterpret_cast<uint4*>(vs + (size_t)c * 16) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // S = Q K^T for 16 keys: two n-tiles of 8 keys
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int mi = lane >> 3;
            const int r = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int cc = 2 * kk + (mi & 1);
                unsigned b00, b01, b10, b11;
                ldmatrix_x4(b00, b01, b10, b11, ks + r * (D * 2) + ((cc ^ (r & 7)) << 4));
                mma_bf16(s0, qf[kk], b00, b01);
                mma_bf16(s1, qf[kk], b10, b11);
            }
        }
        // scale, mask, online softmax (base 2).  Thread holds rows lane/4 and
        // lane/4 + 8, key columns (lane%4)*2 + {0,1} of each n-tile.
        const int kc = key0 + ((lane & 3) << 1);
        float sv[2][4];  // [row half][n-tile 0: 2 cols, n-tile 1: 2 cols]
        sv[0][0] = s0[0]; sv[0][1] = s0[1]; sv[0][2] = s1[0]; sv[0][3] = s1[1];
        sv[1][0] = s0[2]; sv[1][1] = s0[3]; sv[1][2] = s1[2]; sv[1][3] = s1[3];
        unsigned pa[4];
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = kc + (c & 1) + ((c >> 1) << 3);
                const bool ok = key >= start && key < kv_len;
                sv[hrow][c] = ok ? sv[hrow][c] * scale_log2 : -INFINITY;
                mx = fmaxf(mx, sv[hrow][c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[hrow], mx);
            // a row with no visible key so far keeps m = -inf; exp2f(-inf - (-inf)) must not be formed
            const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m[hrow] - m_new);
            float ps = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = (m_new == -INFINITY) ? 0.f : exp2f(sv[hrow][c] - m_new);
                sv[hrow][c] = p;
                ps += p;
            }
            l[hrow] = l[hrow] * alpha + ps;
            m[hrow] = m_new;
#pragma unroll
            for (int i2 = 0; i2 < D / 8; ++i2) {
                o[i2][2 * hrow] *= alpha;
                o[i2][2 * hrow + 1] *= alpha;
            }
        }
        pa[0] = pack_bf16(sv[0][0], sv[0][1]);
        pa[1] = pack_bf16(sv[1][0], sv[1][1]);
        pa[2] = pack_bf16(sv[0][2], sv[0][3]);
        pa[3] = pack_bf16(sv[1][2], sv[1][3]);
        // O += P V
        {
            const int mi = lane >> 3;
            const int r = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
            for (int nt = 0; nt < D / 8; nt += 2) {
                const int cc = nt + (mi >> 1);
                unsigned v00, v01, v10, v11;
                ldmatrix_x4_trans(v00, v01, v10, v11, vs + r * (D * 2) + ((cc ^ (r & 7)) << 4));
                mma_bf16(o[nt], pa, v00, v01);
                mma_bf16(o[nt + 1], pa, v10, v11);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // row sums: add the four threads of a quad
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 1);
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 2);
    }
    // thread holds rows lane/4 (+8), columns nt*8 + (lane%4)*2 + {0,1}
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        const int g = (lane >> 2) + 8 * hrow;
        if (g >= G) continue;
        const int h = hk * G + g;
        if (npieces == 1) {
            const float inv = 1.f / l[hrow];
            bf16* dst = out + (size_t)row_tok * out_row_stride + (size_t)h * D + ((lane & 3) << 1);
#pragma unroll
            for (int nt = 0; nt < D / 8; ++nt)
                *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                    __floats2bfloat162_rn(o[nt][2 * hrow] * inv, o[nt][2 * hrow + 1] * inv);
        } else {
            const size_t p = ((size_t)b * H + h) * max_pieces + piece;
            float* dst = part_o + p * D + ((lane & 3) << 1);
#pragma unroll
            for (int nt = 0; nt < D / 8; ++nt)
                *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * hrow], o[nt][2 * hrow + 1]);
            if ((lane & 3) == 0) *reinterpret_cast<float2*>(part_ml + p * 2) = make_float2(m[hrow], l[hrow]);
        }
    }
}

// Joins the pieces of requests that have several: one block per (request, head),
// pieces added in piece order.
#define JOIN_MAX_PIECES 1024
#define JOIN_EARLY 16   // pieces whose values a thread asks for before it knows their weights
template <int D>
__global__ void paged_decode_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         int max_pieces, const int* __restrict__ token_rows,
                                         const int* __restrict__ positions, bf16* __restrict__ out,
                                         int out_row_stride, int window, int H, int piece_tiles) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int row_tok = token_rows ? token_rows[b] : b;
    const int kv_len = positions[row_tok] + 1;
    const int start = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int ntiles = ((kv_len + 15) >> 4) - (start >> 4);
    const int npieces = min((ntiles + piece_tiles - 1) / piece_tiles, max_pieces);
    pdl_wait();  // on every path: a grid that ends without waiting would let its successor run ahead of its predecessor
    pdl_trigger();
    if (npieces <= 1) return;  // written by the first pass
    const size_t p0 = ((size_t)b * H + h) * max_pieces;
    // this thread's element of the first pieces is on its way while the weights are formed
    const int d0 = threadIdx.x;
    float first[JOIN_EARLY];
#pragma unroll
    for (int u = 0; u < JOIN_EARLY; ++u)
        first[u] = (d0 < D && u < npieces) ? part_o[(p0 + u) * D + d0] : 0.f;
    // weights of the pieces, once per block: w_s = 2^(m_s - M), and L = sum w_s l_s
    // in piece order (so the result does not depend on the number of threads)
    __shared__ float wgt[JOIN_MAX_PIECES];
    __shared__ float inv_l;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float M = -INFINITY;
        for (int s = lane; s < npieces; s += 32) M = fmaxf(M, part_ml[(p0 + s) * 2]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        for (int s = lane; s < npieces; s += 32) {
            const float ms = part_ml[(p0 + s) * 2];
            wgt[s] = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
        }
        __syncwarp();
        if (lane == 0) {
            float L = 0.f;
            for (int s = 0; s < npieces; ++s) L += wgt[s] * part_ml[(p0 + s) * 2 + 1];
            inv_l = 1.f / L;
        }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float* po = part_o + p0 * D + d;
        float O = 0.f;
        int s = 0;
        if (d == d0) {  // (always, for a block as wide as the head)
#pragma unroll
            for (int u = 0; u < JOIN_EARLY; ++u)
                if (u < npieces) O += wgt[u] * first[u];
            s = min(npieces, JOIN_EARLY);
        }
        for (; s + 8 <= npieces; s += 8) {  // eight independent loads at a time, added in piece order
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = po[(size_t)(s + u) * D];
#pragma unroll
            for (int u = 0; u < 8; ++u) O += wgt[s + u] * v[u];
        }
        for (; s < npieces; ++s) O += wgt[s] * po[(size_t)s * D];
        out[(size_t)row_tok * out_row_stride + (size_t)h * D + d] = __float2bfloat16_rn(O * inv_l);
    }
}

// Scratch a launch needs, in floats: accumulators [requests, H, max_pieces, D] then
// (max, sum) [requests, H, max_pieces, 2].  Every element is written before it is
// read; nothing needs clearing.
extern "C" long long vx_paged_decode_scratch_floats(int requests, int H, int D, int max_pieces) {
    return (long long)requests * H * max_pieces * (D + 2);
}

static int dec_sm_count() {
    static int sms[VX_MAX_DEVICES];
    return vx_sm_count(sms);
}

template <int D, int STAGES, int WARPS>
static int launch_decode_pieces(int blocks, const bf16* q, int q_row_stride, const bf16* k_pool, const bf16* v_pool,
                                const int* block_table, int max_blocks, const int* token_rows,
                                const int* seq_of_token, const int* positions, float* part_o, float* part_ml,
                                int max_pieces, bf16* out, int out_row_stride, float scale, int window, int requests,
                                int H, int Hk, int S, int piece_tiles, int early_ok, cudaStream_t stream) {
    const size_t smem = (size_t)WARPS * STAGES * 2 * 16 * D * 2;
    VX_LAUNCH_K(VX_K_ATTENTION, (paged_decode_attention_kernel<D, STAGES, WARPS>), dim3(blocks), WARPS * 32, smem, stream,
                q, q_row_stride, k_pool, v_pool, block_table, max_blocks, token_rows, seq_of_token, positions, part_o,
                part_ml, max_pieces, out, out_row_stride, scale * LOG2E, window, H, Hk, S, piece_tiles, requests, early_ok);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

template <int D, int STAGES, int WARPS>
static cudaError_t configure_decode_pieces() {
    return cudaFuncSetAttribute(paged_decode_attention_kernel<D, STAGES, WARPS>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * STAGES * 2 * 16 * D * 2);
}

// All four shapes of a head size at its first call on a device (the attribute belongs
// to a device's copy of the function), whichever shape that call needs: a later call
// may come from inside a stream capture with a step of another size.  First calls are
// not made from several host threads at once.
template <int D>
static int configure_decode() {
    static bool configured[VX_MAX_DEVICES];
    const int dev = vx_current_device();
    if (dev < 0) return VX_ERR_LIMIT;
    if (configured[dev]) return VX_OK;
    cudaError_t e = configure_decode_pieces<D, 6, 4>();
    if (e == cudaSuccess) e = configure_decode_pieces<D, 3, 4>();
    if (e == cudaSuccess) e = configure_decode_pieces<D, 5, 5>();
    if (e == cudaSuccess) e = configure_decode_pieces<D, 4, 6>();
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
    return VX_OK;
}

template <int D>
static int launch_decode(const bf16* q, int q_row_stride, const bf16* k_pool, const bf16* v_pool,
                         const int* block_table, int max_blocks, const int* token_rows,
                         const int* seq_of_token, const int* positions, float* scratch, int max_pieces,
                         bf16* out, int out_row_stride, float scale, int window, int requests, int H, int Hk,
                         int S, int piece_tiles, int early_ok, cudaStream_t stream) {
    const int ready = configure_decode<D>();
    if (ready != VX_OK) return ready;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)requests * H * max_pieces * D : nullptr;
    const long long pieces = (long long)requests * Hk * max_pieces, sms = dec_sm_count();
    int warps = 4, stages = 3;
    if (pieces <= 4 * sms) stages = 6;
    else if (pieces <= 5 * sms) warps = 5, stages = 5;
    else if (pieces <= 6 * sms) warps = 6, stages = 4;
    const int blocks = (int)((pieces + warps - 1) / warps);
#define DEC_LAUNCH(ST, W)                                                                                            \
    launch_decode_pieces<D, ST, W>(blocks, q, q_row_stride, k_pool, v_pool, block_table, max_blocks, token_rows,       \
                                   seq_of_token, positions, part_o, part_ml, max_pieces, out, out_row_stride, scale, \
                                   window, requests, H, Hk, S, piece_tiles, early_ok, stream)
    int rc;
    if (warps == 5) rc = DEC_LAUNCH(5, 5);
    else if (warps == 6) rc = DEC_LAUNCH(4, 6);
    else rc = stages == 6 ? DEC_LAUNCH(6, 4) : DEC_LAUNCH(3, 4);
#undef DEC_LAUNCH
    if (rc != VX_OK) return rc;
    if (max_pieces > 1) {
        dim3 jgrid(requests, H);
        VX_LAUNCH_K(VX_K_JOIN, (paged_decode_join_kernel<D>), jgrid, D <= 64 ? 64 : 128, 0, stream, part_o, part_ml, max_pieces,
                  token_rows, positions, out, out_row_stride, window, H, piece_tiles);
        VX_LAUNCH_CHECK();
    }
    return VX_OK;
}

// One query token per entry.  `token_rows[i]` is the token row (in q, out,
// seq_of_token, positions) of entry i, or null when entry i is row i; several
// entries may be tokens of one request (a short prompt portion, token by token).
// `early_ok`: every entry is its request's only new token of this step (then a warp
// may ask for keys and values of earlier positions before the kernel before it ends).
// `max_pieces` bounds the pieces of any request: ceil(ceil(max keys / 16) / piece_tiles)
// (one more with a window that does not start on a tile's edge); `scratch` holds
// vx_paged_decode_scratch_floats(...) floats (may be null when max_pieces is 1).
extern "C" int vx_paged_decode_attention(const void* q, int q_row_stride, const void* k_pool,
                                         const void* v_pool, const int* block_table, int max_blocks,
                                         const int* token_rows, const int* seq_of_token,
                                         const int* positions, float* scratch, int max_pieces, void* out,
                                         int out_row_stride, float scale, int window, int requests, int H,
                                         int Hk, int D, int S, int piece_tiles, int early_ok, cudaStream_t stream) {
    if (requests <= 0) return VX_OK;
    if (H <= 0 || Hk <= 0 || H % Hk || H / Hk > 16 || S <= 0 || S % 16 || window < 0) return VX_ERR_SHAPE;
    if (piece_tiles <= 0 || piece_tiles > 32 || max_pieces <= 0 || (max_pieces > 1 && !scratch)) return VX_ERR_SHAPE;
    if (Hk > 65535 || requests > 65535 || max_pieces > JOIN_MAX_PIECES) return VX_ERR_LIMIT;
    if ((long long)requests * Hk * max_pieces > (1ll << 30)) return VX_ERR_LIMIT;   // pieces are numbered in an int
    if ((q_row_stride & 1) || (((uintptr_t)q) & 3) || (out_row_stride & 1) || (((uintptr_t)out) & 3)) return VX_ERR_ALIGN;
    if (D == 128)
        return launch_decode<128>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                                  block_table, max_blocks, token_rows, seq_of_token, positions, scratch,
                                  max_pieces, (bf16*)out, out_row_stride, scale, window, requests, H, Hk, S,
                                  piece_tiles, early_ok, stream);
    if (D == 64)
        return launch_decode<64>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                                 block_table, max_blocks, token_rows, seq_of_token, positions, scratch,
                                 max_pieces, (bf16*)out, out_row_stride, scale, window, requests, H, Hk, S,
                                 piece_tiles, early_ok, stream);
    return VX_ERR_SHAPE;
}

// ----------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in no_alloc.h).
#include "no_alloc.h"

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol lookup, never a device address: the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_static_scratch[VX_DECODE_STATIC_SCRATCH_FLOATS];

static float* g_decode_static_ptr[VX_MAX_DEVICES];  // device address of the array, per device

extern "C" long long vx_paged_decode_static_max_floats(void) { return VX_DECODE_STATIC_SCRATCH_FLOATS; }

extern "C" int vx_paged_decode_attention_static(const void* q, int q_row_stride, const void* k_pool,
                                                const void* v_pool, const int* block_table, int max_blocks,
                                                const int* token_rows, const int* seq_of_token,
                                                const int* positions, int max_splits, void* out,
                                                int out_row_stride, float scale, int window, int requests,
                                                int H, int Hk, int D, int S, int chunk_tiles,
                                                cudaStream_t stream) {
    if (requests <= 0) return VX_OK;
    if (H <= 0 || D <= 0 || max_splits <= 0) return VX_ERR_SHAPE;
    if (vx_paged_decode_scratch_floats(requests, H, D, max_splits) > (long long)VX_DECODE_STATIC_SCRATCH_FLOATS)
        return VX_ERR_LIMIT;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= VX_MAX_DEVICES) return VX_ERR_LIMIT;
    if (!g_decode_static_ptr[dev]) {
        // set-up, once per device, with that device current
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return VX_ERR_ALIGN;
        g_decode_static_ptr[dev] = p;
    }
    // The kernel before this one in the stream is the caller's, not this library's: it may
    // write what these kernels read ahead of their wait on it when launched programmatically
    // (the step's description, keys and values of earlier positions).  So: plain stream order.
    vx_pdl_suppress(1);
    const int rc = vx_paged_decode_attention(q, q_row_stride, k_pool, v_pool, block_table, max_blocks, token_rows,
                                             seq_of_token, positions, g_decode_static_ptr[dev], max_splits, out,
                                             out_row_stride, scale, window, requests, H, Hk, D, S, chunk_tiles, 1, stream);
    vx_pdl_suppress(0);
    return rc;
}
