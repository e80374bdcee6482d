// Paged causal attention, the general kernel: any head size up to 256, any
// number of heads and groups, any page size, an optional
// window, element type float or bfloat16.  It serves prompt portions and decoded
// tokens alike, and it is the whole of the 32-bit path.
//
// One block per (token, query head).  The token's absolute position p gives its
// keys: j in [start, p], start = max(0, p + 1 - window) with a window, else 0.
// Key j of the token's request lies in page block_table[seq, j / S] at offset
// j % S; pools are [page, Hk, S, D]; query head h reads kv head h / (H / Hk).
//
// Each warp takes chunks of 32 keys (chunk c goes to warp c mod 4), one key per
// lane: the lane forms the whole dot product q.k in float32, the warp keeps a
// running maximum m, sum l and accumulator acc (online softmax), and adds the
// 32 values in key order.  The four warps' (m, l, acc) are merged in warp
// order.  The order of every addition depends only on the token's own key
// range, never on the batch around it, so a position's output is bit-identical
// however the tokens were cut into steps.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_pool,
    const T* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions, T* __restrict__ out,
    int out_row_stride, float scale, int window, int H, int Hk, int D, int S) {
    pdl_wait();
    pdl_trigger();
    __shared__ float q_s[ATT_MAX_D];
    __shared__ float acc_s[ATT_WARPS][ATT_MAX_D];
    __shared__ float m_s[ATT_WARPS], l_s[ATT_WARPS];

    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hk = h / (H / Hk);
    const int seq = seq_of_token[t];
    const int kv_len = positions[t] + 1;
    const int start = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int* bt = block_table + (size_t)seq * max_blocks;

    for (int d = threadIdx.x; d < D; d += blockDim.x)
        q_s[d] = to_f32(q[(size_t)t * q_row_stride + (size_t)h * D + d]);
    __syncthreads();

    constexpr int NR = ATT_MAX_D / 32;
    float acc[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int nkeys = kv_len - start;
    const int nchunks = (nkeys + 31) >> 5;
    for (int c = warp; c < nchunks; c += ATT_WARPS) {
        const int j = start + c * 32 + lane;
        const bool valid = j < kv_len;
        size_t base = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / S];
            base = (((size_t)page * Hk + hk) * S + (j % S)) * D;
            const T* kp = k_pool + base;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += q_s[d] * to_f32(kp[d]);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);  // m = -inf on the first chunk: 0
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[i] *= alpha;
        const int nvalid = min(32, kv_len - (start + c * 32));
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, jj);
            const T* vp = v_pool + bj;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] += pj * to_f32(vp[d]);
            }
        }
        m = m_new;
    }

    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc_s[warp][d] = acc[i];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f;
    float wgt[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; ++w) {
        wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - M);
        L += l_s[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w][d] * wgt[w];
        out[(size_t)t * out_row_stride + (size_t)h * D + d] = from_f32<T>(o / L);
    }
}

extern "C" int vx_paged_attention_generic(const void* q, int q_row_stride, const void* k_pool,
                                          const void* v_pool, const int* block_table, int max_blocks,
                                          const int* seq_of_token, const int* positions, void* out,
                                          int out_row_stride, float scale, int window, int tokens,
                                          int H, int Hk, int D, int S, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (H <= 0 || Hk <= 0 || H % Hk || D <= 0 || D > ATT_MAX_D || S <= 0 || max_blocks <= 0)
        return VX_ERR_SHAPE;
    if (window < 0) return VX_ERR_SHAPE;
    dim3 grid(tokens, H);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ATTENTION, (paged_attention_generic_kernel<float>), grid, ATT_WARPS * 32, 0, stream, (const float*)q, q_row_stride, (const float*)k_pool, (const float*)v_pool, block_table,
            max_blocks, seq_of_token, positions, (float*)out, out_row_stride, scale, window, H, Hk, D, S);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ATTENTION, (paged_attention_generic_kernel<bf16>), grid, ATT_WARPS * 32, 0, stream, (const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table,
            max_blocks, seq_of_token, positions, (bf16*)out, out_row_stride, scale, window, H, Hk, D, S);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
