// Per-head RMSNorm of queries and keys, rotary position encoding, and the write
// of the new keys and values into the paged cache, in one pass over the packed
// projection output.
//
// qkv is [tokens, row_stride] with, in each row, H query heads, then Hk key
// heads, then Hk value heads, each of D elements.  One warp handles one head of
// one token:
//   q, k:  x = x * rsqrt(mean(x^2) + eps) * w[d]          (if a weight is given)
//          pairs (i, i + rot/2), i < rot/2, rotated by angle = pos * inv_freq[i]
//          (half-split convention; angle, sine and cosine in float32, computed
//          here rather than read from a table rounded to the element type)
//   q is written back in place; k goes to k_pool, v (untouched) to v_pool at
//   slot_mapping[token] = page * S + offset, pools laid out [page, Hk, S, D].
// A token whose slot is negative writes nothing.  Without a slot mapping (a layer
// that reads another layer's cache, or a caller that encodes positions itself)
// nothing is written to the pools and the keys are normed and rotated in place.
#include "common.cuh"

#define ROPE_WARPS 4
#define ROPE_MAX_D 512

template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, int row_stride,
                                       const float* __restrict__ q_weight,
                                       const float* __restrict__ k_weight, float eps,
                                       const float* __restrict__ inv_freq, int rot_dim,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ slot_mapping, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, int H, int Hk, int D, int S) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * ROPE_WARPS + warp;
    if (head >= H + 2 * Hk) return;
    float* buf = smem + warp * D;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    const int slot = slot_mapping ? slot_mapping[t] : -1;

    if (head >= H + Hk) {  // value head: copy into the cache
        if (slot < 0) return;
        const int hk = head - H - Hk;
        T* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        for (int d = lane; d < D; d += 32) dst[d] = src[d];
        return;
    }
    const bool is_q = head < H;
    if (!is_q && slot_mapping && slot < 0) return;
    const float* w = is_q ? q_weight : k_weight;

    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float x = to_f32(src[d]);
        buf[d] = x;
        ss += x * x;
    }
    if (w) {
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) buf[d] = buf[d] * rstd * w[d];
    }
    __syncwarp();
    if (inv_freq && rot_dim > 0) {
        const int half = rot_dim >> 1;
        const float pos = (float)positions[t];
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            const float a = buf[i], b = buf[i + half];
            buf[i] = a * cs - b * sn;
            buf[i + half] = a * sn + b * cs;
        }
        __syncwarp();
    }
    if (is_q || !slot_mapping) {  // without a slot mapping keys are treated in place too
        for (int d = lane; d < D; d += 32) src[d] = from_f32<T>(buf[d]);
    } else {
        const int hk = head - H;
        T* dst = k_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(buf[d]);
    }
}

// The same for bfloat16 heads of 128 with full rotation, the whole head in
// registers: lane l holds elements 2l, 2l+1 (first half) and 64+2l, 64+2l+1 (their
// partners), loaded and stored as pairs.  Eight warps, one head each.
#define ROPE128_WARPS 8
__global__ void __launch_bounds__(ROPE128_WARPS * 32)
qk_norm_rope_kv_128_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                           const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                           const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                           bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int H, int Hk, int S) {
    pdl_wait();
    pdl_trigger();
    constexpr int D = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * ROPE128_WARPS + warp;
    if (head >= H + 2 * Hk) return;
    bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if (head >= H + Hk) {  // value head: copy into the cache (8 bytes per lane)
        if (slot < 0) return;
        const int hk = head - H - Hk;
        bf16* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
        return;
    }
    const bool is_q = head < H;
    if (!is_q && slot_mapping && slot < 0) return;
    const float* w = is_q ? q_weight : k_weight;
    float2 lo = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
    float2 hi = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
    if (w) {
        const float ss = warp_sum(lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y);
        const float rstd = rsqrtf(ss / (float)D + eps);
        const float2 wl = reinterpret_cast<const float2*>(w)[lane], wh = reinterpret_cast<const float2*>(w + 64)[lane];
        lo.x = lo.x * rstd * wl.x; lo.y = lo.y * rstd * wl.y;
        hi.x = hi.x * rstd * wh.x; hi.y = hi.y * rstd * wh.y;
    }
    if (inv_freq) {
        const float pos = (float)positions[t];
        const float2 f = reinterpret_cast<const float2*>(inv_freq)[lane];
        float sn, cs;
        sincosf(pos * f.x, &sn, &cs);
        const float a0 = lo.x * cs - hi.x * sn, b0 = lo.x * sn + hi.x * cs;
        sincosf(pos * f.y, &sn, &cs);
        const float a1 = lo.y * cs - hi.y * sn, b1 = lo.y * sn + hi.y * cs;
        lo = make_float2(a0, a1);
        hi = make_float2(b0, b1);
    }
    bf16* dst = src;
    if (!is_q && slot_mapping)
        dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
    reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(lo.x, lo.y);
    reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(hi.x, hi.y);
}

extern "C" int vx_qk_norm_rope_kv(void* qkv, int row_stride, const float* q_weight,
                                  const float* k_weight, float eps, const float* inv_freq,
                                  int rot_dim, const int* positions, const int* slot_mapping,
                                  void* k_pool, void* v_pool, int tokens, int H, int Hk, int D, int S,
                                  int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (H <= 0 || Hk <= 0 || D <= 0 || S <= 0 || D > ROPE_MAX_D) return VX_ERR_SHAPE;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1)) return VX_ERR_SHAPE;
    if (row_stride < (H + 2 * Hk) * D) return VX_ERR_SHAPE;
    if (slot_mapping && (!k_pool || !v_pool)) return VX_ERR_SHAPE;
    if (dtype == VX_BF16 && D == 128 && (rot_dim == D || !inv_freq) && !(row_stride & 3) &&
        !((((uintptr_t)qkv) | ((uintptr_t)k_pool) | ((uintptr_t)v_pool)) & 7)) {
        dim3 grid128(tokens, (H + 2 * Hk + ROPE128_WARPS - 1) / ROPE128_WARPS);
        VX_LAUNCH_K(VX_K_ROPE, qk_norm_rope_kv_128_kernel, grid128, ROPE128_WARPS * 32, 0, stream, (bf16*)qkv,
                    row_stride, q_weight, k_weight, eps, (rot_dim == D) ? inv_freq : (const float*)nullptr, positions,
                    slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, Hk, S);
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    dim3 grid(tokens, (H + 2 * Hk + ROPE_WARPS - 1) / ROPE_WARPS);
    const size_t smem = (size_t)ROPE_WARPS * D * sizeof(float);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_kernel<float>), grid, ROPE_WARPS * 32, smem, stream, (float*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
            (float*)k_pool, (float*)v_pool, H, Hk, D, S);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_kernel<bf16>), grid, ROPE_WARPS * 32, smem, stream, (bf16*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
            (bf16*)k_pool, (bf16*)v_pool, H, Hk, D, S);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
