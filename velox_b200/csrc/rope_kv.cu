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

// The arithmetic of a head of 128 written out with explicit roundings, so that the
// two kernels below give the same bits whatever the compiler would like to fuse.
__device__ __forceinline__ float head128_squares(float2 lo, float2 hi) {
    return __fmaf_rn(hi.y, hi.y, __fmaf_rn(hi.x, hi.x, __fmaf_rn(lo.y, lo.y, __fmul_rn(lo.x, lo.x))));
}
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& ra, float& rb) {
    ra = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
    rb = __fmaf_rn(a, sn, __fmul_rn(b, cs));
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
    constexpr int D = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * ROPE128_WARPS + warp;
    // What depends on no earlier kernel is fetched before the wait: the norm's weights, the
    // frequencies, and the step's description (copied to the device before the step's first kernel).
    const bool in_range = head < H + 2 * Hk;
    const bool is_q = head < H;
    const float* w = is_q ? q_weight : k_weight;
    float2 wl = make_float2(1.f, 1.f), wh = wl, f = make_float2(0.f, 0.f);
    float pos = 0.f;
    int slot = -1;
    if (in_range) {
        slot = slot_mapping ? slot_mapping[t] : -1;
        if (head < H + Hk) {
            if (w) { wl = reinterpret_cast<const float2*>(w)[lane]; wh = reinterpret_cast<const float2*>(w + 64)[lane]; }
            if (inv_freq) { f = reinterpret_cast<const float2*>(inv_freq)[lane]; pos = (float)positions[t]; }
        }
    }
    pdl_wait();
    pdl_trigger();
    if (!in_range) return;
    bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    if (head >= H + Hk) {  // value head: copy into the cache (8 bytes per lane)
        if (slot < 0) return;
        const int hk = head - H - Hk;
        bf16* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
        return;
    }
    if (!is_q && slot_mapping && slot < 0) return;
    float2 lo = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
    float2 hi = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
    if (w) {
        const float ss = warp_sum(head128_squares(lo, hi));
        const float rstd = rsqrtf(ss / (float)D + eps);
        lo.x = __fmul_rn(__fmul_rn(lo.x, rstd), wl.x); lo.y = __fmul_rn(__fmul_rn(lo.y, rstd), wl.y);
        hi.x = __fmul_rn(__fmul_rn(hi.x, rstd), wh.x); hi.y = __fmul_rn(__fmul_rn(hi.y, rstd), wh.y);
    }
    if (inv_freq) {
        float sn, cs, a0, b0, a1, b1;
        sincosf(__fmul_rn(pos, f.x), &sn, &cs);
        rotate_pair(lo.x, hi.x, cs, sn, a0, b0);
        sincosf(__fmul_rn(pos, f.y), &sn, &cs);
        rotate_pair(lo.y, hi.y, cs, sn, a1, b1);
        lo = make_float2(a0, a1);
        hi = make_float2(b0, b1);
    }
    bf16* dst = src;
    if (!is_q && slot_mapping)
        dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
    reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(lo.x, lo.y);
    reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(hi.x, hi.y);
}

// The same for many tokens (a prompt portion): one block per token works through
// all heads of its row, eight warps taking the heads in turn, with the token's 64
// cosines and sines computed once into shared memory instead of once per head
// (40 or more heads share them; the sincosf calls were most of the kernel's time).
#define ROPE128_TOKEN_MIN 64   // tokens from which this variant is used
__global__ void __launch_bounds__(ROPE128_WARPS * 32)
qk_norm_rope_kv_128_row_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                               const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                               const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                               bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int H, int Hk, int S) {
    pdl_wait();
    pdl_trigger();
    constexpr int D = 128;
    __shared__ float2 cs_sn[D / 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    if (inv_freq && threadIdx.x < D / 2) {
        float sn, cs;
        sincosf(__fmul_rn((float)positions[t], inv_freq[threadIdx.x]), &sn, &cs);
        cs_sn[threadIdx.x] = make_float2(cs, sn);
    }
    __syncthreads();
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    for (int head = warp; head < H + 2 * Hk; head += ROPE128_WARPS) {
        bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
        if (head >= H + Hk) {  // value head: copy into the cache (8 bytes per lane)
            if (slot < 0) continue;
            const int hk = head - H - Hk;
            bf16* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
            reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
            continue;
        }
        const bool is_q = head < H;
        if (!is_q && slot_mapping && slot < 0) continue;
        const float* w = is_q ? q_weight : k_weight;
        float2 lo = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
        float2 hi = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
        if (w) {
            const float ss = warp_sum(head128_squares(lo, hi));
            const float rstd = rsqrtf(ss / (float)D + eps);
            const float2 wl = reinterpret_cast<const float2*>(w)[lane], wh = reinterpret_cast<const float2*>(w + 64)[lane];
            lo.x = __fmul_rn(__fmul_rn(lo.x, rstd), wl.x); lo.y = __fmul_rn(__fmul_rn(lo.y, rstd), wl.y);
            hi.x = __fmul_rn(__fmul_rn(hi.x, rstd), wh.x); hi.y = __fmul_rn(__fmul_rn(hi.y, rstd), wh.y);
        }
        if (inv_freq) {
            const float2 c0 = cs_sn[2 * lane], c1 = cs_sn[2 * lane + 1];
            float a0, b0, a1, b1;
            rotate_pair(lo.x, hi.x, c0.x, c0.y, a0, b0);
            rotate_pair(lo.y, hi.y, c1.x, c1.y, a1, b1);
            lo = make_float2(a0, a1);
            hi = make_float2(b0, b1);
        }
        bf16* dst = src;
        if (!is_q && slot_mapping)
            dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
        reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(lo.x, lo.y);
        reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(hi.x, hi.y);
    }
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
        if (tokens >= ROPE128_TOKEN_MIN) {
            VX_LAUNCH_K(VX_K_ROPE, qk_norm_rope_kv_128_row_kernel, tokens, ROPE128_WARPS * 32, 0, stream, (bf16*)qkv,
                        row_stride, q_weight, k_weight, eps, (rot_dim == D) ? inv_freq : (const float*)nullptr,
                        positions, slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, Hk, S);
            VX_LAUNCH_CHECK();
            return VX_OK;
        }
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
