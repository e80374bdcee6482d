// Embedding lookup, residual-add + RMSNorm, plain RMSNorm, gated activation.
//
// The residual stream is float32 in both precisions of the engine: a sublayer's
// output (element type T) is added to it in float32, and the norm's statistics
// and scaling are float32; only the normed activations that feed the next
// matrix product are rounded to T.
#include "common.cuh"

// out[t, :] = table[ids[t], :] widened to float32.  An id outside [0, vocab)
// yields a row of NaN: the host checks ids before a step, and a fault in that
// check then shows in every comparison instead of reading foreign memory.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int vx_embedding(const int* ids, const void* table, float* out, int tokens, int hidden,
                            int vocab, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (hidden <= 0 || vocab <= 0) return VX_ERR_SHAPE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (embedding_kernel<float>), tokens, threads, 0, stream, ids, (const float*)table, out, hidden, vocab);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (embedding_kernel<bf16>), tokens, threads, 0, stream, ids, (const bf16*)table, out, hidden, vocab);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// One block per output row r.  Source row s = row_index ? row_index[r] : r.
//   x = residual_in[s] (+ delta[s])            float32
//   residual_out[r] = x                         (if given)
//   out[r] = x * rsqrt(mean(x^2) + eps) * w     rounded to T
template <typename T>
__global__ void add_rmsnorm_kernel(const float* __restrict__ residual_in, const T* __restrict__ delta,
                                   const int* __restrict__ row_index, float* __restrict__ residual_out,
                                   const float* __restrict__ weight, T* __restrict__ out, int width,
                                   float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int s = row_index ? row_index[r] : r;
    const float* xin = residual_in + (size_t)s * width;
    const T* din = delta ? delta + (size_t)s * width : nullptr;
    float* xout = residual_out ? residual_out + (size_t)r * width : nullptr;
    T* o = out + (size_t)r * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float x = xin[i];
        if (din) x += to_f32(din[i]);
        if (xout) xout[i] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        // This thread wrote xout[i] itself in the first loop (same indices), so
        // the re-read is ordered, and it is right when residual_out aliases
        // residual_in (the sum must not be formed twice).
        float x;
        if (xout) {
            x = xout[i];
        } else {
            x = xin[i];
            if (din) x += to_f32(din[i]);
        }
        o[i] = from_f32<T>(x * rstd * weight[i]);
    }
}

// The same with 8 elements per thread and access (width a multiple of 8, at most
// 8 * 256 * RN_MAX_ITER): the row stays in registers between the two passes.
#define RN_THREADS 256
#define RN_MAX_ITER 4

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}

template <typename T, int ITER>
__global__ void __launch_bounds__(RN_THREADS)
add_rmsnorm_vec_kernel(const float* __restrict__ residual_in, const T* __restrict__ delta,
                       const int* __restrict__ row_index, float* __restrict__ residual_out,
                       const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int chunks = width >> 3;
    // the norm's weights depend on no earlier kernel: they are asked for before the wait
    float w[ITER][8];
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
        if (c < chunks) load8(weight + c * 8, w[i]);
    }
    const int s = row_index ? row_index[r] : r;   // (the step's description: on the device before the step's first kernel)
    const float* xin = residual_in + (size_t)s * width;
    const T* din = delta ? delta + (size_t)s * width : nullptr;
    float* xout = residual_out ? residual_out + (size_t)r * width : nullptr;
    T* o = out + (size_t)r * width;
    float x[ITER][8];
    // With a delta, the delta is what the kernel before this one wrote; the residual is older
    // (the delta was computed from it) and is read before the wait.  Without one the residual
    // itself may be that kernel's output (the embedding), and everything waits.
    if (din) {
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int c = threadIdx.x + i * RN_THREADS;
            if (c < chunks) load8(xin + c * 8, x[i]);
        }
    }
    pdl_wait();
    pdl_trigger();
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
        if (c < chunks) {
            if (din) {
                float d[8];
                load8(din + c * 8, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[i][j] += d[j];
            } else {
                load8(xin + c * 8, x[i]);
            }
            if (xout) store8(xout + c * 8, x[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += x[i][j] * x[i][j];
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int c = threadIdx.x + i * RN_THREADS;
        if (c < chunks) {
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = x[i][j] * rstd * w[i][j];
            store8(o + c * 8, y);
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(const float* residual_in, const T* delta, const int* row_index, float* residual_out,
                              const float* weight, T* out, int rows, int width, float eps, cudaStream_t stream) {
    const bool aligned = !((((uintptr_t)residual_in) | ((uintptr_t)delta) | ((uintptr_t)residual_out) |
                            ((uintptr_t)weight) | ((uintptr_t)out)) & 15);
    if (width % 8 == 0 && aligned && width <= 8 * RN_THREADS * RN_MAX_ITER) {
        const int iter = (width / 8 + RN_THREADS - 1) / RN_THREADS;
        if (iter <= 1)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_vec_kernel<T, 1>), rows, RN_THREADS, 0, stream, residual_in,
                        delta, row_index, residual_out, weight, out, width, eps);
        else if (iter == 2)
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_vec_kernel<T, 2>), rows, RN_THREADS, 0, stream, residual_in,
                        delta, row_index, residual_out, weight, out, width, eps);
        else
            VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_vec_kernel<T, 4>), rows, RN_THREADS, 0, stream, residual_in,
                        delta, row_index, residual_out, weight, out, width, eps);
    } else {
        const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_kernel<T>), rows, threads, 0, stream, residual_in, delta,
                    row_index, residual_out, weight, out, width, eps);
    }
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_add_rmsnorm(const float* residual_in, const void* delta, const int* row_index,
                              float* residual_out, const float* weight, void* out, int rows,
                              int width, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0) return VX_ERR_SHAPE;
    // In place (residual_out == residual_in) is only sound without a gather.
    if (row_index && residual_out == residual_in) return VX_ERR_SHAPE;
    if (dtype == VX_F32)
        return launch_add_rmsnorm<float>(residual_in, (const float*)delta, row_index, residual_out, weight,
                                         (float*)out, rows, width, eps, stream);
    if (dtype == VX_BF16)
        return launch_add_rmsnorm<bf16>(residual_in, (const bf16*)delta, row_index, residual_out, weight,
                                        (bf16*)out, rows, width, eps, stream);
    return VX_ERR_DTYPE;
}

// Plain RMSNorm of rows of element type T (no residual), statistics in float32.
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                               T* __restrict__ out, int width, float eps) {
    pdl_wait();
    pdl_trigger();
    __shared__ float scratch[32];
    const T* xin = x + (size_t)blockIdx.x * width;
    T* o = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32(xin[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = from_f32<T>(to_f32(xin[i]) * rstd * weight[i]);
}

extern "C" int vx_rmsnorm(const void* x, const float* weight, void* out, int rows, int width,
                          float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0) return VX_ERR_SHAPE;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (rmsnorm_kernel<float>), rows, threads, 0, stream, (const float*)x, weight, (float*)out, width, eps);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (rmsnorm_kernel<bf16>), rows, threads, 0, stream, (const bf16*)x, weight, (bf16*)out, width, eps);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// out[t, i] = act(gate) * up, activation and product in float32.  Where gate i
// and up i sit in a row of 2 * inner values: with block == 0 the gate half is
// followed by the up half; with block > 0 the row is made of tiles of 2 * block
// values, `block` gates followed by their `block` ups.
template <typename T, typename TO>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, TO* __restrict__ out, long long total,
                                 int inner, int act, int block) {
    pdl_wait();
    pdl_trigger();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inner;
        const int i = (int)(idx - t * inner);
        const T* row = gate_up + t * 2 * inner;
        const int gi = block > 0 ? (i / block) * 2 * block + i % block : i;
        const int ui = block > 0 ? gi + block : inner + i;
        out[idx] = from_f32<TO>(activation(to_f32(row[gi]), act) * to_f32(row[ui]));
    }
}

// Eight features per thread: with tiles of 8 (block == 8) the gates of a tile are
// 16 contiguous bytes (bf16) followed by its ups; with halves (block == 0) eight
// gates and eight ups are contiguous each.  inner a multiple of 8, 16-byte aligned.
template <typename T, typename TO>
__global__ void gated_act_vec_kernel(const T* __restrict__ gate_up, TO* __restrict__ out, long long chunks,
                                     int inner, int act, int block) {
    pdl_wait();
    pdl_trigger();
    const int per_row = inner >> 3;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / per_row;
        const int c = (int)(idx - t * per_row);
        const T* row = gate_up + t * 2 * inner;
        float g[8], u[8], y[8];
        if (block == 8) {
            load8(row + c * 16, g);
            load8(row + c * 16 + 8, u);
        } else {
            load8(row + c * 8, g);
            load8(row + inner + c * 8, u);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = activation(g[j], act) * u[j];
        store8(out + t * inner + c * 8, y);
    }
}

template <typename T, typename TO>
static int launch_gated_act(const void* gate_up, void* out, bool vec, long long blocks, int threads, long long items,
                            long long total, int inner, int act, int block, cudaStream_t stream) {
    if (vec)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_act_vec_kernel<T, TO>), (int)blocks, threads, 0, stream, (const T*)gate_up,
                    (TO*)out, items, inner, act, block);
    else
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_act_kernel<T, TO>), (int)blocks, threads, 0, stream, (const T*)gate_up,
                    (TO*)out, total, inner, act, block);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// act(gate) * up of rows [gates | ups] (block == 0) or tiles of `block` gates and their
// ups.  The input may be float32 with a bfloat16 result: a library product then hands
// over its float32 sums and nothing is rounded before the activation.
extern "C" int vx_gated_act(const void* gate_up, void* out, int rows, int inner, int act, int block, int dtype,
                            int out_dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (inner <= 0 || act < 0 || act > 3 || block < 0 || (block > 0 && inner % block)) return VX_ERR_SHAPE;
    const long long total = (long long)rows * inner;
    const int threads = 256;
    const bool vec = inner % 8 == 0 && (block == 0 || block == 8) &&
                     !((((uintptr_t)gate_up) | ((uintptr_t)out)) & 15);
    const long long items = vec ? total / 8 : total;
    long long blocks = (items + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == VX_F32 && out_dtype == VX_F32)
        return launch_gated_act<float, float>(gate_up, out, vec, blocks, threads, items, total, inner, act, block, stream);
    if (dtype == VX_BF16 && out_dtype == VX_BF16)
        return launch_gated_act<bf16, bf16>(gate_up, out, vec, blocks, threads, items, total, inner, act, block, stream);
    if (dtype == VX_F32 && out_dtype == VX_BF16)
        return launch_gated_act<float, bf16>(gate_up, out, vec, blocks, threads, items, total, inner, act, block, stream);
    return VX_ERR_DTYPE;
}

// out[m, n] = in[m, n] + bias[n], float32 in, float32 or bfloat16 out: the bias of a
// library product is added to its float32 sums, and the result rounded once.
template <typename TO>
__global__ void add_bias_kernel(const float* __restrict__ in, const float* __restrict__ bias, TO* __restrict__ out,
                                long long total, int n) {
    pdl_wait();
    pdl_trigger();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x)
        out[idx] = from_f32<TO>(in[idx] + bias[idx % n]);
}

extern "C" int vx_add_bias(const float* in, const float* bias, void* out, int rows, int n, int out_dtype,
                           cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return VX_OK;
    const long long total = (long long)rows * n;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_bias_kernel<float>), (int)blocks, 256, 0, stream, in, bias, (float*)out, total, n);
    else if (out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_bias_kernel<bf16>), (int)blocks, 256, 0, stream, in, bias, (bf16*)out, total, n);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
