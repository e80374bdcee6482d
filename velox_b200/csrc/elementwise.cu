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
    pdl_trigger();
    pdl_wait();
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
    pdl_trigger();
    pdl_wait();
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

extern "C" int vx_add_rmsnorm(const float* residual_in, const void* delta, const int* row_index,
                              float* residual_out, const float* weight, void* out, int rows,
                              int width, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0) return VX_ERR_SHAPE;
    // In place (residual_out == residual_in) is only sound without a gather.
    if (row_index && residual_out == residual_in) return VX_ERR_SHAPE;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_kernel<float>), rows, threads, 0, stream, residual_in, (const float*)delta, row_index, residual_out, weight, (float*)out, width, eps);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (add_rmsnorm_kernel<bf16>), rows, threads, 0, stream, residual_in, (const bf16*)delta, row_index, residual_out, weight, (bf16*)out, width, eps);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// Plain RMSNorm of rows of element type T (no residual), statistics in float32.
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ weight,
                               T* __restrict__ out, int width, float eps) {
    pdl_trigger();
    pdl_wait();
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
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total,
                                 int inner, int act, int block) {
    pdl_trigger();
    pdl_wait();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inner;
        const int i = (int)(idx - t * inner);
        const T* row = gate_up + t * 2 * inner;
        const int gi = block > 0 ? (i / block) * 2 * block + i % block : i;
        const int ui = block > 0 ? gi + block : inner + i;
        out[idx] = from_f32<T>(activation(to_f32(row[gi]), act) * to_f32(row[ui]));
    }
}

extern "C" int vx_gated_act(const void* gate_up, void* out, int rows, int inner, int act, int block, int dtype,
                            cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (inner <= 0 || act < 0 || act > 3 || block < 0 || (block > 0 && inner % block)) return VX_ERR_SHAPE;
    const long long total = (long long)rows * inner;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_act_kernel<float>), (int)blocks, threads, 0, stream, (const float*)gate_up, (float*)out, total, inner, act, block);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (gated_act_kernel<bf16>), (int)blocks, threads, 0, stream, (const bf16*)gate_up, (bf16*)out, total, inner, act, block);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
