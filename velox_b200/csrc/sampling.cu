// Token sampling from float32 logits: greedy, temperature, temperature + top-p.
//
// One block per row.  For row r with temperature T, nucleus mass P and a
// uniform number u in [0,1) that the host drew for this (request, step):
//   T <= 1e-7:  the argmax, the lowest index winning ties.
//   otherwise:  e_i = exp((x_i - max) / T);  with 0 < P < 1 only the most likely
//               tokens stay whose mass reaches P (the one that crosses P and
//               its ties included), found by bisecting the threshold on e over
//               float bit patterns;  the token is the first index, in index
//               order, whose cumulative kept mass exceeds u times the kept total.
// All arithmetic is float32 and the order of additions is fixed, so the same
// logits and u give the same token on every run.
#include "common.cuh"
#include <limits.h>

#define SAMPLE_THREADS 1024

__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    v = lane < nwarps ? sv[lane] : -INFINITY;
    idx = lane < nwarps ? si[lane] : INT_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

__device__ __forceinline__ int block_min_int(int v, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) si[warp] = v;
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    v = lane < nwarps ? si[lane] : INT_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float scan[SAMPLE_THREADS];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)r * ld;

    float best = -INFINITY;
    int best_i = INT_MAX;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }  // ascending i: the first maximum stays
    }
    block_argmax(best, best_i, sv, si);
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 1e-7f)) {
        if (tid == 0) out[r] = best_i;
        return;
    }
    const float inv_t = 1.f / temp;
    const float xmax = best;

    // contiguous chunk of this thread, for the ordered scan
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo_i = min(tid * chunk, V), hi_i = min(lo_i + chunk, V);

    float z = 0.f;
    for (int i = lo_i; i < hi_i; ++i) z += expf((x[i] - xmax) * inv_t);
    const float Z = block_sum(z, sv);

    float threshold = 0.f;
    const float P = top_p ? top_p[r] : 1.f;
    if (P > 0.f && P < 1.f) {
        const float target = P * Z;
        unsigned lo = 0u, hi = __float_as_uint(1.0f) + 1u;  // f(lo) >= target, f(hi) < target
        while (hi - lo > 1u) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            const float th = __uint_as_float(mid);
            float f = 0.f;
            for (int i = lo_i; i < hi_i; ++i) {
                const float e = expf((x[i] - xmax) * inv_t);
                if (e >= th) f += e;
            }
            f = block_sum(f, sv);
            if (f >= target) lo = mid; else hi = mid;
        }
        threshold = __uint_as_float(lo);
    }

    // kept mass of this thread's chunk, then an inclusive scan over threads
    float mine = 0.f;
    int last_kept = -1;
    for (int i = lo_i; i < hi_i; ++i) {
        const float e = expf((x[i] - xmax) * inv_t);
        if (e >= threshold) { mine += e; last_kept = i; }
    }
    __syncthreads();
    scan[tid] = mine;
    __syncthreads();
    for (int off = 1; off < SAMPLE_THREADS; off <<= 1) {
        const float add = tid >= off ? scan[tid - off] : 0.f;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
    }
    const float incl = scan[tid];
    const float excl = incl - mine;
    const float total = scan[SAMPLE_THREADS - 1];
    const float target = uniform[r] * total;

    int cand = INT_MAX;
    if (incl > target && last_kept >= 0) {
        float run = excl;
        cand = last_kept;
        for (int i = lo_i; i < hi_i; ++i) {
            const float e = expf((x[i] - xmax) * inv_t);
            if (e >= threshold) {
                run += e;
                if (run > target) { cand = i; break; }
            }
        }
    }
    cand = block_min_int(cand, si);
    if (cand == INT_MAX) {  // rounding left nobody above the target: the last kept token
        const int neg = block_min_int(last_kept >= 0 ? -last_kept : INT_MAX, si);
        cand = neg == INT_MAX ? best_i : -neg;
    }
    if (tid == 0) out[r] = cand;
}

extern "C" int vx_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                         const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (vocab <= 0 || ld < vocab) return VX_ERR_SHAPE;
    if (temperature && !uniform) return VX_ERR_SHAPE;
    VX_LAUNCH_K(VX_K_SAMPLE, (sample_kernel), rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, top_p, uniform, out);
    VX_LAUNCH_CHECK();
    return VX_OK;
}
