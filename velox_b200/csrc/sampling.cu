// Token sampling from float32 logits: greedy, temperature, temperature + top-p.
//
// One block per row.  For row r with temperature T, nucleus mass P and a
// uniform number u in [0,1) that the host drew for this (request, step):
//   T <= 1e-7:  the argmax, the lowest index winning ties.
//   otherwise:  e_i = 2^((x_i - max) log2(e) / T);  with 0 < P < 1 only the most
//               likely tokens stay whose mass reaches P (the one that crosses P and
//               its ties included): the kept tokens are those with e_i >= the largest
//               float t whose mass {e >= t} still reaches P times the whole;  the token
//               is the first index, in index order, whose cumulative kept mass
//               exceeds u times the kept total.
// Every pass over the row reads it with consecutive lanes on consecutive elements.
// The threshold t is found ten bits a pass: a histogram, over the next ten bits of
// the patterns of e (positive floats order like their patterns), of the mass in each
// bin, as exact integers so that the order of the additions does not matter, then a
// scan from the top for the bin in which the mass crosses.  Three passes fix all
// thirty bits in which floats of (0, 1] can differ.  (A search of the pattern bit by
// bit, one pass a bit, took 1.1 ms a row at a vocabulary of 151,936.)
// The same logits and u give the same token on every run.
#include "common.cuh"
#include <limits.h>

#define SAMPLE_THREADS 1024
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
#define SAMPLE_BINS 1024
#define SAMPLE_GROUPS 256  // groups of 32 elements per warp: rows of up to 2^18 elements
static_assert(SAMPLE_BINS == SAMPLE_THREADS, "the scan below gives every thread one bin");

__device__ __forceinline__ float sample_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// f(index, value) for every element of the row, each thread its share in ascending
// index order.  Sixteen elements a thread are asked for before the first is used
// (four 16-byte loads when the row allows it): one SM has to pull the whole row, and
// with one load in flight per thread a pass over 151,936 logits took 43 us.
template <typename F>
__device__ __forceinline__ void row_for_each(const float* __restrict__ x, int V, F f) {
    const int tid = threadIdx.x;
    if ((((uintptr_t)x) & 15) == 0) {
        const int n4 = V >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int j0 = tid; j0 < n4; j0 += SAMPLE_THREADS * 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * SAMPLE_THREADS;
                if (j < n4) v[u] = x4[j];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * SAMPLE_THREADS;
                if (j < n4) {
                    f(4 * j, v[u].x);
                    f(4 * j + 1, v[u].y);
                    f(4 * j + 2, v[u].z);
                    f(4 * j + 3, v[u].w);
                }
            }
        }
        for (int i = (n4 << 2) + tid; i < V; i += SAMPLE_THREADS) f(i, x[i]);
    } else {
        for (int i0 = tid; i0 < V; i0 += SAMPLE_THREADS * 4) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * SAMPLE_THREADS;
                if (i < V) v[u] = x[i];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * SAMPLE_THREADS;
                if (i < V) f(i, v[u]);
            }
        }
    }
}

// the lanes' values added up in lane order: lane l gets v_0 + ... + v_l
__device__ __forceinline__ float warp_scan(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
    }
    return v;
}

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
    v = lane < SAMPLE_WARPS ? sv[lane] : -INFINITY;
    idx = lane < SAMPLE_WARPS ? si[lane] : INT_MAX;
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
    v = lane < SAMPLE_WARPS ? si[lane] : INT_MAX;
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
    __shared__ unsigned hist_lo[SAMPLE_BINS], hist_hi[SAMPLE_BINS];
    __shared__ unsigned long long warp_total[SAMPLE_WARPS];
    __shared__ unsigned long long above_s;
    __shared__ int first_s;
    __shared__ float warp_mass[SAMPLE_WARPS];
    __shared__ float group_mass[SAMPLE_WARPS][SAMPLE_GROUPS];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * ld;

    float best = -INFINITY;
    int best_i = INT_MAX;
    row_for_each(x, V, [&](int i, float v) {
        if (v > best) { best = v; best_i = i; }  // ascending i: the first maximum stays
    });
    block_argmax(best, best_i, sv, si);
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 1e-7f)) {
        if (tid == 0) out[r] = best_i;
        return;
    }
    const float k = 1.4426950408889634f / temp;  // e_i = 2^((x_i - max) k)
    const float xmax = best;

    float threshold = 0.f;
    const float P = top_p ? top_p[r] : 1.f;
    if (P > 0.f && P < 1.f) {
        unsigned prefix = 0u;             // the bits of the threshold's pattern found so far
        unsigned long long above = 0ull;  // mass of the patterns above the bins still in question
        unsigned long long target = 0ull;
        for (int shift = 20; shift >= 0; shift -= 10) {
            hist_lo[tid] = 0u;
            hist_hi[tid] = 0u;
            if (tid == 0) first_s = SAMPLE_THREADS;
            __syncthreads();
            // All elements of a bin have the same exponent, so a bin's mass is the sum of
            // their 24-bit mantissas times a power of two; the mantissas' low and high 12
            // bits are summed apart, each sum below 2^30 (64-bit atomics in shared memory
            // are a compare-and-swap loop: the same pass took 70 us with them, 18 us so).
            row_for_each(x, V, [&](int, float v) {
                const unsigned pat = __float_as_uint(sample_ex2((v - xmax) * k));
                if (pat != 0u && (pat >> (shift + 10)) == prefix) {
                    const unsigned bin = (pat >> shift) & (SAMPLE_BINS - 1);
                    const unsigned m = (pat & 0x7FFFFFu) | 0x800000u;
                    atomicAdd(&hist_lo[bin], m & 0xFFFu);
                    atomicAdd(&hist_hi[bin], m >> 12);
                }
            });
            __syncthreads();
            // thread t looks at bin 1023 - t: its mass in fixed point (2^40 for 1.0) ...
            const unsigned bin_of_thread = SAMPLE_BINS - 1 - tid;
            const int exponent = (int)(((((prefix << 10) | bin_of_thread) << shift) >> 23) & 0xFFu);
            unsigned long long s = ((unsigned long long)hist_hi[bin_of_thread] << 12) + hist_lo[bin_of_thread];
            s = exponent >= 110 ? s << (exponent - 110) : (110 - exponent < 64 ? s >> (110 - exponent) : 0ull);
            // ... and with it the mass of all bins above it
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xffffffffu, s, o);
                if (lane >= o) s += up;
            }
            if (lane == 31) warp_total[warp] = s;
            __syncthreads();
            for (int w = 0; w < warp; ++w) s += warp_total[w];
            if (shift == 20) {  // the first pass has seen the whole row: the nucleus' target
                if (tid == SAMPLE_THREADS - 1) above_s = s;
                __syncthreads();
                target = (unsigned long long)((double)P * (double)above_s);
                __syncthreads();
            }
            // the highest bin with which the mass reaches the target
            if (above + s >= target) atomicMin(&first_s, tid);
            __syncthreads();
            // (if rounding left the target above everything, the lowest bin: everything is kept)
            const int chosen = first_s < SAMPLE_THREADS ? first_s : SAMPLE_THREADS - 1;
            if (tid == max(chosen - 1, 0)) above_s = chosen == 0 ? above : above + s;
            __syncthreads();
            above = above_s;
            prefix = (prefix << 10) | (unsigned)(SAMPLE_BINS - 1 - chosen);
            __syncthreads();
        }
        threshold = __uint_as_float(prefix);
    }

    // Kept mass, then the token.  The warps' stretches of the row follow each other in index
    // order; a stretch is walked in groups of 32 consecutive elements, one a lane, and the
    // kept mass of every group is noted, so that the walk for the token only has to look
    // at the groups' masses and then at one group.
    const int groups = ((V + SAMPLE_WARPS - 1) / SAMPLE_WARPS + 31) >> 5;   // per warp; at most SAMPLE_GROUPS
    const int w0 = min(warp * groups * 32, V), w1 = min(w0 + groups * 32, V);
    float* gm = group_mass[warp];
    int last_kept = -1;
    for (int g0 = 0; g0 < groups; g0 += 4) {
        float xv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = w0 + (g0 + u) * 32 + lane;
            xv[u] = (g0 + u < groups && i < w1) ? x[i] : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (g0 + u >= groups) break;
            float e = sample_ex2((xv[u] - xmax) * k);   // (nothing there: 2^-inf = 0)
            if (!(e >= threshold) || xv[u] == -INFINITY) e = 0.f;
            const unsigned kept = __ballot_sync(0xffffffffu, e > 0.f);
            if (kept) last_kept = w0 + (g0 + u) * 32 + 31 - __clz(kept);
            const float incl = warp_scan(e, lane);
            if (lane == 31) gm[g0 + u] = incl;
        }
    }
    __syncwarp();
    float mine = 0.f;   // the groups' masses added up in group order
    for (int c = 0; c < groups; c += 32) mine += __shfl_sync(0xffffffffu, warp_scan(c + lane < groups ? gm[c + lane] : 0.f, lane), 31);
    __syncthreads();
    if (lane == 0) warp_mass[warp] = mine;
    __syncthreads();
    float excl = 0.f, total = 0.f;
    for (int w = 0; w < SAMPLE_WARPS; ++w) {  // in warp order, the same in every thread
        if (w == warp) excl = total;
        total += warp_mass[w];
    }
    const float target = uniform[r] * total;

    int cand = INT_MAX;
    if (excl + mine > target) {
        // the token lies in this warp's stretch or before it: the first group whose mass crosses ...
        float run = excl;
        int group = -1;
        for (int c = 0; c < groups && group < 0; c += 32) {
            const float incl = warp_scan(c + lane < groups ? gm[c + lane] : 0.f, lane);
            const unsigned hit = __ballot_sync(0xffffffffu, run + incl > target);
            if (hit) {
                const int l = __ffs(hit) - 1;
                group = c + l;
                const float before = __shfl_sync(0xffffffffu, incl, l > 0 ? l - 1 : 0);
                if (l > 0) run += before;
            } else {
                run += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        if (group >= 0) {
            // ... and in it the first kept element with which the mass crosses
            const int i = w0 + group * 32 + lane;
            float e = 0.f;
            if (i < w1) {
                e = sample_ex2((x[i] - xmax) * k);
                if (!(e >= threshold)) e = 0.f;
            }
            const float incl = warp_scan(e, lane);
            const unsigned hit = __ballot_sync(0xffffffffu, e > 0.f && run + incl > target);
            if (hit) cand = w0 + group * 32 + __ffs(hit) - 1;
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
    if (vocab > (1 << 18)) return VX_ERR_LIMIT;  // the fixed-point mass of a row has to fit 64 bits
    if (temperature && !uniform) return VX_ERR_SHAPE;
    VX_LAUNCH_K(VX_K_SAMPLE, (sample_kernel), rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, top_p, uniform, out);
    VX_LAUNCH_CHECK();
    return VX_OK;
}
