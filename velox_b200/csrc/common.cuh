// Shared helpers of the kernels: element types, conversions, warp and block
// reductions, the error convention of the C entry points.
//
// Every entry point is `extern "C"`, takes raw device pointers and a stream,
// launches on that stream and returns 0 or a negative code (VX_ERR_*) for a
// refused size, or the positive cudaError_t of a failed launch.  Nothing here
// allocates device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VX_OK 0
#define VX_ERR_SHAPE (-1)    // a size the kernel does not take
#define VX_ERR_DTYPE (-2)    // an element type code the kernel does not know
#define VX_ERR_ALIGN (-3)    // a pointer or stride that is not aligned as needed
#define VX_ERR_LIMIT (-4)    // beyond a stated maximum
#define VX_ERR_DRIVER (-5)   // the driver lacks an entry point the kernel needs

#define VX_F32 0
#define VX_BF16 1

#define VX_LAUNCH_CHECK()                          \
    do {                                           \
        cudaError_t e__ = cudaGetLastError();      \
        if (e__ != cudaSuccess) return (int)e__;   \
    } while (0)

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch (on unless vx_set_pdl(0)).  With it, the next
// kernel in the stream may become resident while this one is still running, so
// that its launch and its prologue (for the matrix products: the first loads of
// weights, which depend on nothing) overlap this kernel's work.  The rules every
// kernel here keeps:
//   - pdl_wait() before it reads anything an earlier kernel wrote and before it
//     writes anything at all; it returns when all earlier work in the stream is
//     complete and visible.  At least one block of every launch reaches it: a grid
//     that ended without waiting would let its successor run ahead of its
//     predecessor.
//   - pdl_trigger() (dependents may be launched) only AFTER pdl_wait().  So at most
//     one successor is resident beside the running kernel.  Triggering first let
//     the whole chain of later kernels pile up on the SMs, and a decode step ran
//     18 % slower.
// Launched without the attribute (or after a kernel of another library) both
// calls do nothing and the order is the stream's.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Set-up that belongs to a device's copy of a kernel (the opt-in to more dynamic
// shared memory, the SM count) is remembered per device: a process may hold engines
// on several GPUs.  The index of the current device, or -1 if it cannot be had or
// is beyond VX_MAX_DEVICES.
#define VX_MAX_DEVICES 64
static inline int vx_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= VX_MAX_DEVICES) return -1;
    return dev;
}
// Sets a kernel's dynamic shared-memory limit once per device (`done`: VX_MAX_DEVICES flags).
template <typename K>
static inline int vx_configure_smem(K kernel, size_t smem, bool* done) {
    const int dev = vx_current_device();
    if (dev < 0) return VX_ERR_LIMIT;
    if (done[dev]) return VX_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    done[dev] = true;
    return VX_OK;
}
// Multiprocessors of the current device (`cache`: VX_MAX_DEVICES ints, zero at first).
static inline int vx_sm_count(int* cache) {
    const int dev = vx_current_device();
    if (dev < 0) return 148;
    if (!cache[dev] && (cudaDeviceGetAttribute(&cache[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
                        cache[dev] <= 0))
        cache[dev] = 148;
    return cache[dev];
}

extern "C" int vx_pdl_is_enabled(void);
// While set (per host thread), kernels are launched in plain stream order whatever
// vx_set_pdl says: for entry points whose predecessor in the stream is not this library's.
extern "C" void vx_pdl_suppress(int on);
extern "C" int vx_pdl_mask(void);

// Kernel classes, for switching programmatic dependent launch on and off per class
// (vx_set_pdl_mask; bit i = class i).
#define VX_K_ELEMENTWISE 0
#define VX_K_ROPE 1
#define VX_K_ATTENTION 2
#define VX_K_GEMM 3
#define VX_K_SAMPLE 4
#define VX_K_JOIN 5

template <typename... KArgs, typename... Args>
static inline cudaError_t vx_launch_class(int kclass, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (vx_pdl_is_enabled() && ((vx_pdl_mask() >> kclass) & 1)) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t vx_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vx_pdl_is_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define VX_LAUNCH_K(kclass, kernel, grid, block, smem, stream, ...)                                       \
    do {                                                                                                 \
        cudaError_t e__ = vx_launch_class(kclass, kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__); \
        if (e__ != cudaSuccess) return (int)e__;                                                         \
    } while (0)

#define VX_LAUNCH(kernel, grid, block, smem, stream, ...)                                          \
    do {                                                                                           \
        cudaError_t e__ = vx_launch(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__);   \
        if (e__ != cudaSuccess) return (int)e__;                                                   \
    } while (0)

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  Every
// thread gets the result.  The order of the additions is fixed by the block
// size alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Activation functions of gated feed-forwards, by code.
#define VX_ACT_SILU 0
#define VX_ACT_GELU 1
#define VX_ACT_GELU_TANH 2
#define VX_ACT_RELU 3

__device__ __forceinline__ float activation(float z, int act) {
    switch (act) {
        case VX_ACT_SILU: return z / (1.f + expf(-z));
        case VX_ACT_GELU: return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
        case VX_ACT_GELU_TANH: {
            const float c = 0.7978845608028654f;
            return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
        }
        default: return fmaxf(z, 0.f);
    }
}
