// out[M,N] = x[M,K] * W[N,K]^T (+ bias) for a handful of rows (M <= 8): the
// matrix products of a decode step, where the whole cost is reading W once.
//
// The product is formed transposed, out^T = W x^T, so that 16 rows of W fill the
// 16-row side of a tensor-core tile (mma.sync.m16n8k16, bf16 in, float32 out) and
// the few rows of x sit on the 8-column side.  A block owns 16 rows of W (or,
// with a gated epilogue, 8 gate rows and their 8 up rows) and the whole of K; its
// warps take the 32-wide k chunks in turn (chunk c goes to warp c mod the number of warps), each
// thread loading 16 contiguous bytes of two W rows per chunk straight from global
// memory into registers, four chunks in flight, with no shared memory on the way:
// every byte of W is used exactly once.  The first chunks are asked for before the
// wait on earlier kernels (programmatic dependent launch): weights depend on
// nothing, so they stream while the previous kernel finishes.  x is read through
// L1/L2 (every block reads all of it).  The k order inside a tile is permuted the
// same way for both operands, which a dot product does not notice.  The 8 warps'
// partial tiles are added in shared memory in warp order, so the result is the
// same on every run and a row's result does not depend on the rows beside it.
//
// Epilogues: plain (bf16 or float32 out, optional bias), or gated: row r < 8 of a
// tile is a gate row, row r + 8 its up row, out = act(gate) * up (float32 math).
//
// Sizes: M <= 8; K a multiple of 32; N any (a multiple of 16 with the gated
// epilogue); 16-byte aligned rows.
#include "common.cuh"

// Warps per block and chunks a warp keeps in flight are template parameters: a
// matrix of few rows gives few blocks, and then each block must keep more bytes
// on their way to fill the memory pipe (see pick_variant).

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool GATED, typename TOut, int SK_WARPS, int SK_UNROLL, int MIN_BLOCKS>
__global__ void __launch_bounds__(SK_WARPS * 32, MIN_BLOCKS)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const float* __restrict__ bias,
                   TOut* __restrict__ out, int M, int N, int K, int ldx, int ldw, int ldo, int act, int R) {
    __shared__ float red[SK_WARPS][16][9];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // A block owns R <= 16 rows of W (gated: R <= 8 output features, each a gate row
    // and the up row 8 below it in its 16-row tile); rows of the tile beyond R are
    // not loaded.  R is chosen so that the blocks fill whole waves of the GPU.
    const int row0 = blockIdx.x * R;
    int ra, rb;
    bool va, vb;
    if (!GATED) {
        ra = row0 + g;
        rb = row0 + g + 8;
        va = g < R && ra < N;
        vb = g + 8 < R && rb < N;
    } else {
        const int f = row0 + g;  // output feature
        ra = ((f >> 3) << 4) + (f & 7);
        rb = ra + 8;
        va = vb = g < R && rb < N;
    }
    const bf16* wa = W + (size_t)(va ? ra : 0) * ldw + t * 8;
    const bf16* wb = W + (size_t)(vb ? rb : 0) * ldw + t * 8;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    // row of x this thread loads: column g of the 8-column tile
    const bool xok = g < M;
    const bf16* xr = x + (size_t)min(g, M - 1) * ldx + t * 8;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    const int nchunks = K >> 5;
    int c = warp;
    uint4 a[SK_UNROLL], b[SK_UNROLL];
    bool loaded = false;
    if (c + (SK_UNROLL - 1) * SK_WARPS < nchunks) {
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            const int k = (c + u * SK_WARPS) << 5;
            a[u] = va ? ld_stream16(wa + k) : zero4;
            b[u] = vb ? ld_stream16(wb + k) : zero4;
        }
        loaded = true;
    }
    pdl_wait();
    pdl_trigger();
    for (; c + (SK_UNROLL - 1) * SK_WARPS < nchunks; c += SK_UNROLL * SK_WARPS) {
        if (!loaded) {
#pragma unroll
            for (int u = 0; u < SK_UNROLL; ++u) {
                const int k = (c + u * SK_WARPS) << 5;
                a[u] = va ? ld_stream16(wa + k) : zero4;
                b[u] = vb ? ld_stream16(wb + k) : zero4;
            }
        }
        loaded = false;
        uint4 xv[SK_UNROLL];
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u)
            xv[u] = xok ? *reinterpret_cast<const uint4*>(xr + ((c + u * SK_WARPS) << 5)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < SK_UNROLL; ++u) {
            mma_bf16_16816(acc, a[u].x, b[u].x, a[u].y, b[u].y, xv[u].x, xv[u].y);
            mma_bf16_16816(acc, a[u].z, b[u].z, a[u].w, b[u].w, xv[u].z, xv[u].w);
        }
    }
    for (; c < nchunks; c += SK_WARPS) {
        const int k = c << 5;
        const uint4 ta = va ? ld_stream16(wa + k) : zero4, tb = vb ? ld_stream16(wb + k) : zero4;
        const uint4 xv = xok ? *reinterpret_cast<const uint4*>(xr + k) : make_uint4(0, 0, 0, 0);
        mma_bf16_16816(acc, ta.x, tb.x, ta.y, tb.y, xv.x, xv.y);
        mma_bf16_16816(acc, ta.z, tb.z, ta.w, tb.w, xv.z, xv.w);
    }
    // thread holds out^T[row g (c0,c1) and g+8 (c2,c3)][x rows 2t, 2t+1]
    red[warp][g][2 * t] = acc[0];
    red[warp][g][2 * t + 1] = acc[1];
    red[warp][g + 8][2 * t] = acc[2];
    red[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();
    if (!GATED) {
        if (threadIdx.x < 16 * 8) {
            const int r = threadIdx.x & 15, m = threadIdx.x >> 4;  // consecutive threads -> consecutive output columns
            const int nrow = row0 + r;
            if (m < M && r < R && nrow < N) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < SK_WARPS; ++w) v += red[w][r][m];
                if (bias) v += bias[nrow];
                out[(size_t)m * ldo + nrow] = from_f32<TOut>(v);
            }
        }
    } else {
        if (threadIdx.x < 8 * 8) {
            const int r = threadIdx.x & 7, m = threadIdx.x >> 3;
            const int col = row0 + r;  // output feature
            if (m < M && r < R && col * 2 < N) {
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < SK_WARPS; ++w) { gate += red[w][r][m]; up += red[w][r + 8][m]; }
                out[(size_t)m * ldo + col] = from_f32<TOut>(activation(gate, act) * up);
            }
        }
    }
}

// Variants (warps, chunks in flight per warp, blocks per SM the registers allow):
//   1: 8, 4, 4   many blocks: four per SM keep the pipe full
//   2: 16, 4, 2  fewer blocks than 4 per SM: twice the warps on each tile
//   3: 8, 8, 2
//   4: 16, 8, 1
//   5: 16, 2, 4
//   6: 8, 8, 3
//   7: 4, 8, 4
// Measured on a B200 (M = 8, microseconds, back to back under programmatic
// launch, variants 1/2/3/7): 4096x4096 9.2/7.4/7.0/7.6; 4096x12288 24/19/16.8/18.7;
// 6144x4096 11.4/11.4/10.3/9.6; 24576x4096 gated 44/45/33.6/35.4; 151936x4096
// 218/204/178/200; 5120x5120 12.1/13.7/13.7/9.8; 5120x17408 37/40/34/30;
// 10240x5120 23/23/22/19.  Variant 1 fills the register file, which keeps the
// next kernel's blocks out until it ends.
static int sm_count() {
    static int sms[VX_MAX_DEVICES];
    return vx_sm_count(sms);
}

static int pick_variant(int N, int K) {
    const int sms = sm_count();
    const int tiles = (N + 15) / 16;
    if (tiles <= 2 * sms || tiles >= 8 * sms) return 3;
    return 7;
}

template <bool GATED, typename TOut>
static int launch_skinny(const bf16* x, const bf16* W, const float* bias, TOut* out, int M, int N, int K, int ldx,
                         int ldw, int ldo, int act, int variant, cudaStream_t stream) {
    const bool balance = variant < 100;  // variant + 100: whole tiles per block, for comparison
    if (variant >= 100) variant -= 100;
    if (variant == 0) variant = pick_variant(N, K);
    // Rows (gated: features) per block: the most a tile holds, lowered until the
    // blocks fill whole waves (slots = SMs x blocks per SM of the variant).
    const int units = GATED ? N / 2 : N, tile = GATED ? 8 : 16;
    int R = tile;
    if (variant >= 1 && variant <= 7 && balance) {
        static const int per_sm[8] = {0, 4, 2, 2, 1, 4, 3, 4};
        const long long slots = (long long)sm_count() * per_sm[variant];
        const long long tiles = (units + tile - 1) / tile;
        const long long waves = (tiles + slots - 1) / slots;
        R = (int)((units + waves * slots - 1) / (waves * slots));
        R = R < 1 ? 1 : (R > tile ? tile : R);
    }
    const int blocks = (units + R - 1) / R;
#define SK_GO(WARPS, UNROLL, MINB)                                                                                  \
    VX_LAUNCH_K(VX_K_GEMM, (gemm_skinny_kernel<GATED, TOut, WARPS, UNROLL, MINB>), blocks, WARPS * 32, 0, stream, x, W, \
                bias, out, M, N, K, ldx, ldw, ldo, act, R)
    switch (variant) {
        case 1: SK_GO(8, 4, 4); break;
        case 2: SK_GO(16, 4, 2); break;
        case 3: SK_GO(8, 8, 2); break;
        case 4: SK_GO(16, 8, 1); break;
        case 5: SK_GO(16, 2, 4); break;
        case 6: SK_GO(8, 8, 3); break;
        case 7: SK_GO(4, 8, 4); break;
        default: return VX_ERR_SHAPE;
    }
#undef SK_GO
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// gated: 0 plain; 1: W rows come in tiles of 16 = 8 gate rows then their 8 up
// rows, and out is [M, N/2] = act(gate) * up.  out_dtype: VX_BF16 or VX_F32.
// variant: 0 lets the sizes choose (pick_variant); 1..5 name one, for tuning.
extern "C" int vx_gemm_skinny(const void* x, const void* W, const float* bias, void* out, int M, int N, int K,
                              int ldx, int ldw, int ldo, int gated, int act, int out_dtype, int variant,
                              cudaStream_t stream) {
    if (M <= 0 || N <= 0) return VX_OK;
    if (M > 8 || K <= 0 || (K & 31)) return VX_ERR_SHAPE;
    if (ldx < K || ldw < K || (ldx & 7) || (ldw & 7)) return VX_ERR_ALIGN;
    if ((((uintptr_t)x) | ((uintptr_t)W)) & 15) return VX_ERR_ALIGN;
    if (gated && ((N & 15) || bias || act < 0 || act > 3)) return VX_ERR_SHAPE;
    if (ldo < (gated ? N / 2 : N)) return VX_ERR_SHAPE;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
#define SK_CALL(G, T) launch_skinny<G, T>(xp, wp, bias, (T*)out, M, N, K, ldx, ldw, ldo, act, variant, stream)
    if (out_dtype == VX_BF16) return gated ? SK_CALL(true, bf16) : SK_CALL(false, bf16);
    if (out_dtype == VX_F32) return gated ? SK_CALL(true, float) : SK_CALL(false, float);
#undef SK_CALL
    return VX_ERR_DTYPE;
}
