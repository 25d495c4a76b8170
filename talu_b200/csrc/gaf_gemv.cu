// Decode GEMV (M <= 16) for grouped-affine weights on sm_100a, plus the
// shape-agnostic kernel and the bit-exact dequant kernel.
//
// Replaces talu_gaffine_u4_matvec_f32
// (core/src/compute/cuda/kernels/ops/quant_ops.cu:46-93) and the CPU
// micro-kernels behind matmulGaffineU4Prefill / U8Prefill
// (core/src/compute/cpu/matmul_prefill.zig:28-480, :488-864).
//
// Arithmetic (same deferred form as the CPU reference, matmul_prefill.zig:163-337):
//     y[m,n] = sum_g ( s[n,g] * sum_{k in g} q[n,k] x[m,k] + b[n,g] * sum_{k in g} x[m,k] )
//
// How the fast kernel spends its instructions.  At HBM rate a B200 SM must
// retire ~40 weights per clock, which leaves no room for an int->float convert
// and an FMA per weight on the CUDA cores once M > 1.  So the codes go through
// the tensor cores as exact small integers:
//   * a packed word is split with four (shift, and, or) steps into bf16x2 pairs
//     0x4300|q, i.e. the bf16 value 128+q (exact for q < 128);
//   * warp-level mma.sync m16n8k16 (bf16 x bf16 -> f32) multiplies 16 weight rows
//     by up to 8 activation rows; the k order inside a fragment is free, so the
//     canonical [N, K/8] u32 layout is consumed as is, and the activations are
//     permuted to match with two byte-permutes per word;
//   * a second MMA with an all-ones A operand yields sum_k x[m,k] per group in the
//     same register layout as the accumulators;
//   * per group: y += s*acc + (b - 128 s) * xsum, in fp32.
// 8-bit codes reuse all of it: a byte is two nibbles, q = lo + 16 hi, and 16 x is
// exact in bf16, so a gaf8 row is a gaf4 row of twice the length against the
// activation vector (x0, 16 x0, x1, 16 x1, ...).
// f32 activations are split into bf16 hi + lo parts (two MMAs), which keeps ~16
// mantissa bits of x.
//
// Work split: one CTA = one block of 16 weight rows; its NW warps take
// consecutive K ranges (whole groups); gridDim.y further CTAs split K when there
// are too few row blocks to fill the machine.  Warps reduce through shared
// memory; CTAs through an fp32 scratch and a per-row-block arrival counter whose
// last arriver sums the partials in a fixed order (no spinning anywhere).
//
// Loads: every quad (4 lanes) reads one group of one row per step, so each
// lane's load width is a quarter of the group's bytes (8 B for gaf4_64).  Weights
// are read once (ld.global.nc, no L1 allocation) and prefetched a batch of groups
// ahead in registers; activations are re-read by every warp and stay in L1.
#include "gaf_internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tgaf {
namespace {

constexpr uint32_t kMagic128 = 0x43004300u;  // bf16x2 {128, 128}
constexpr uint32_t kOnesBf16 = 0x3F803F80u;  // bf16x2 {1, 1}
constexpr uint32_t kNibMask = 0x000F000Fu;

struct GemvParams {
    const uint8_t *packed;
    const uint16_t *scales;
    const uint16_t *biases;
    const void *x;
    void *y;
    float *partials;
    unsigned int *counters;
    uint32_t N, K, M;
    uint32_t groups;     // K / G
    uint32_t row_bytes;  // packed bytes per weight row
    uint32_t group;      // G
    uint32_t gpw;        // groups per warp slice
    uint32_t ks;         // CTAs along K (gridDim.y)
    uint32_t sdtype;     // 0 f16, 1 bf16
    uint32_t n_pad;      // gridDim.x * 16
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// streaming (read-once) global loads: no L1 allocation
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream_u64(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_stream_u128(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int WPT>
__device__ __forceinline__ void load_words(const uint8_t *p, uint32_t (&w)[WPT]) {
    if constexpr (WPT == 1) {
        w[0] = ldg_stream_u32(p);
    } else if constexpr (WPT == 2) {
        uint2 v = ldg_stream_u64(p);
        w[0] = v.x;
        w[1] = v.y;
    } else {
#pragma unroll
        for (int i = 0; i < WPT / 4; ++i) {
            uint4 v = ldg_stream_u128(p + 16 * i);
            w[4 * i + 0] = v.x;
            w[4 * i + 1] = v.y;
            w[4 * i + 2] = v.z;
            w[4 * i + 3] = v.w;
        }
    }
}

__device__ __forceinline__ float decode_sb(uint16_t raw, uint32_t sdtype) {
    // core/src/compute/cuda/kernels/ops/common_decode.cuh:1-13
    if (sdtype == 0) return __half2float(__ushort_as_half(raw));
    return __uint_as_float(static_cast<uint32_t>(raw) << 16);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float bf16lo_to_f32(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t mul16_bf16x2(uint32_t v) {
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&v);
    const __nv_bfloat162 k = __floats2bfloat162_rn(16.f, 16.f);
    a = __hmul2(a, k);
    return *reinterpret_cast<uint32_t *>(&a);
}

// Activation fragments for one packed word and one 8-row activation tile.
// frag[0..3] pair with the nibble pairs (0,4), (1,5), (2,6), (3,7) of the word.
// Plain (coherent) loads: the activations may have been written by the kernel
// this one was launched behind, and are only read after griddepcontrol.wait.
template <int BITS, bool XF32>
__device__ __forceinline__ void load_x_frags(const void *xrow, uint32_t kx, bool valid,
                                             uint32_t (&hi)[4], uint32_t (&lo)[4]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) hi[i] = lo[i] = 0u;
        return;
    }
    if constexpr (!XF32) {
        const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16 *>(xrow) + kx;
        if constexpr (BITS == 4) {
            const uint4 v = *reinterpret_cast<const uint4 *>(xp);
            hi[0] = prmt(v.x, v.z, 0x5410u);  // {x0, x4}
            hi[1] = prmt(v.x, v.z, 0x7632u);  // {x1, x5}
            hi[2] = prmt(v.y, v.w, 0x5410u);  // {x2, x6}
            hi[3] = prmt(v.y, v.w, 0x7632u);  // {x3, x7}
        } else {
            const uint2 v = *reinterpret_cast<const uint2 *>(xp);
            const uint32_t e = prmt(v.x, v.y, 0x5410u);  // {x0, x2}
            const uint32_t o = prmt(v.x, v.y, 0x7632u);  // {x1, x3}
            hi[0] = e;
            hi[1] = mul16_bf16x2(e);
            hi[2] = o;
            hi[3] = mul16_bf16x2(o);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) lo[i] = 0u;
    } else {
        const float *xp = static_cast<const float *>(xrow) + kx;
        float a[4], b[4];
        const float4 va = *reinterpret_cast<const float4 *>(xp);
        a[0] = va.x, a[1] = va.y, a[2] = va.z, a[3] = va.w;
        if constexpr (BITS == 4) {
            const float4 vb = *reinterpret_cast<const float4 *>(xp + 4);
            b[0] = vb.x, b[1] = vb.y, b[2] = vb.z, b[3] = vb.w;
#pragma unroll
            for (int i = 0; i < 4; ++i) {  // pair (x_i, x_{i+4})
                const uint32_t h = pack_bf16x2(a[i], b[i]);
                hi[i] = h;
                lo[i] = pack_bf16x2(a[i] - bf16lo_to_f32(h), b[i] - bf16hi_to_f32(h));
            }
        } else {
            // pairs (x0,x2) and (x1,x3), each also scaled by 16 for the high nibble
            const uint32_t he = pack_bf16x2(a[0], a[2]);
            const uint32_t ho = pack_bf16x2(a[1], a[3]);
            const uint32_t le = pack_bf16x2(a[0] - bf16lo_to_f32(he), a[2] - bf16hi_to_f32(he));
            const uint32_t lo_ = pack_bf16x2(a[1] - bf16lo_to_f32(ho), a[3] - bf16hi_to_f32(ho));
            hi[0] = he, hi[1] = mul16_bf16x2(he), hi[2] = ho, hi[3] = mul16_bf16x2(ho);
            lo[0] = le, lo[1] = mul16_bf16x2(le), lo[2] = lo_, lo[3] = mul16_bf16x2(lo_);
        }
    }
}

template <int GB, int BITS, int MT, bool XF32, int NW>
__global__ void __launch_bounds__(NW * 32)
gaf_gemv_mma_kernel(const GemvParams p) {
    constexpr int LW = GB / 4;                      // bytes one lane reads per group and row
    constexpr int WPT = LW / 4;                     // packed words per lane per group and row
    constexpr int XPB = 8 / BITS;                   // activations per packed byte
    constexpr float OFF = BITS == 4 ? 128.f : 2176.f;  // sum of the +128 offsets per unit of x
    constexpr int U = WPT >= 4 ? 2 : 4;             // groups per prefetch batch
    constexpr int MROWS = MT * 8;
    static_assert(WPT >= 1, "group too small for the fast path");

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;  // weight row inside the block (and +8); activation row inside a tile
    const int t = lane & 3;   // position inside the quad: which quarter of the group

    const uint32_t rb = blockIdx.x;
    const uint32_t n0 = min(rb * 16u + g, p.N - 1u);
    const uint32_t n1 = min(rb * 16u + g + 8u, p.N - 1u);
    const uint32_t slice = blockIdx.y * NW + warp;
    const uint32_t g_begin = min(slice * p.gpw, p.groups);
    const uint32_t g_end = min(g_begin + p.gpw, p.groups);

    const uint8_t *w0 = p.packed + static_cast<size_t>(n0) * p.row_bytes + t * LW;
    const uint8_t *w1 = p.packed + static_cast<size_t>(n1) * p.row_bytes + t * LW;
    const uint16_t *s0p = p.scales + static_cast<size_t>(n0) * p.groups;
    const uint16_t *s1p = p.scales + static_cast<size_t>(n1) * p.groups;
    const uint16_t *b0p = p.biases + static_cast<size_t>(n0) * p.groups;
    const uint16_t *b1p = p.biases + static_cast<size_t>(n1) * p.groups;

    uint32_t cur0[U][WPT], cur1[U][WPT];
    uint16_t csb[U][4];
    auto load_batch = [&](uint32_t gi, uint32_t (&a)[U][WPT], uint32_t (&b)[U][WPT], uint16_t (&sb)[U][4]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (gi + u < g_end) {
                load_words<WPT>(w0 + static_cast<size_t>(gi + u) * GB, a[u]);
                load_words<WPT>(w1 + static_cast<size_t>(gi + u) * GB, b[u]);
                sb[u][0] = __ldg(s0p + gi + u);
                sb[u][1] = __ldg(b0p + gi + u);
                sb[u][2] = __ldg(s1p + gi + u);
                sb[u][3] = __ldg(b1p + gi + u);
            }
        }
    };

    // Weights do not depend on the previous kernel in the stream: start fetching
    // them, then wait for it (no-op unless launched as a programmatic dependent).
    if (g_begin < g_end) load_batch(g_begin, cur0, cur1, csb);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;

    const size_t x_elt = XF32 ? 4 : 2;
    const uint8_t *xbase = static_cast<const uint8_t *>(p.x);

    for (uint32_t gi = g_begin; gi < g_end; gi += U) {
        uint32_t nxt0[U][WPT], nxt1[U][WPT];
        uint16_t nsb[U][4];
        if (gi + U < g_end) load_batch(gi + U, nxt0, nxt1, nsb);

#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (gi + u < g_end) {
                float acc[MT][4], xs[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][i] = xs[mt][i] = 0.f;

#pragma unroll
                for (int j = 0; j < WPT; ++j) {
                    const uint32_t kx = (gi + u) * p.group + (t * LW + 4 * j) * XPB;
                    const uint32_t wa = cur0[u][j], wb = cur1[u][j];
                    uint32_t pa[4], pb[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        pa[i] = ((wa >> (4 * i)) & kNibMask) | kMagic128;
                        pb[i] = ((wb >> (4 * i)) & kNibMask) | kMagic128;
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t m = mt * 8 + g;
                        uint32_t xh[4], xl[4];
                        load_x_frags<BITS, XF32>(xbase + static_cast<size_t>(m) * p.K * x_elt, kx, m < p.M, xh, xl);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            // group sums of x: all-ones A (for 8-bit, only the low-nibble slots)
                            mma_bf16_16816(xs[mt], kOnesBf16, kOnesBf16, BITS == 4 ? kOnesBf16 : 0u,
                                           BITS == 4 ? kOnesBf16 : 0u, xh[2 * h], xh[2 * h + 1]);
                            mma_bf16_16816(acc[mt], pa[2 * h], pb[2 * h], pa[2 * h + 1], pb[2 * h + 1],
                                           xh[2 * h], xh[2 * h + 1]);
                            if constexpr (XF32) {
                                mma_bf16_16816(xs[mt], kOnesBf16, kOnesBf16, BITS == 4 ? kOnesBf16 : 0u,
                                               BITS == 4 ? kOnesBf16 : 0u, xl[2 * h], xl[2 * h + 1]);
                                mma_bf16_16816(acc[mt], pa[2 * h], pb[2 * h], pa[2 * h + 1], pb[2 * h + 1],
                                               xl[2 * h], xl[2 * h + 1]);
                            }
                        }
                    }
                }
                const float s0 = decode_sb(csb[u][0], p.sdtype), b0 = decode_sb(csb[u][1], p.sdtype);
                const float s1 = decode_sb(csb[u][2], p.sdtype), b1 = decode_sb(csb[u][3], p.sdtype);
                const float b0o = fmaf(-OFF, s0, b0), b1o = fmaf(-OFF, s1, b1);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    yacc[mt][0] = fmaf(s0, acc[mt][0], yacc[mt][0]);
                    yacc[mt][1] = fmaf(s0, acc[mt][1], yacc[mt][1]);
                    yacc[mt][2] = fmaf(s1, acc[mt][2], yacc[mt][2]);
                    yacc[mt][3] = fmaf(s1, acc[mt][3], yacc[mt][3]);
                    yacc[mt][0] = fmaf(b0o, xs[mt][0], yacc[mt][0]);
                    yacc[mt][1] = fmaf(b0o, xs[mt][1], yacc[mt][1]);
                    yacc[mt][2] = fmaf(b1o, xs[mt][0], yacc[mt][2]);
                    yacc[mt][3] = fmaf(b1o, xs[mt][1], yacc[mt][3]);
                }
            }
        }
        if (gi + U < g_end) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int j = 0; j < WPT; ++j) cur0[u][j] = nxt0[u][j], cur1[u][j] = nxt1[u][j];
#pragma unroll
                for (int i = 0; i < 4; ++i) csb[u][i] = nsb[u][i];
            }
        }
    }

    // ---- reduce the NW warp slices through shared memory ----
    __shared__ float red[NW][MROWS][17];
    __shared__ unsigned int s_last;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        red[warp][mt * 8 + 2 * t][g] = yacc[mt][0];
        red[warp][mt * 8 + 2 * t + 1][g] = yacc[mt][1];
        red[warp][mt * 8 + 2 * t][g + 8] = yacc[mt][2];
        red[warp][mt * 8 + 2 * t + 1][g + 8] = yacc[mt][3];
    }
    __syncthreads();

    const int tid = threadIdx.x;
    const bool owner = tid < MROWS * 16;
    const uint32_t m = tid >> 4, nl = tid & 15;
    const uint32_t n = rb * 16u + nl;
    float v = 0.f;
    if (owner) {
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w][m][nl];
    }

    auto store = [&](float val) {
        if (m < p.M && n < p.N) {
            if constexpr (XF32)
                static_cast<float *>(p.y)[static_cast<size_t>(m) * p.N + n] = val;
            else
                static_cast<__nv_bfloat16 *>(p.y)[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(val);
        }
    };

    if (p.ks == 1) {
        if (owner) store(v);
        return;
    }

    // ---- reduce the gridDim.y CTAs through the fp32 scratch; the last CTA to
    // arrive at this row block's counter sums all partials in slice order ----
    if (owner) p.partials[(static_cast<size_t>(blockIdx.y) * MROWS + m) * p.n_pad + n] = v;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&p.counters[rb], 1u) == p.ks - 1u) ? 1u : 0u;
    __syncthreads();
    if (s_last) {
        __threadfence();
        if (owner) {
            float sum = 0.f;
            for (uint32_t k = 0; k < p.ks; ++k)
                sum += __ldcg(&p.partials[(static_cast<size_t>(k) * MROWS + m) * p.n_pad + n]);
            store(sum);
        }
        if (tid == 0) p.counters[rb] = 0u;  // ready for the next launch
    }
}

// ---------------------------------------------------------------------------
// Shape-agnostic kernel: any K % vpw == 0, G % vpw == 0, K % G == 0, any M.
// One warp per output feature, grid.y = activation row; the arithmetic is the
// reference CUDA kernel's (quant_ops.cu:78-89): acc = fmaf(x, q*s + b, acc).
// ---------------------------------------------------------------------------
template <bool XF32>
__global__ void __launch_bounds__(256)
gaf_gemv_generic_kernel(const uint8_t *packed, const uint16_t *scales, const uint16_t *biases,
                        const void *x, void *y, uint32_t N, uint32_t K, uint32_t group, uint32_t bits,
                        uint32_t sdtype, uint32_t row_bytes, uint32_t groups, uint32_t M) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t m = blockIdx.y;
    if (n >= N || m >= M) return;
    const uint32_t vpw = 32u / bits;
    const uint32_t mask = bits == 4 ? 0xFu : 0xFFu;
    const uint32_t words = K / vpw;
    const uint8_t *prow = packed + static_cast<size_t>(n) * row_bytes;
    float acc = 0.f;
    for (uint32_t wi = lane; wi < words; wi += 32u) {
        // packed rows may be only byte aligned when the caller wraps its own buffers
        uint32_t word;
        if ((reinterpret_cast<uintptr_t>(prow) & 3u) == 0) {
            word = reinterpret_cast<const uint32_t *>(prow)[wi];
        } else {
            const uint8_t *b = prow + 4u * wi;
            word = b[0] | (b[1] << 8) | (b[2] << 16) | (static_cast<uint32_t>(b[3]) << 24);
        }
        const uint32_t k0 = wi * vpw;
        const uint32_t gi = k0 / group;  // vpw divides G, so a word never straddles groups
        const float s = decode_sb(scales[static_cast<size_t>(n) * groups + gi], sdtype);
        const float b = decode_sb(biases[static_cast<size_t>(n) * groups + gi], sdtype);
        for (uint32_t j = 0; j < vpw; ++j) {
            const float q = static_cast<float>((word >> (j * bits)) & mask);
            float xv;
            if constexpr (XF32)
                xv = static_cast<const float *>(x)[static_cast<size_t>(m) * K + k0 + j];
            else
                xv = __bfloat162float(static_cast<const __nv_bfloat16 *>(x)[static_cast<size_t>(m) * K + k0 + j]);
            acc = fmaf(xv, fmaf(q, s, b), acc);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) {
        if constexpr (XF32)
            static_cast<float *>(y)[static_cast<size_t>(m) * N + n] = acc;
        else
            static_cast<__nv_bfloat16 *>(y)[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(acc);
    }
}

// ---------------------------------------------------------------------------
// Dequant: one thread per packed word, out[n, k] = fmaf(q, s, b) (bit-exact with
// core/src/compute/cpu/quant_decode.zig:64-130).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gaf_dequant_f32_kernel(const uint8_t *packed, const uint16_t *scales, const uint16_t *biases, float *out,
                       uint32_t N, uint32_t K, uint32_t group, uint32_t bits, uint32_t sdtype,
                       uint32_t row_bytes, uint32_t groups) {
    const uint32_t vpw = 32u / bits;
    const uint32_t words = K / vpw;
    const size_t total = static_cast<size_t>(N) * words;
    const uint32_t mask = bits == 4 ? 0xFu : 0xFFu;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t n = static_cast<uint32_t>(idx / words);
        const uint32_t wi = static_cast<uint32_t>(idx - static_cast<size_t>(n) * words);
        const uint8_t *bp = packed + static_cast<size_t>(n) * row_bytes + 4u * wi;
        uint32_t word;
        if ((reinterpret_cast<uintptr_t>(bp) & 3u) == 0)
            word = *reinterpret_cast<const uint32_t *>(bp);
        else
            word = bp[0] | (bp[1] << 8) | (bp[2] << 16) | (static_cast<uint32_t>(bp[3]) << 24);
        const uint32_t k0 = wi * vpw;
        const uint32_t gi = k0 / group;
        const float s = decode_sb(scales[static_cast<size_t>(n) * groups + gi], sdtype);
        const float b = decode_sb(biases[static_cast<size_t>(n) * groups + gi], sdtype);
        float *o = out + static_cast<size_t>(n) * K + k0;
        for (uint32_t j = 0; j < vpw; ++j) o[j] = fmaf(static_cast<float>((word >> (j * bits)) & mask), s, b);
    }
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
struct GemvPlan {
    int nw;
    uint32_t ks;
    uint32_t gpw;
    uint32_t rbs;
};

constexpr uint32_t kMaxKs = 32;

GemvPlan plan_gemv(const WeightView &w, const GemvTuning &tune, int sm_count) {
    GemvPlan pl;
    pl.rbs = (w.N + 15u) / 16u;
    const uint32_t target = tune.slices_target > 0 ? static_cast<uint32_t>(tune.slices_target)
                                                   : static_cast<uint32_t>(sm_count) * 32u;
    uint32_t s_total = (target + pl.rbs - 1u) / pl.rbs;
    if (s_total < 1u) s_total = 1u;
    if (s_total > w.groups) s_total = w.groups;
    int nw = tune.warps > 0 ? tune.warps : (s_total > 4u ? 8 : 4);
    if (nw != 4 && nw != 8) nw = 8;
    pl.nw = nw;
    uint32_t ks = (s_total + nw - 1u) / nw;
    if (ks > kMaxKs) ks = kMaxKs;
    pl.gpw = (w.groups + ks * nw - 1u) / (ks * nw);
    pl.ks = (w.groups + pl.gpw * nw - 1u) / (pl.gpw * nw);
    return pl;
}

template <int GB, int BITS, int MT, bool XF32, int NW>
cudaError_t launch_gemv(const GemvParams &p, dim3 grid, bool pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gaf_gemv_mma_kernel<GB, BITS, MT, XF32, NW>, p);
}

template <int GB, int BITS>
cudaError_t dispatch_gemv(const GemvParams &p, dim3 grid, int mt, bool xf32, int nw, bool pdl,
                          cudaStream_t stream) {
#define TGAF_CASE(MTv, XFv, NWv) \
    if (mt == MTv && xf32 == XFv && nw == NWv) return launch_gemv<GB, BITS, MTv, XFv, NWv>(p, grid, pdl, stream);
    TGAF_CASE(1, false, 4)
    TGAF_CASE(1, false, 8)
    TGAF_CASE(2, false, 4)
    TGAF_CASE(2, false, 8)
    TGAF_CASE(1, true, 4)
    TGAF_CASE(1, true, 8)
    TGAF_CASE(2, true, 4)
    TGAF_CASE(2, true, 8)
#undef TGAF_CASE
    return cudaErrorNotSupported;
}

}  // namespace

bool gemv_mma_eligible(const WeightView &w, const void *x, const void *y, bool x_f32) {
    const uint32_t gb = w.group * w.bits / 8u;
    if (gb != 16u && gb != 32u && gb != 64u && gb != 128u) return false;
    if (w.row_bytes != w.K * w.bits / 8u) return false;
    // each lane reads gb/4 bytes at a time (up to 16): row starts and rows must keep that alignment
    const uint32_t lw = gb / 4u > 16u ? 16u : gb / 4u;
    if (reinterpret_cast<uintptr_t>(w.packed) % lw != 0 || w.row_bytes % lw != 0) return false;
    if (reinterpret_cast<uintptr_t>(w.scales) % 2u != 0 || reinterpret_cast<uintptr_t>(w.biases) % 2u != 0) return false;
    // activation rows are read 16 bytes at a time
    const size_t xrow = static_cast<size_t>(w.K) * (x_f32 ? 4u : 2u);
    if (reinterpret_cast<uintptr_t>(x) % 16u != 0 || xrow % 16u != 0) return false;
    if (reinterpret_cast<uintptr_t>(y) % (x_f32 ? 4u : 2u) != 0) return false;
    return true;
}

size_t gemv_mma_scratch_bytes(const WeightView &w, uint32_t M, const GemvTuning &tune, int sm_count) {
    const GemvPlan pl = plan_gemv(w, tune, sm_count);
    if (pl.ks <= 1u) return 0;
    const uint32_t mrows = M <= 8u ? 8u : 16u;
    return static_cast<size_t>(pl.ks) * mrows * (static_cast<size_t>(pl.rbs) * 16u) * sizeof(float);
}

cudaError_t gemv_mma(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                     const Scratch &scratch, const GemvTuning &tune, cudaStream_t stream, int sm_count) {
    if (M == 0 || M > 16u) return cudaErrorNotSupported;
    if (!gemv_mma_eligible(w, x, y, x_f32)) return cudaErrorNotSupported;
    const GemvPlan pl = plan_gemv(w, tune, sm_count);
    const int mt = M <= 8u ? 1 : 2;
    if (pl.ks > 1u) {
        const size_t need = static_cast<size_t>(pl.ks) * (mt * 8) * (static_cast<size_t>(pl.rbs) * 16u) * sizeof(float);
        if (need > scratch.partial_bytes || pl.rbs > scratch.counter_count) return cudaErrorMemoryAllocation;
    }
    GemvParams p;
    p.packed = w.packed;
    p.scales = w.scales;
    p.biases = w.biases;
    p.x = x;
    p.y = y;
    p.partials = scratch.partials;
    p.counters = scratch.counters;
    p.N = w.N;
    p.K = w.K;
    p.M = M;
    p.groups = w.groups;
    p.row_bytes = w.row_bytes;
    p.group = w.group;
    p.gpw = pl.gpw;
    p.ks = pl.ks;
    p.sdtype = w.sdtype;
    p.n_pad = pl.rbs * 16u;
    const dim3 grid(pl.rbs, pl.ks);
    const bool pdl = tune.pdl != 0;
    const uint32_t gb = w.group * w.bits / 8u;
    if (w.bits == 4) {
        if (gb == 16u) return dispatch_gemv<16, 4>(p, grid, mt, x_f32, pl.nw, pdl, stream);
        if (gb == 32u) return dispatch_gemv<32, 4>(p, grid, mt, x_f32, pl.nw, pdl, stream);
        if (gb == 64u) return dispatch_gemv<64, 4>(p, grid, mt, x_f32, pl.nw, pdl, stream);
    } else {
        if (gb == 32u) return dispatch_gemv<32, 8>(p, grid, mt, x_f32, pl.nw, pdl, stream);
        if (gb == 64u) return dispatch_gemv<64, 8>(p, grid, mt, x_f32, pl.nw, pdl, stream);
        if (gb == 128u) return dispatch_gemv<128, 8>(p, grid, mt, x_f32, pl.nw, pdl, stream);
    }
    return cudaErrorNotSupported;
}

cudaError_t gemv_generic(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                         cudaStream_t stream) {
    if (M == 0) return cudaErrorInvalidValue;
    // grid.y is limited to 65535 rows per launch
    for (uint32_t m0 = 0; m0 < M; m0 += 65535u) {
        const uint32_t mc = (M - m0) < 65535u ? (M - m0) : 65535u;
        const dim3 grid((w.N + 7u) / 8u, mc);
        const size_t xoff = static_cast<size_t>(m0) * w.K * (x_f32 ? 4u : 2u);
        const size_t yoff = static_cast<size_t>(m0) * w.N * (x_f32 ? 4u : 2u);
        const void *xp = static_cast<const uint8_t *>(x) + xoff;
        void *yp = static_cast<uint8_t *>(y) + yoff;
        if (x_f32)
            gaf_gemv_generic_kernel<true><<<grid, 256, 0, stream>>>(w.packed, w.scales, w.biases, xp, yp, w.N, w.K,
                                                                    w.group, w.bits, w.sdtype, w.row_bytes,
                                                                    w.groups, mc);
        else
            gaf_gemv_generic_kernel<false><<<grid, 256, 0, stream>>>(w.packed, w.scales, w.biases, xp, yp, w.N, w.K,
                                                                     w.group, w.bits, w.sdtype, w.row_bytes,
                                                                     w.groups, mc);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t dequant_f32(const WeightView &w, float *out, cudaStream_t stream) {
    const size_t total = static_cast<size_t>(w.N) * (w.K / (32u / w.bits));
    size_t blocks = (total + 255u) / 256u;
    if (blocks > 148u * 32u) blocks = 148u * 32u;
    if (blocks == 0) blocks = 1;
    gaf_dequant_f32_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        w.packed, w.scales, w.biases, out, w.N, w.K, w.group, w.bits, w.sdtype, w.row_bytes, w.groups);
    return cudaGetLastError();
}

}  // namespace tgaf
