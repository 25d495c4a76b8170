// Prefill dequant-GEMM for gaf4 weights on the 5th-generation tensor cores.
//
//   y[M, N] (bf16) = x[M, K] (bf16) * W^T,  W[n, k] = q * scale + bias (gaf4, group 32 / 64 / 128)
//
// Replaces, for large M, the CPU 4x2 micro-kernel path (core/src/compute/cpu/matmul_prefill.zig:121-358)
// and the reference CUDA backend's loop of the matvec kernel over rows
// (core/src/inference/backend/cuda/engine.zig:4433-4473).
//
// One persistent CTA per SM computes 256 x 256 output tiles:
//   * warp 0 (one lane): TMA producer.  Per 64-deep K block it loads two 128-row x 64 activation
//     tiles (128-byte swizzle, the layout the MMA descriptor names) and the packed codes of 256
//     weight rows (256 x 32 bytes) into a 3-stage shared-memory ring.
//   * warps 2..9 (256 threads, one weight row each): unpack the 64 codes of their row, apply
//     scale and bias in bf16 (one fused multiply-add per pair, a single rounding of q*s+b), and
//     write the row of the K-major bf16 B tile with the same 128-byte swizzle.
//   * warp 1 (one lane): issues tcgen05.mma (128 x 256 x 16, bf16 -> fp32) for the two 128-row
//     halves of the tile, accumulators in tensor memory (2 x 256 columns), and commits to the
//     ring's mbarriers.
//   * after the last K block warps 2..9 read the accumulators back (tcgen05.ld), round to bf16
//     and store y.
// Tiles are walked N-tile major so that the CTAs running at the same time share weight rows in L2.
//
// All waits on mbarriers are bounded; a wait that runs out sets the host-visible error word and
// a CTA-wide abort flag, every role then falls through to the common exit where tensor memory is
// released.
#include "gaf_internal.h"

#include <cuda.h>
#include <cuda_bf16.h>

namespace tgaf {
namespace {

constexpr int kBM = 256;           // tile rows of x (two UMMA M = 128 halves)
constexpr int kBN = 256;           // tile rows of W (UMMA N)
constexpr int kBK = 64;            // K block: 64 bf16 = 128 bytes, the swizzle span
constexpr int kStagesTc = 3;
constexpr int kATile = 128 * 128;  // 128 rows x 128 bytes
constexpr int kBTile = kBN * 128;  // 256 rows x 128 bytes
constexpr int kPTile = kBN * 32;   // packed codes: 256 rows x 32 bytes
constexpr int kStageTc = 2 * kATile + kBTile + kPTile;  // 73728
constexpr int kSmemTc = kStagesTc * kStageTc + 1024;
constexpr int kDequantWarps = 8;
constexpr int kThreadsTc = (2 + kDequantWarps) * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWaitLimitTc = 1u << 22;

struct GemmParams {
    const uint16_t *scales;
    const uint16_t *biases;
    void *y;
    unsigned int *error_word;
    uint32_t M, N, K;
    uint32_t groups;   // K / G
    uint32_t group;    // G
    uint32_t sdtype;   // 1 bf16, 0 f16
    uint32_t m_tiles, n_tiles, k_blocks;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait that also gives up as soon as another role has raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          unsigned int *error_word, uint32_t code) {
    for (uint32_t it = 0; it < kWaitLimitTc; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) {
            if (*abort_flag) return false;
            __nanosleep(it > 4096 ? 128 : 20);
        }
    }
    atomicOr(error_word, code);
    *abort_flag = 1u;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, uint32_t c0, uint32_t c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused with swizzle): 1
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: 8 rows x 128 bytes
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle
    return d;
}
// bf16 x bf16 -> f32, both operands K-major, M = 128, N = 256
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// one of the eight 16-bit values held in a uint4, as a bf16x2 register {v, v} (f16 sources are converted)
__device__ __forceinline__ uint32_t pick_pair(const uint4 &v, uint32_t idx, uint32_t sdtype) {
    const uint32_t w = (idx & 4u) ? ((idx & 2u) ? v.w : v.z) : ((idx & 2u) ? v.y : v.x);
    uint32_t h = (idx & 1u) ? (w >> 16) : (w & 0xFFFFu);
    if (sdtype == 0u) {
        const float f = __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
        h = __bfloat16_as_ushort(__float2bfloat16_rn(f));  // only exact for f16 values with <= 8 significant bits
    }
    return h | (h << 16);
}

__global__ void __launch_bounds__(kThreadsTc, 1)
gaf_gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kStagesTc];    // TMA landed (x tiles + packed codes)
    __shared__ __align__(8) uint64_t s_bready[kStagesTc];  // B tile dequantized
    __shared__ __align__(8) uint64_t s_empty[kStagesTc];   // MMAs that read the stage have completed
    __shared__ __align__(8) uint64_t s_acc_full;           // all MMAs of the tile have completed
    __shared__ __align__(8) uint64_t s_acc_empty;          // accumulators have been read back
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        s_abort = 0u;
        for (int s = 0; s < kStagesTc; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_bready[s]), kDequantWarps);
            mbar_init(smem_u32(&s_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_acc_full), 1);
        mbar_init(smem_u32(&s_acc_empty), kDequantWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // tensor memory: all 512 columns (two 128 x 256 fp32 accumulators); this warp also frees them
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;

    const uint32_t total_tiles = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_p)) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const uint32_t n0 = (tile / p.m_tiles) * kBN, m0 = (tile % p.m_tiles) * kBM;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t stage = it % kStagesTc, round = it / kStagesTc;
                    if (round > 0 && !mbar_wait(smem_u32(&s_empty[stage]), (round - 1u) & 1u, &s_abort, p.error_word, 0x100u)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sb = base + stage * kStageTc;
                    const uint32_t full = smem_u32(&s_full[stage]);
                    mbar_arrive_expect_tx(full, 2 * kATile + kPTile);  // out-of-range rows arrive as zeros
                    tma_load_2d(sb, &tmap_x, kb * kBK, m0, full);
                    tma_load_2d(sb + kATile, &tmap_x, kb * kBK, m0 + 128u, full);
                    tma_load_2d(sb + 2 * kATile + kBTile, &tmap_p, kb * 32u, n0, full);
                }
            }
            if (!ok) {
                // copies already issued get a bounded time to land before shared memory is released
                const uint32_t pending = it < static_cast<uint32_t>(kStagesTc) ? it : static_cast<uint32_t>(kStagesTc);
                for (uint32_t i = 0; i < pending; ++i) {
                    const uint32_t idx = it - 1u - i;
                    for (uint32_t spin = 0; spin < (1u << 20); ++spin)
                        if (mbar_try_wait(smem_u32(&s_full[idx % kStagesTc]), (idx / kStagesTc) & 1u)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++ti) {
                if (ti > 0 && !mbar_wait(smem_u32(&s_acc_empty), (ti - 1u) & 1u, &s_abort, p.error_word, 0x200u)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // rows 128..255 of the tile exist only when M reaches them (skinny M: half the tensor work)
                const bool two_halves = (tile % p.m_tiles) * kBM + 128u < p.M;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t stage = it % kStagesTc, par = (it / kStagesTc) & 1u;
                    if (!mbar_wait(smem_u32(&s_full[stage]), par, &s_abort, p.error_word, 0x400u) ||
                        !mbar_wait(smem_u32(&s_bready[stage]), par, &s_abort, p.error_word, 0x800u)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sb = base + stage * kStageTc;
                    const uint64_t a0 = umma_desc_sw128(sb), a1 = umma_desc_sw128(sb + kATile);
                    const uint64_t bd = umma_desc_sw128(sb + 2 * kATile);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBK / 16; ++k16) {
                        const uint32_t acc = (kb | k16) ? 1u : 0u;
                        // advancing 16 elements (32 bytes) along K inside the swizzle span: +2 in the address field
                        umma_f16(tmem_base, a0 + 2 * k16, bd + 2 * k16, kInstrDesc, acc);
                        if (two_halves) umma_f16(tmem_base + 256u, a1 + 2 * k16, bd + 2 * k16, kInstrDesc, acc);
                    }
                    umma_commit(smem_u32(&s_empty[stage]));  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(smem_u32(&s_acc_full));
            }
        }
    } else {
        // ------------------------------ dequant + epilogue warps ------------------------------
        const uint32_t r = (warp - 2) * 32 + lane;  // weight row of the tile this thread dequantizes
        const uint32_t q = warp & 3;                // tensor-memory lane quadrant this warp may read
        const uint32_t hsel = (warp - 2) >> 2;      // accumulator (128-row half of the tile) this warp writes out
        const uint32_t gshift = p.group == 32u ? 5u : (p.group == 64u ? 6u : 7u);
        uint32_t it = 0, ti = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++ti) {
            const uint32_t n0 = (tile / p.m_tiles) * kBN, m0 = (tile % p.m_tiles) * kBM;
            const uint32_t nrow = min(n0 + r, p.N - 1u);  // rows past N: read a valid row, never stored
            const uint16_t *srow = p.scales + static_cast<size_t>(nrow) * p.groups;
            const uint16_t *brow = p.biases + static_cast<size_t>(nrow) * p.groups;
            uint4 sv = make_uint4(0, 0, 0, 0), bv = make_uint4(0, 0, 0, 0);
            uint32_t have = 0xFFFFFFFFu;  // first group index held in sv / bv
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb, ++it) {
                const uint32_t stage = it % kStagesTc, par = (it / kStagesTc) & 1u;
                // scales / biases: eight consecutive groups per 16-byte load
                const uint32_t g_first = (kb * kBK) >> gshift;
                if ((g_first & ~7u) != have) {
                    have = g_first & ~7u;
                    sv = __ldg(reinterpret_cast<const uint4 *>(srow + have));
                    bv = __ldg(reinterpret_cast<const uint4 *>(brow + have));
                }
                if (!mbar_wait(smem_u32(&s_full[stage]), par, &s_abort, p.error_word, 0x1000u)) {
                    ok = false;
                    break;
                }
                const uint32_t sb = base + stage * kStageTc;
                const uint32_t prow = sb + 2 * kATile + kBTile + r * 32u;
                uint32_t w[8];
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(prow));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(prow + 16u));
                const uint32_t brow_s = sb + 2 * kATile + r * 128u;
                const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t gi = (kb * kBK + half * 32u) >> gshift;
                    const uint32_t s2u = pick_pair(sv, gi & 7u, p.sdtype), b2u = pick_pair(bv, gi & 7u, p.sdtype);
                    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&s2u);
                    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162 *>(&b2u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t word = w[half * 4 + j];
                        uint32_t pr[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) pr[i] = ((word >> (4 * i)) & 0x000F000Fu) | 0x43004300u;  // {128+q_i, 128+q_{i+4}}
                        // natural K order: {q0,q1} {q2,q3} {q4,q5} {q6,q7}
                        uint32_t nat[4] = {prmt(pr[0], pr[1], 0x5410u), prmt(pr[2], pr[3], 0x5410u),
                                           prmt(pr[0], pr[1], 0x7632u), prmt(pr[2], pr[3], 0x7632u)};
                        uint32_t o[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162 *>(&nat[i]);
                            v = __hsub2(v, k128);        // exact: the code itself
                            v = __hfma2(v, s2, b2);      // bf16(q * s + b), one rounding
                            o[i] = *reinterpret_cast<uint32_t *>(&v);
                        }
                        const uint32_t chunk = half * 4 + j;  // 16-byte chunk = 8 consecutive k
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(brow_s + (((chunk ^ r) & 7u) << 4)),
                                     "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                     : "memory");
                    }
                }
                // make the generic-proxy writes visible to the tensor core's reads, then signal
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_bready[stage]));
            }
            if (!ok) break;

            // ---- epilogue: accumulators -> bf16 -> y ----
            if (!mbar_wait(smem_u32(&s_acc_full), ti & 1u, &s_abort, p.error_word, 0x2000u)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t mrow = m0 + hsel * 128u + q * 32u + lane;
            __nv_bfloat16 *yrow = static_cast<__nv_bfloat16 *>(p.y) + static_cast<size_t>(mrow) * p.N;
#pragma unroll 1
            for (uint32_t c = 0; c < kBN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((q * 32u) << 16) + hsel * 256u + c * 32u, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const uint32_t col0 = n0 + c * 32u;
                if (mrow < p.M && col0 < p.N) {
                    if (col0 + 32u <= p.N && (p.N & 7u) == 0u) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 o;
                            __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
                            __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
                            __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
                            o.x = *reinterpret_cast<uint32_t *>(&t0);
                            o.y = *reinterpret_cast<uint32_t *>(&t1);
                            o.z = *reinterpret_cast<uint32_t *>(&t2);
                            o.w = *reinterpret_cast<uint32_t *>(&t3);
                            *reinterpret_cast<uint4 *>(yrow + col0 + 8 * i) = o;
                        }
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < p.N) yrow[col0 + i] = __float2bfloat16_rn(__uint_as_float(v[i]));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_acc_empty));
        }
    }

    // common exit: everybody meets, then the allocating warp returns tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

bool gemm_tc_eligible(const WeightView &w, uint32_t M) {
    if (M <= 16u) return false;                                   // the decode GEMV kernels take M <= 16
    if (w.bits != 4u) return false;
    if (w.group != 32u && w.group != 64u && w.group != 128u) return false;
    if (w.K % kBK != 0u || w.groups % 8u != 0u) return false;      // whole K blocks; 16-byte loads of scales
    if (w.row_bytes != w.K / 2u || w.row_bytes % 16u != 0u) return false;
    if (reinterpret_cast<uintptr_t>(w.packed) % 16u != 0 || reinterpret_cast<uintptr_t>(w.scales) % 16u != 0 ||
        reinterpret_cast<uintptr_t>(w.biases) % 16u != 0)
        return false;
    return encode_fn() != nullptr;
}

cudaError_t gemm_tc(const WeightView &w, const void *x_bf16, void *y_bf16, uint32_t M, cudaStream_t stream,
                    int sm_count, unsigned int *d_error_word) {
    if (!gemm_tc_eligible(w, M)) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(x_bf16) % 16u != 0 || reinterpret_cast<uintptr_t>(y_bf16) % 16u != 0 ||
        (static_cast<size_t>(w.K) * 2u) % 16u != 0)
        return cudaErrorNotSupported;
    EncodeTiledFn enc = encode_fn();
    CUtensorMap tmx, tmp;
    {
        const cuuint64_t dims[2] = {w.K, M};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w.K) * 2u};
        const cuuint32_t box[2] = {kBK, 128};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&tmx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x_bf16), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {w.row_bytes, w.N};
        const cuuint64_t strides[1] = {w.row_bytes};
        const cuuint32_t box[2] = {32, kBN};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.packed), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    GemmParams p;
    p.scales = w.scales;
    p.biases = w.biases;
    p.y = y_bf16;
    p.error_word = d_error_word;
    p.M = M;
    p.N = w.N;
    p.K = w.K;
    p.groups = w.groups;
    p.group = w.group;
    p.sdtype = w.sdtype;
    p.m_tiles = (M + kBM - 1u) / kBM;
    p.n_tiles = (w.N + kBN - 1u) / kBN;
    p.k_blocks = w.K / kBK;
    static bool configured[64] = {};  // per device: the opt-in belongs to the function on one device
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gaf_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    const uint32_t ctas = tiles < static_cast<uint32_t>(sm_count) ? tiles : static_cast<uint32_t>(sm_count);
    gaf_gemm_tc_kernel<<<ctas, kThreadsTc, kSmemTc, stream>>>(p, tmx, tmp);
    return cudaGetLastError();
}

}  // namespace tgaf
