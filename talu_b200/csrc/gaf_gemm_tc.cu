// Dequant-GEMM for grouped-affine weights on the 5th-generation tensor cores (M > 16).
//
//   y[M, N] (bf16) = x[M, K] (bf16) * W^T,  W[n, k] = q * scale + bias (gaf4 / gaf8, group 32 / 64 / 128)
//
// Replaces, for M > 16, the CPU 4x2 micro-kernel paths (core/src/compute/cpu/matmul_prefill.zig:121-358 for
// 4-bit codes, :572-759 for 8-bit codes) and the reference CUDA backend's loop of the matvec kernel over rows
// (core/src/inference/backend/cuda/engine.zig:4433-4473).
//
// One persistent CTA per SM.  A = activations (two 128-row halves of a 256-row tile when M > 128 and the codes
// are 4-bit; one half otherwise), B = 256 weight rows: D[128 x 256] in tensor memory per half.  Roles:
//   * warp 0 (one lane): TMA producer.  Per 64-deep K block it loads the activation tile (128-byte swizzle,
//     the layout the MMA descriptor names) into a stage of the ring; per 128 (or 64) packed bytes of K it loads
//     the packed codes of 256 weight rows into a ring of their own, which the dequant warps hand back.
//   * warps 2..17 (512 threads, half a weight row each): unpack the 32 codes of their half row, apply scale
//     and bias and write their 64 bytes of the K-major bf16 weight tile (same 128-byte swizzle) into the
//     stage.  4-bit codes with bf16 scales: the affine runs in bf16 (one fused multiply-add per pair, a
//     single rounding of q*s+b); 8-bit codes and f16 scales: fmaf(q, s, b) in fp32 (exact product), then one
//     rounding to bf16.  Scales and biases are fetched eight groups at a time, one fetch ahead of their use.
//     A waiting warp polls with one lane and backs off: polling by all 512 threads floods the pipeline that
//     the copy and MMA issuing threads go through too.
//   * warp 1 (one lane): issues tcgen05.mma (bf16 -> fp32, 128 x 256 x 16), accumulators in tensor memory, and
//     commits to the ring's mbarriers.  This thread is the pace-maker (a timeline of one CTA showed ~250 cycles
//     per mbarrier wait even when satisfied, ~100 per tcgen05 instruction, against 135 cycles of tensor work per
//     MMA), so per K block it waits ONCE (the dequant warps signal only after the activation tile has landed
//     too) and commits ONCE (activation tile and weight tile live in the same stage).  An earlier form with
//     the weights as the A operand for M <= 128 (tensor work proportional to M) needed twice as many MMA
//     instructions per K block and was slower for that reason alone.
//   * warps 2..17 again: read the accumulators back (tcgen05.ld), round to bf16 and store y.
//
// Work is dealt stream-K fashion: the (tile, K block) pairs of the whole problem, tile-major, are cut into
// equal contiguous ranges, one per CTA, so every SM gets the same number of K blocks whatever the tile count
// (a 70B-shaped o / down projection at M = 64 has 32 tiles; the prefill benchmark shape has 448 = 3.03 waves).
// A CTA whose range covers only part of a tile's K blocks either owns the tile (it holds K block 0: it gets
// there at the END of its range) or parks its fp32 partial tile in its workspace slot and raises a flag.  The
// owner adds the partials in CTA order (reproducible sums) and clears the flags.  A CTA writes at most one
// partial per launch, so the workspace is one tile per CTA.
//
// All waits (mbarriers, flags of other CTAs) are bounded; a wait that runs out sets the host-visible error
// word and a CTA-wide abort flag, every role then falls through to the common exit where tensor memory is
// released.
#include "gaf_internal.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tgaf {
namespace {

constexpr int kBN = 256;           // weight rows per tile
constexpr int kBK = 64;            // K block: 64 bf16 = 128 bytes, the swizzle span
constexpr int kMaxRing = 8;        // deepest ring
constexpr int kHalfTile = 128 * 128;  // 128 rows x 128 bytes
constexpr int kWTile = kBN * 128;     // 256 weight rows x 128 bytes of bf16
constexpr int kDequantWarps = 16;
constexpr int kFirstDequantWarp = 3;   // warps 0, 1, 2: activation copies, MMA issue, packed-code copies
constexpr int kThreadsTc = (kFirstDequantWarp + kDequantWarps) * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWaitLimitTc = 1u << 22;
// how long a thread may stay suspended inside one mbarrier.try_wait before it looks again (it is woken at once
// when the phase completes); an mbarrier wait as a whole gives up after four seconds
constexpr uint32_t kSuspendHintNs = 20000u;
constexpr unsigned long long kWaitLimitNs = 4000000000ull;
constexpr uint32_t kTileFloats = 256 * 256;   // workspace slot of one CTA (fp32 partial tile)

// Optional timeline of one CTA (debug builds with -DTGAF_GEMM_TRACE only): SM clock at the hand-over points of
// the first kTraceLen K blocks, read back by tgaf_debug_gemm_trace.
#ifdef TGAF_GEMM_TRACE
constexpr int kTraceLen = 256, kTraceRows = 12;
__device__ unsigned long long g_gemm_trace[kTraceRows][kTraceLen];
__device__ unsigned long long g_gemm_cta[160][8];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TGAF_CTA(slot) g_gemm_cta[blockIdx.x < 160u ? blockIdx.x : 159u][slot] = gtime()
#define TGAF_TRACE(row, idx)                                                                    \
    do {                                                                                        \
        if (blockIdx.x == 1u && (idx) < static_cast<uint32_t>(kTraceLen)) g_gemm_trace[row][idx] = clock64(); \
    } while (0)
#else
#define TGAF_CTA(slot) \
    do {               \
    } while (0)
#define TGAF_TRACE(row, idx) \
    do {                     \
    } while (0)
#endif

struct GemmParams {
    const uint16_t *scales;
    const uint16_t *biases;
    void *y;
    float *ws;              // [ctas][kTileFloats] partial tiles
    unsigned int *flags;    // [ctas][kDequantWarps], zero between launches
    unsigned int *error_word;
    uint32_t M, N, K;
    uint32_t groups;   // K / G
    uint32_t group;    // G
    uint32_t sdtype;   // 1 bf16, 0 f16
    uint32_t m_tiles, n_tiles, k_blocks;
    uint32_t bm;            // activation rows per tile: 256 or 128
    uint32_t x_bytes;       // activation bytes per stage
    uint32_t x_stages, p_stages, w_stages;   // depths of the activation, packed-code and weight-tile rings
    uint32_t p_row;         // packed bytes per row and packed stage: 128 (swizzled; 4 or 2 K blocks) or 64
    uint32_t total_units;   // tiles * k_blocks
    uint32_t wait_limit;    // polls for another CTA's flag
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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait that also gives up once another role has raised the abort flag.  Every lane waits in the
// try_wait itself (which suspends the thread in hardware until the phase completes or a time-out): a version
// that polled with one lane and slept between polls lost more in wake-up latency at each hand-over of the
// pipeline (three or four per K block) than it saved in polling traffic.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                               unsigned int *error_word, uint32_t code) {
    unsigned long long t0 = 0ull;
    for (uint32_t it = 0; it < kWaitLimitTc; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0ull) t0 = now;
            else if (now - t0 > kWaitLimitNs) break;
        }
    }
    atomicOr(error_word, code);
    *abort_flag = 1u;
    return false;
}
// One lane of a converged warp.  The copy and MMA issuing warps run their loops with all lanes, so that ring
// positions, addresses and descriptors are warp-uniform values (the compiler keeps them in uniform registers, which
// is where tcgen05 and TMA instructions take their operands from), and only the issuing instruction is elected.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0u;
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
// bf16 x bf16 -> f32, both operands K-major, M = 128, N = n (a multiple of 16, 16..256)
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the accumulate flag fixed to "add to the accumulator"
__device__ __forceinline__ void umma_f16_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc)
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

__device__ __forceinline__ float sb_f32(uint32_t raw, uint32_t sdtype) {
    // core/src/compute/cuda/kernels/ops/common_decode.cuh:1-13
    if (sdtype == 0u) return __half2float(__ushort_as_half(static_cast<unsigned short>(raw)));
    return __uint_as_float(raw << 16);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// contiguous, near-equal unit ranges: the first `rem` CTAs take one unit more
__device__ __forceinline__ uint32_t range_begin(uint32_t cta, uint32_t units, uint32_t ctas) {
    const uint32_t q = units / ctas, rem = units % ctas;
    return cta * q + (cta < rem ? cta : rem);
}
__device__ __forceinline__ uint32_t unit_owner(uint32_t u, uint32_t units, uint32_t ctas) {
    const uint32_t q = units / ctas, rem = units % ctas;
    const uint32_t cut = rem * (q + 1u);
    return u < cut ? u / (q + 1u) : rem + (u - cut) / q;
}

// Position in a ring of `n` stages with the mbarrier phase parity of the current pass; advanced without a
// division (the ring depths are run-time values).
struct RingPos {
    uint32_t stage, parity;
    __device__ __forceinline__ void advance(uint32_t n) {
        if (++stage == n) stage = 0u, parity ^= 1u;
    }
};

// A CTA's range as segments: maximal runs of K blocks inside one tile.
struct Segment {
    uint32_t tile, kb0, kb1;
};
__device__ __forceinline__ Segment segment_at(uint32_t u, uint32_t u_end, uint32_t k_blocks) {
    Segment s;
    s.tile = u / k_blocks;
    s.kb0 = u - s.tile * k_blocks;
    const uint32_t left = u_end - u;
    s.kb1 = s.kb0 + left < k_blocks ? s.kb0 + left : k_blocks;
    return s;
}

// BITS: code width.  FAST: bf16 scales on 4-bit codes (affine in bf16).
template <int BITS, bool FAST>
__global__ void __launch_bounds__(kThreadsTc, 1)
gaf_gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_p) {
    static_assert(!FAST || BITS == 4, "the bf16 affine is for 4-bit codes");
    constexpr uint32_t kRowPacked = kBK * BITS / 8;  // packed bytes per weight row and K block: 32 or 64
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_xfull[kMaxRing];     // TMA landed (activation tile)
    __shared__ __align__(8) uint64_t s_pfull[kMaxRing];     // TMA landed (packed codes)
    __shared__ __align__(8) uint64_t s_pempty[kMaxRing];    // every dequant warp has read the packed codes
    __shared__ __align__(8) uint64_t s_wready[kMaxRing];    // weight tile dequantized AND its activation tile landed
    __shared__ __align__(8) uint64_t s_wempty[kMaxRing];    // the MMAs that read the weight tile AND the activation tile of the same K block have completed
    __shared__ __align__(8) uint64_t s_acc_full;            // all MMAs of the segment have completed
    __shared__ __align__(8) uint64_t s_acc_empty;           // accumulators have been read back
    __shared__ uint32_t s_tmem_base;
    __shared__ volatile uint32_t s_abort;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t kPacked = kBN * p.p_row;                        // a packed stage: the codes of `kpp` K blocks
    const uint32_t kpp = p.p_row / kRowPacked;
    const bool pswz = p.p_row == 128u;                             // 128-byte packed rows are swizzled like the operand tiles
    const uint32_t NX = p.x_stages, NP = p.p_stages, NW = p.w_stages;
    const uint32_t xring = base;                                   // activation tiles,
    const uint32_t wring = xring + NX * p.x_bytes;                 // then weight tiles,
    const uint32_t pring = wring + NW * kWTile;                    // then packed codes

    if (threadIdx.x == 0) {
        s_abort = 0u;
        for (uint32_t s = 0; s < NX; ++s) {
            mbar_init(smem_u32(&s_xfull[s]), 1);
        }
        for (uint32_t s = 0; s < NP; ++s) {
            mbar_init(smem_u32(&s_pfull[s]), 1);
            mbar_init(smem_u32(&s_pempty[s]), kDequantWarps);
        }
        for (uint32_t s = 0; s < NW; ++s) {
            mbar_init(smem_u32(&s_wready[s]), kDequantWarps / 2);
            mbar_init(smem_u32(&s_wempty[s]), 1);
        }
        mbar_init(smem_u32(&s_acc_full), 1);
        mbar_init(smem_u32(&s_acc_empty), kDequantWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // tensor memory: all 512 columns; this warp also frees them
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;
    if (threadIdx.x == 0) TGAF_TRACE(10, 0u);
    if (threadIdx.x == 0) TGAF_CTA(0);

    const uint32_t u_begin = range_begin(blockIdx.x, p.total_units, gridDim.x);
    const uint32_t u_end = range_begin(blockIdx.x + 1u, p.total_units, gridDim.x);
    // tile -> first weight row and first activation row (tiles are walked weight-tile major so that CTAs
    // running at the same time share weight rows in L2)
    auto tile_n0 = [&](uint32_t tile) { return (tile / p.m_tiles) * static_cast<uint32_t>(kBN); };
    auto tile_m0 = [&](uint32_t tile) { return (tile % p.m_tiles) * p.bm; };

    if (warp == 0 || warp == 2) {
        // ---------------- TMA producers (whole warp, elected issue): warp 0 activations, warp 2 packed codes ----------------
        // Each runs as far ahead as its own ring allows: the codes (the only HBM traffic when M is small) up to
        // eight K blocks, so that neither copy latency is part of the dequantize -> MMA -> free cycle.
        const bool codes = warp == 2;
        const uint32_t n_stages = codes ? NP : NX;
        // the activation ring is as deep as the weight ring and shares its "free" barriers: one commit per K block
        uint64_t *fullb = codes ? s_pfull : s_xfull, *emptyb = codes ? s_pempty : s_wempty;
        if (lane == 0)
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(codes ? &tmap_p : &tmap_x)) : "memory");
        uint32_t it = 0;
        RingPos rp = {0u, 0u};
        bool ok = true;
        for (uint32_t u = u_begin; u < u_end && ok;) {
            const Segment sg = segment_at(u, u_end, p.k_blocks);
            const uint32_t n0 = tile_n0(sg.tile), m0 = tile_m0(sg.tile);
            for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb) {
                // a packed stage holds the codes of `kpp` K blocks: one copy per stage, at its first K block
                if (codes && kb != sg.kb0 && kb % kpp != 0u) continue;
                // from the second pass over the ring on, a stage is refilled once its readers are done with it
                if (it >= n_stages && !mbar_wait_warp(smem_u32(&emptyb[rp.stage]), rp.parity ^ 1u, &s_abort, p.error_word, codes ? 0x80u : 0x100u)) {
                    ok = false;
                    break;
                }
                const uint32_t full = smem_u32(&fullb[rp.stage]);
                if (elect_one()) {
                    if (codes) {
                        mbar_arrive_expect_tx(full, kPacked);  // out-of-range rows arrive as zeros
                        tma_load_2d(pring + rp.stage * kPacked, &tmap_p, (kb - kb % kpp) * kRowPacked, n0, full);
                    } else {
                        TGAF_TRACE(0, it);
                        const uint32_t sb = xring + rp.stage * p.x_bytes;
                        mbar_arrive_expect_tx(full, p.x_bytes);
                        tma_load_2d(sb, &tmap_x, kb * kBK, m0, full);
                        if (p.bm > 128u) tma_load_2d(sb + kHalfTile, &tmap_x, kb * kBK, m0 + 128u, full);
                    }
                }
                __syncwarp();
                ++it;
                rp.advance(n_stages);
            }
            u += sg.kb1 - sg.kb0;
        }
        if (!ok && lane == 0) {
            // copies already issued get a bounded time to land before shared memory is released (error path:
            // the divisions do not matter here)
            const uint32_t pending = it < n_stages ? it : n_stages;
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t idx = it - 1u - i;
                for (uint32_t spin = 0; spin < (1u << 20); ++spin)
                    if (mbar_try_wait(smem_u32(&fullb[idx % n_stages]), (idx / n_stages) & 1u)) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // Measured on this part: every instruction of this one thread is expensive (a satisfied mbarrier wait
        // ~250 cycles, a tcgen05.mma ~100 to issue, a commit ~100) against 135 cycles of tensor work per
        // 128 x 256 x 16 MMA, so it does the minimum per K block: ONE wait (the dequant warps arrive only after
        // the activation tile has landed too), the MMAs, ONE commit (activation and weight tile share a stage).
        {
            uint32_t si = 0, mit = 0;
            RingPos xp = {0u, 0u}, wp = {0u, 0u};
            bool ok = true;
            const uint32_t idesc = instr_desc(static_cast<uint32_t>(kBN));
            // descriptors differ from stage to stage in the address field (16-byte units) only
            const uint64_t xd0 = umma_desc_sw128(xring), wd0 = umma_desc_sw128(wring);
            const uint32_t x_step = p.x_bytes >> 4, w_step = kWTile >> 4;
            for (uint32_t u = u_begin; u < u_end && ok; ++si) {
                const Segment sg = segment_at(u, u_end, p.k_blocks);
                if (si > 0 && !mbar_wait_warp(smem_u32(&s_acc_empty), (si - 1u) & 1u, &s_abort, p.error_word, 0x200u)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // the second accumulator (activation rows 128.. of the tile) exists only when the tile reaches it
                const bool second = p.bm > 128u && tile_m0(sg.tile) + 128u < p.M;
                for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb, xp.advance(NX), wp.advance(NW)) {
                    if (lane == 0) TGAF_TRACE(1, mit);
                    if (!mbar_wait_warp(smem_u32(&s_wready[wp.stage]), wp.parity, &s_abort, p.error_word, 0x800u)) {
                        ok = false;
                        break;
                    }
                    if (lane == 0) TGAF_TRACE(2, mit);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t xd = xd0 + xp.stage * x_step, wd = wd0 + wp.stage * w_step;
                    const uint32_t wfree = smem_u32(&s_wempty[wp.stage]);
                    if (elect_one()) {
                        TGAF_TRACE(4, mit);
                        // advancing 16 elements (32 bytes) along K inside the swizzle span: +2 in the address field;
                        // the second 128-row half of the activation tile lies 16 KB further: +1024
                        const uint32_t acc0 = kb > sg.kb0 ? 1u : 0u;
                        umma_f16(tmem_base, xd, wd, idesc, acc0);
                        if (second) umma_f16(tmem_base + 256u, xd + 1024, wd, idesc, acc0);
                        TGAF_TRACE(8, mit);
#pragma unroll
                        for (uint32_t k16 = 1; k16 < kBK / 16; ++k16) {
                            umma_f16_acc(tmem_base, xd + 2 * k16, wd + 2 * k16, idesc);
                            if (second) umma_f16_acc(tmem_base + 256u, xd + 1024 + 2 * k16, wd + 2 * k16, idesc);
                        }
                        TGAF_TRACE(9, mit);
                        umma_commit(wfree);  // frees the activation tile and the weight tile once these MMAs have read them
                        TGAF_TRACE(3, mit);
                    }
                    __syncwarp();
                    ++mit;
                }
                if (ok && elect_one()) umma_commit(smem_u32(&s_acc_full));
                __syncwarp();
                u += sg.kb1 - sg.kb0;
            }
        }
    } else {
        // ------------------------------ dequant + epilogue warps ------------------------------
        const uint32_t wi = warp - kFirstDequantWarp;   // 0..15
        const uint32_t r = (wi & 7u) * 32 + lane;   // weight row of the tile this thread dequantizes
        // Two groups of eight warps take alternate K blocks.  What a warp spends per K block is mostly latency
        // (shared-memory round trips, the proxy fence, the barrier hand-overs: ~900 cycles whether it unpacks 32 or
        // 64 codes per thread), so two K blocks in flight in the dequant stage double its throughput.
        const uint32_t grp = wi >> 3;
        const uint32_t q = warp & 3;                // tensor-memory lane quadrant this warp may read
        const uint32_t hsel = (wi >> 2) & 1u;       // accumulator this warp writes out ...
        const uint32_t cfirst = wi >> 3;            // ... and its 32-column chunks: cfirst, cfirst + 2, ...
        const uint32_t gshift = p.group == 32u ? 5u : (p.group == 64u ? 6u : 7u);
        uint32_t it = 0, si = 0;
        RingPos xp = {0u, 0u}, pp = {0u, 0u}, wp = {0u, 0u};
        bool ok = true;
        // this thread's fixed offsets: its packed bytes inside a packed stage, its row of a weight tile (whose 16-byte
        // chunks are swizzled: chunk index XOR (row & 7))
        const uint32_t prow_off = r * p.p_row;
        const uint32_t wrow_off = r * 128u;
        const uint32_t rx = (r & 7u) << 4;
        for (uint32_t u = u_begin; u < u_end && ok; ++si) {
            const Segment sg = segment_at(u, u_end, p.k_blocks);
            const uint32_t n0 = tile_n0(sg.tile), m0 = tile_m0(sg.tile);
            const uint32_t nrow = min(n0 + r, p.N - 1u);  // rows past N: read a valid row, never stored
            const uint16_t *srow = p.scales + static_cast<size_t>(nrow) * p.groups;
            const uint16_t *brow = p.biases + static_cast<size_t>(nrow) * p.groups;
            // scales / biases of eight consecutive groups per 16-byte load; the next eight are fetched as soon as
            // these come into use, so that no load is waited for
            uint4 sv = make_uint4(0, 0, 0, 0), bv = make_uint4(0, 0, 0, 0), sv_n = sv, bv_n = bv;
            uint32_t have = 0xFFFFFFFFu, have_n = 0xFFFFFFFFu;  // first group index held in sv / bv and in sv_n / bv_n
            uint32_t sub = sg.kb0 % kpp;   // K block inside its packed stage
            bool p_waited = false;         // this warp has seen the current packed stage land
            for (uint32_t kb = sg.kb0; kb < sg.kb1; ++kb, ++it, xp.advance(NX), wp.advance(NW)) {
                const bool mine = (it & 1u) == grp;   // else: the other group's K block
                const uint32_t g_first = (kb * kBK) >> gshift;
                if (mine) {
                if ((g_first & ~7u) != have) {
                    have = g_first & ~7u;
                    if (have == have_n) {
                        sv = sv_n, bv = bv_n;
                    } else {
                        sv = __ldg(reinterpret_cast<const uint4 *>(srow + have));
                        bv = __ldg(reinterpret_cast<const uint4 *>(brow + have));
                    }
                    have_n = have + 8u;
                    if (have_n < p.groups) {
                        sv_n = __ldg(reinterpret_cast<const uint4 *>(srow + have_n));
                        bv_n = __ldg(reinterpret_cast<const uint4 *>(brow + have_n));
                    }
                }
                if (wi == 0 && lane == 0) TGAF_TRACE(5, it);
                // the codes have landed, and the MMAs that read the previous contents of the weight tile are done
                if ((!p_waited && !mbar_wait_warp(smem_u32(&s_pfull[pp.stage]), pp.parity, &s_abort, p.error_word, 0x1000u)) ||
                    (it >= NW && !mbar_wait_warp(smem_u32(&s_wempty[wp.stage]), wp.parity ^ 1u, &s_abort, p.error_word, 0x8000u))) {
                    ok = false;
                    break;
                }
                p_waited = true;
                if (wi == 0 && lane == 0) TGAF_TRACE(6, it);
                const uint32_t pb = pring + pp.stage * kPacked, sb = wring + wp.stage * kWTile;
                uint32_t w[kRowPacked / 4];
#pragma unroll
                for (int i = 0; i < static_cast<int>(kRowPacked / 16); ++i) {
                    const uint32_t chunk = sub * (kRowPacked / 16) + i;   // 16-byte chunk of the packed row
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3])
                                 : "r"(pb + prow_off + ((pswz ? ((chunk ^ r) & 7u) : chunk) << 4)));
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t gi = (kb * kBK + half * 32u) >> gshift;
                    // the 16-bit value number (gi & 7) of sv / bv, already doubled into both halves of a register
                    const uint32_t sel = 0x1010u + 0x2222u * (gi & 3u);
                    const uint32_t s2u = prmt((gi & 4u) ? sv.z : sv.x, (gi & 4u) ? sv.w : sv.y, sel);
                    const uint32_t b2u = prmt((gi & 4u) ? bv.z : bv.x, (gi & 4u) ? bv.w : bv.y, sel);
                    if constexpr (FAST) {
                        const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&s2u);
                        const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162 *>(&b2u);
                        const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t word = w[half * 4 + j];
                            // byte i of `word` holds code 2i in its low nibble; byte i of `word >> 4` holds code 2i + 1
                            // there: one byte permute and one mask-or per pair of consecutive codes
                            const uint32_t wsh = word >> 4;
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t pr = (prmt(word, wsh, 0x0400u + 0x0101u * i) & 0x000F000Fu) | 0x43004300u;
                                __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162 *>(&pr);  // {128 + q[2i], 128 + q[2i+1]}
                                v = __hsub2(v, k128);        // exact: the code itself
                                v = __hfma2(v, s2, b2);      // bf16(q * s + b), one rounding
                                o[i] = *reinterpret_cast<uint32_t *>(&v);
                            }
                            const uint32_t chunk = half * 4 + j;  // 16-byte chunk = 8 consecutive k
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sb + wrow_off + ((chunk << 4) ^ rx)), "r"(o[0]),
                                         "r"(o[1]), "r"(o[2]), "r"(o[3])
                                         : "memory");
                        }
                    } else {
                        const float s = sb_f32(s2u & 0xFFFFu, p.sdtype), b = sb_f32(b2u & 0xFFFFu, p.sdtype);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float f[8];
                            if constexpr (BITS == 4) {
                                const uint32_t word = w[half * 4 + j];
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    f[i] = __uint_as_float(0x4B000000u | ((word >> (4 * i)) & 0xFu)) - 8388608.f;   // exact q
                            } else {
                                const uint32_t w0 = w[half * 8 + 2 * j], w1 = w[half * 8 + 2 * j + 1];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    f[i] = __uint_as_float(prmt(w0, 0x4B000000u, 0x7650u + i)) - 8388608.f;
                                    f[4 + i] = __uint_as_float(prmt(w1, 0x4B000000u, 0x7650u + i)) - 8388608.f;
                                }
                            }
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)  // fmaf(q, s, b) exactly as the reference dequant, then one rounding to bf16
                                o[i] = pack_bf16x2(fmaf(f[2 * i], s, b), fmaf(f[2 * i + 1], s, b));
                            const uint32_t chunk = half * 4 + j;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sb + wrow_off + ((chunk << 4) ^ rx)), "r"(o[0]),
                                         "r"(o[1]), "r"(o[2]), "r"(o[3])
                                         : "memory");
                        }
                    }
                }
                // make the generic-proxy writes visible to the tensor core's reads, then signal; the first dequant
                // warp signals only once the K block's activation tile has landed as well, so that the MMA warp
                // has a single barrier to wait for
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if ((wi & 7u) == 0u && !mbar_wait_warp(smem_u32(&s_xfull[xp.stage]), xp.parity, &s_abort, p.error_word, 0x400u)) {
                    ok = false;
                    break;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_wready[wp.stage]));
                if (wi == 0 && lane == 0) TGAF_TRACE(7, it);
                }  // mine
                if (++sub == kpp || kb + 1u == sg.kb1) {
                    // last K block of the packed stage (or of the segment): every warp hands the stage back, whether or
                    // not its group had a K block in it
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&s_pempty[pp.stage]));
                    pp.advance(NP);
                    sub = 0u;
                    p_waited = false;
                }
            }
            if (!ok) break;

            // ---- the segment's accumulators: to y, to the workspace, or to y together with the others' ----
            if (wi == 0 && lane == 0) TGAF_TRACE(10, 1u + 4u * si);
            if (wi == 0 && lane == 0 && si < 3u) TGAF_CTA(1 + 2 * si);
            if (!mbar_wait_warp(smem_u32(&s_acc_full), si & 1u, &s_abort, p.error_word, 0x2000u)) break;
            if (wi == 0 && lane == 0) TGAF_TRACE(10, 2u + 4u * si);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool whole = sg.kb0 == 0u && sg.kb1 == p.k_blocks;
            const bool owner = sg.kb0 == 0u;
            const bool acc_live = hsel == 0u || (p.bm > 128u && m0 + 128u < p.M);
            // partial tiles of the CTAs after this one that hold the rest of the tile's K blocks
            uint32_t last_cta = blockIdx.x;
            bool peers_ok = true;
            if (owner && !whole) {
                last_cta = unit_owner(sg.tile * p.k_blocks + p.k_blocks - 1u, p.total_units, gridDim.x);
                for (uint32_t c = blockIdx.x + 1u; c <= last_cta && peers_ok; ++c) {
                    const unsigned int *flag = p.flags + c * kDequantWarps + wi;
                    bool got = false;
                    if (lane == 0) {
                        for (uint32_t spin = 0; spin < p.wait_limit; ++spin) {
                            unsigned int v;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                            if (v != 0u) {
                                got = true;
                                break;
                            }
                            if (s_abort) break;
                            __nanosleep(spin > 4096 ? 256 : 64);
                        }
                    }
                    got = __shfl_sync(0xFFFFFFFFu, got ? 1u : 0u, 0) != 0u;   // the warp barrier also orders the others' reads
                    if (!got) {
                        if (lane == 0) atomicOr(p.error_word, 0x4000u);
                        s_abort = 1u;
                        peers_ok = false;
                    }
                }
            }
            float *my_ws = p.ws + static_cast<size_t>(blockIdx.x) * kTileFloats;
            if (wi == 0 && lane == 0) TGAF_TRACE(10, 3u + 4u * si);
            if (acc_live && peers_ok) {
#pragma unroll 1
                for (uint32_t c = cfirst; c < kBN / 32u; c += 2u) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((q * 32u) << 16) + hsel * 256u + c * 32u, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // workspace layout: [accumulator][chunk][column quad 0..7][128 lanes] of float4, so that the 32
                    // lanes of a warp read and write 512 contiguous bytes per instruction
                    const size_t slot = (((static_cast<size_t>(hsel) * 8u + c) * 8u) * 128u + q * 32u + lane) * 4u;
                    if (!owner) {
                        float4 *dst = reinterpret_cast<float4 *>(my_ws + slot);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            dst[i * 128] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                        continue;
                    }
                    // CTA order: reproducible sums; two peers' loads in flight at a time
                    for (uint32_t pc = blockIdx.x + 1u; pc <= last_cta; pc += 2u) {
                        const float4 *src0 = reinterpret_cast<const float4 *>(p.ws + static_cast<size_t>(pc) * kTileFloats + slot);
                        const bool two = pc + 1u <= last_cta;
                        const float4 *src1 = two ? src0 + kTileFloats / 4u : src0;
                        float4 t0[8], t1[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) t0[i] = __ldcg(src0 + i * 128);
#pragma unroll
                        for (int i = 0; i < 8; ++i) t1[i] = two ? __ldcg(src1 + i * 128) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[4 * i] = __float_as_uint((__uint_as_float(v[4 * i]) + t0[i].x) + t1[i].x);
                            v[4 * i + 1] = __float_as_uint((__uint_as_float(v[4 * i + 1]) + t0[i].y) + t1[i].y);
                            v[4 * i + 2] = __float_as_uint((__uint_as_float(v[4 * i + 2]) + t0[i].z) + t1[i].z);
                            v[4 * i + 3] = __float_as_uint((__uint_as_float(v[4 * i + 3]) + t0[i].w) + t1[i].w);
                        }
                    }
                    const uint32_t mrow = m0 + hsel * 128u + q * 32u + lane;
                    __nv_bfloat16 *yrow = static_cast<__nv_bfloat16 *>(p.y) + static_cast<size_t>(mrow) * p.N;
                    const uint32_t col0 = n0 + c * 32u;
                    if (mrow < p.M && col0 < p.N) {
                        if (col0 + 32u <= p.N && (p.N & 7u) == 0u) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
                                o.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
                                o.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
                                o.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
                                *reinterpret_cast<uint4 *>(yrow + col0 + 8 * i) = o;
                            }
                        } else {
                            for (int i = 0; i < 32; ++i)
                                if (col0 + i < p.N) yrow[col0 + i] = __float2bfloat16_rn(__uint_as_float(v[i]));
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&s_acc_empty));
                if (!owner) {
                    // this warp's share of the partial tile is in the workspace: raise its flag
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + blockIdx.x * kDequantWarps + wi), "r"(1u) : "memory");
                } else if (!whole && peers_ok) {
                    for (uint32_t c = blockIdx.x + 1u; c <= last_cta; ++c)  // consumed: ready for the next launch
                        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.flags + c * kDequantWarps + wi), "r"(0u) : "memory");
                }
            }
            if (!peers_ok) break;
            if (wi == 0 && lane == 0) TGAF_TRACE(10, 4u + 4u * si);
            if (wi == 0 && lane == 0 && si < 3u) TGAF_CTA(2 + 2 * si);
            u += sg.kb1 - sg.kb0;
        }
    }
    if (threadIdx.x == 0) TGAF_TRACE(11, 0u);
    if (threadIdx.x == 0) TGAF_CTA(7);

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

template <int BITS, bool FAST>
cudaError_t launch_gemm(const GemmParams &p, const CUtensorMap &tmx, const CUtensorMap &tmp, uint32_t ctas, int smem,
                        cudaStream_t stream) {
    auto kern = gaf_gemm_tc_kernel<BITS, FAST>;
    static int configured[64] = {};  // per device: the largest opt-in made for this instance
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    kern<<<ctas, kThreadsTc, smem, stream>>>(p, tmx, tmp);
    return cudaGetLastError();
}

}  // namespace

#ifdef TGAF_GEMM_TRACE
extern "C" int tgaf_debug_gemm_cta(unsigned long long *out) {
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemm_cta, sizeof(unsigned long long) * 160 * 8));
}
extern "C" int tgaf_debug_gemm_trace(unsigned long long *out) {
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemm_trace, sizeof(unsigned long long) * kTraceRows * kTraceLen));
}
#endif

size_t gemm_tc_workspace_bytes(int sm_count) { return static_cast<size_t>(sm_count) * kTileFloats * sizeof(float); }
size_t gemm_tc_flag_count(int sm_count) { return static_cast<size_t>(sm_count) * kDequantWarps; }

bool gemm_tc_eligible(const WeightView &w, uint32_t M, uint32_t min_m) {
    if (M < min_m) return false;                                  // the decode GEMV kernels take the rows below
    if (w.bits != 4u && w.bits != 8u) return false;
    if (w.group != 32u && w.group != 64u && w.group != 128u) return false;
    if (w.K % kBK != 0u || w.groups % 8u != 0u) return false;      // whole K blocks; 16-byte loads of scales
    if (w.row_bytes != w.K * w.bits / 8u || w.row_bytes % 16u != 0u) return false;
    if (reinterpret_cast<uintptr_t>(w.packed) % 16u != 0 || reinterpret_cast<uintptr_t>(w.scales) % 16u != 0 ||
        reinterpret_cast<uintptr_t>(w.biases) % 16u != 0)
        return false;
    return encode_fn() != nullptr;
}

cudaError_t gemm_tc(const WeightView &w, const void *x_bf16, void *y_bf16, uint32_t M, cudaStream_t stream,
                    int sm_count, unsigned int *d_error_word, float *ws, size_t ws_bytes, unsigned int *flags,
                    size_t flag_count) {
    if (!gemm_tc_eligible(w, M, 1u)) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(x_bf16) % 16u != 0 || reinterpret_cast<uintptr_t>(y_bf16) % 16u != 0 ||
        (static_cast<size_t>(w.K) * 2u) % 16u != 0)
        return cudaErrorNotSupported;
    if (!ws || !flags || ws_bytes < gemm_tc_workspace_bytes(sm_count) || flag_count < gemm_tc_flag_count(sm_count))
        return cudaErrorMemoryAllocation;
    EncodeTiledFn enc = encode_fn();
    GemmParams p;
    p.scales = w.scales;
    p.biases = w.biases;
    p.y = y_bf16;
    p.ws = ws;
    p.flags = flags;
    p.error_word = d_error_word;
    p.M = M;
    p.N = w.N;
    p.K = w.K;
    p.groups = w.groups;
    p.group = w.group;
    p.sdtype = w.sdtype;
    p.n_tiles = (w.N + kBN - 1u) / kBN;
    p.k_blocks = w.K / kBK;
    // two activation halves per tile when there are rows for them and the ring still gets three stages
    p.bm = (M > 128u && w.bits == 4u) ? 256u : 128u;
    p.m_tiles = (M + p.bm - 1u) / p.bm;
    p.x_bytes = p.bm * 128u;
    // 227 KB per CTA, minus the static part and the slack that aligns the rings = 225 KB.  Three weight tiles
    // (96 KB) cover the dequantize -> MMA -> free cycle, with as many activation stages (48 or 96 KB).  With one
    // activation half: two packed stages of 128-byte rows (64 KB: the codes are fetched as full 128-byte lines,
    // four K blocks of 4-bit codes per row at once); with two halves: two packed stages of 64-byte rows (32 KB).
    p.w_stages = 3u;
    p.x_stages = 3u;   // = w_stages: the two rings share their "free" barriers
    p.p_stages = 2u;
    p.p_row = p.bm > 128u ? 64u : 128u;
    p.total_units = p.m_tiles * p.n_tiles * p.k_blocks;
    p.wait_limit = kWaitLimitTc;
    const int smem = static_cast<int>(p.w_stages * kWTile + p.x_stages * p.x_bytes + p.p_stages * kBN * p.p_row + 1024u);
    if (smem > 226 * 1024) return cudaErrorNotSupported;

    CUtensorMap tmx, tmp;
    {
        const cuuint64_t dims[2] = {w.K, M};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(w.K) * 2u};
        const cuuint32_t box[2] = {kBK, 128u};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&tmx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x_bf16), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {w.row_bytes, w.N};
        const cuuint64_t strides[1] = {w.row_bytes};
        const cuuint32_t box[2] = {p.p_row, kBN};   // p_row bytes of every row: the codes of several K blocks at once
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&tmp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.packed), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, p.p_row == 128u ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const uint32_t ctas = p.total_units < static_cast<uint32_t>(sm_count) ? p.total_units : static_cast<uint32_t>(sm_count);
    if (w.bits == 4u)
        return w.sdtype == 1u ? launch_gemm<4, true>(p, tmx, tmp, ctas, smem, stream)
                              : launch_gemm<4, false>(p, tmx, tmp, ctas, smem, stream);
    return launch_gemm<8, false>(p, tmx, tmp, ctas, smem, stream);
}

}  // namespace tgaf
