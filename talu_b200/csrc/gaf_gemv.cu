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
// Instruction budget.  At HBM rate a B200 SM must retire ~40 weights per clock,
// which leaves no room for an int->float convert and an FMA per weight on the
// CUDA cores.  So the codes go through the tensor cores as exact small integers:
//   * a packed word is split with four (shift, and, or) steps into bf16x2 pairs
//     0x4300|q, i.e. the bf16 value 128+q (exact for q < 128);
//   * warp-level mma.sync m16n8k16 (bf16 x bf16 -> f32) multiplies 16 weight rows
//     by up to 8 activation rows; the k order inside a fragment is free, so the
//     canonical [N, K/8] u32 layout is consumed as is and the activations are
//     permuted to match with byte-permutes;
//   * a second MMA with an all-ones A operand yields sum_k x[m,k] per group in
//     the accumulators' register layout;
//   * per group: y += s*acc + (b - 128 s) * xsum, in fp32.
// 8-bit codes reuse all of it: a byte is two nibbles, q = lo + 16 hi, and 16 x is
// exact in bf16, so a gaf8 row is a gaf4 row of twice the length against the
// activation vector (x0, 16 x0, x1, 16 x1, ...).
// f32 activations are split into bf16 hi + lo parts (two MMAs), which keeps ~16
// mantissa bits of x.
//
// Data movement.  A persistent grid (one CTA per SM) walks "units" of
// 128 weight rows x 256 packed bytes.  A producer thread streams each unit into a
// 3-deep shared-memory ring with two TMA tensor copies (128 rows x 128 bytes each,
// 128-byte swizzle) that complete on an mbarrier, so the weights never pass
// through the load/store units on their way in and ~100 KB per SM can be in
// flight.  Eight consumer warps each own 16 of the 128 rows: they read their rows
// from the ring with 4/8/16-byte shared loads, take scales / biases for the whole
// unit with one vector load per row, and read activations through L1.  No warp
// ever exchanges data with another warp of the CTA.
// The MMA fixes which lanes hold which row (lane / 4) but not which weight row
// that is, so each warp permutes its rows such that the lanes of one shared-load
// wavefront touch rows whose swizzle patterns do not collide (rho below): the
// fragment loads are bank-conflict free on the swizzled tile.
//
// Units are dealt to CTAs as equal contiguous ranges (row group major, K chunk
// minor), so a row group can be shared by neighbouring CTAs.  Each warp then
// parks its fp32 partial in a scratch slot and bumps a per-(row group, warp)
// arrival counter; whoever arrives last adds the slots in slot order and writes
// y (nobody spins; counters reset themselves).
//
// Every wait on an mbarrier has an iteration limit; a warp that runs out sets an
// error word for the host and leaves.
//
// Programmatic dependent launch: the producer starts copying weights at once
// (they never change), consumers execute griddepcontrol.wait before they touch
// activations, outputs or scratch, so back-to-back GEMVs overlap tail and head.
#include "gaf_internal.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <type_traits>

namespace tgaf {
namespace {

constexpr uint32_t kMagic128 = 0x43004300u;  // bf16x2 {128, 128}
constexpr uint32_t kOnesBf16 = 0x3F803F80u;  // bf16x2 {1, 1}
constexpr uint32_t kNibMask = 0x000F000Fu;

constexpr int kRows = 128;        // weight rows per unit (8 consumer warps x 16)
constexpr int kChunkBytes = 256;  // packed bytes per row per unit
constexpr int kStages = 3;
constexpr int kRowBlocks = 8;      // 16-row blocks per unit
constexpr int kConsumerWarps = 16;  // two K halves x eight row blocks
constexpr int kThreads = (kConsumerWarps + 2) * 32;  // + producer warp + writer warp
constexpr uint32_t kWaitLimit = 1u << 22;  // polls (with back-off) before a wait gives up

struct GemvParams {
    const uint8_t *packed;
    const uint16_t *scales;
    const uint16_t *biases;
    const void *x;
    void *y;
    float *partials;         // [row group][slot][128][MT*8]
    unsigned int *counters;  // [row group]
    unsigned long long *tagged;  // M <= 4 kernel: {value, tag} words [row group][slot][128][M]; null = use partials + counters
    unsigned int *error_word;
    uint32_t N, K, M;
    uint32_t groups;      // K / G
    uint32_t row_bytes;   // packed bytes per weight row
    uint32_t group;       // G
    uint32_t sdtype;      // 0 f16, 1 bf16
    uint32_t chunks;      // K chunks per row group
    uint32_t units;       // row groups * chunks
    uint32_t max_slots;   // scratch slots per row group
    uint32_t next_units;     // head-of-next-weight L2 prefetch: units of the next weight (0 = no hint)
    uint32_t next_chunks;    //   its K chunks per row group
    uint32_t next_ctas;      //   the grid it will run on
    uint32_t next_gps;       //   its groups per unit
    uint32_t next_prefetch;  //   units to prefetch at the head of each of its CTA ranges
    uint8_t *fuse_region[kPeerMaxRanks];  // fused all-reduce: every rank's exchange region ([fuse_rank] is local)
    uint32_t fuse_rank, fuse_size;        //   fuse_size == 0: plain GEMV
    uint32_t y_f32;          // M <= 4 kernel: write y as fp32 although x is bf16 (first half of the fused FFN)
    uint32_t act;            // M <= 4 kernel: 1 / 2 = x is fp32 [M][2K] and the operand is silu / gelu(x[:, :K]) * x[:, K:]
    unsigned int *grid_bar;  // M <= 4 kernel, several operations per launch: arrival counters, zero between launches
    uint32_t dep;            // M <= 4 kernel, several operations per launch: 1 = x of this operation is written by an earlier
                             // operation of the launch (wait for the grid-wide arrival at the previous operation)
    uint8_t *xq;             // launch lists, one activation row: this operation's quantised activations in global memory,
                             // [K chunk][quantised unit + {scale, sum} pairs], built once per launch at its very start and
                             // copied into every ring stage beside the weights (null: each CTA quantises for itself)
    uint32_t xq_pair0;       //   index of this operation's first (operation, K chunk) pair among all such pairs of the list
    uint32_t rot;            // launch lists: CTA b takes the unit range of index (b + rot) mod grid, so that the CTAs with one
                             //   unit more than the others are different ones from operation to operation
};

// One operation's exchange as the writer warp needs it to collect the peers' words later on.
struct FusedOp {
    void *y;
    uint8_t *region;   // this rank's exchange region
    uint32_t N, M, y_f32, size, epoch, phase;
};

// A launch list for the M <= 4 kernel: operations in order, three tensor maps (packed, scales, biases) per operation,
// all in device memory (written by the host before the launch).
// One (operation, K chunk) pair of a launch list whose activations are quantised at the start of the launch.
struct XqPair {
    const void *x;     // the operation's bf16 activations [M][K]
    uint8_t *dst;      // where this chunk's quantised unit goes
    uint32_t kc, groups, K, M;
};

struct GemvOpList {
    const GemvParams *ops;
    const CUtensorMap *maps;
    uint32_t count;
    unsigned int *grid_bar;   // `count` arrival counters (+ one for the quantised activations), zero between launches
    uint32_t xq_pairs;        // (operation, K chunk) pairs whose activations are quantised at the start of the launch (0: none)
    const XqPair *xq_tab;     // one entry per pair
};

// ---- small PTX wrappers ----------------------------------------------------
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
// Bounded wait: false (and the error word set) when the limit runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int *error_word, uint32_t code) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
    }
    atomicOr(error_word, code);
    return false;
}
// one TMA tile: box {128 bytes, 128 rows} of the packed matrix at (byte column c0, row c1)
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, uint32_t c0, uint32_t c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// the same tile as an L2 prefetch (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *tmap, uint32_t c0, uint32_t c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(tmap)),
                 "r"(c0), "r"(c1)
                 : "memory");
}

constexpr uint32_t kPeerPollLimit = 1u << 23;  // polls with back-off (several seconds) before a rank gives up on a peer

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same with a zero accumulator input (first MMA of a group)
__device__ __forceinline__ void mma_bf16_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Packed words of one lane for one group and row, from a swizzled panel.
// `addr` = shared address of the lane's first piece (swizzle already applied).
// Pieces wider than one 16-byte chunk continue in the following chunks, whose
// positions differ from the first by the XOR of the chunk index with `xr` = row & 7.
template <int WPT>
__device__ __forceinline__ void lds_row(uint32_t addr, uint32_t xr, uint32_t (&w)[WPT]) {
    if constexpr (WPT == 1) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(addr));
    } else if constexpr (WPT == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
    } else if constexpr (WPT == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    } else {
        // two chunks c and c + 1 with c even: their swizzled positions differ in bit 4 only
        static_assert(WPT == 8, "unsupported load width");
        (void)xr;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(addr ^ 16u));
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

// contiguous, near-equal unit ranges: the first `rem` CTAs take one unit more
__device__ __host__ __forceinline__ uint32_t range_begin(uint32_t cta, uint32_t units, uint32_t ctas) {
    const uint32_t q = units / ctas, rem = units % ctas;
    return cta * q + (cta < rem ? cta : rem);
}
// launch lists: the range index of CTA `cta` in an operation whose ranges are dealt from CTA (grid - rot) on
__device__ __forceinline__ uint32_t range_index(uint32_t cta, uint32_t rot, uint32_t ctas) {
    const uint32_t v = cta + rot;
    return v >= ctas ? v - ctas : v;
}
__device__ __host__ __forceinline__ uint32_t unit_owner(uint32_t u, uint32_t units, uint32_t ctas) {
    const uint32_t q = units / ctas, rem = units % ctas;
    const uint32_t cut = rem * (q + 1u);
    return u < cut ? u / (q + 1u) : rem + (u - cut) / q;
}

constexpr int kPanelBytes = 128;                       // bytes per row in one TMA tile (the swizzle span)
constexpr int kPanels = kChunkBytes / kPanelBytes;     // TMA tiles per unit (= K halves, one per warp set)
constexpr int kPanelSize = kRows * kPanelBytes;        // 16 KB
constexpr int kWeightBytes = kPanels * kPanelSize;     // 32 KB of packed codes per unit
constexpr int kFragItems = 16;                         // (group, word) pairs per unit: 256 B / 16 B
constexpr int kMaxBlockUnits = 16;                     // units whose activation fragments are built together

template <int GB>
struct StreamGeom {
    static constexpr int GPS = kChunkBytes / GB;   // groups per unit
    static constexpr int GPP = kPanelBytes / GB;   // groups per panel = groups per warp and unit
    static constexpr int LW = GB / 4;              // bytes one lane reads per group and row
    static constexpr int WPT = LW / 4;             // packed words per lane per group and row
    // scales / biases of one unit: a TMA box of SBOX bytes x 128 rows (16 bytes is the smallest box)
    static constexpr int SBOX = GPS * 2 > 16 ? GPS * 2 : 16;
    static constexpr int SB_BYTES = kRows * SBOX;
    static constexpr int STAGE_BYTES = kWeightBytes + 2 * SB_BYTES;  // multiple of 1024
};

// shared-memory plan (all offsets from the 1024-byte aligned ring base)
template <int GB, int MT, bool XF32>
struct SmemPlan {
    static constexpr int NF = XF32 ? 2 : 1;
    static constexpr int UNIT_FRAG_MAX = kFragItems * MT * NF * 512;            // one unit's fragments, 8 rows per tile
    // one block of units: at least two (32-element groups with two tiles have room for one)
    static constexpr int FRAG_MIN = (GB == 16 && MT == 2) ? 16384 : 32768;
    static constexpr int FRAG_BUF = UNIT_FRAG_MAX > FRAG_MIN ? UNIT_FRAG_MAX : FRAG_MIN;
    static constexpr int XS_UNIT = (kChunkBytes / GB) * MT * 8 * 4;             // group sums of one unit
    static constexpr int XS_BUF = kMaxBlockUnits * XS_UNIT;
    static constexpr int OUT_BUF = 2 * kRowBlocks * 32 * MT * 4 * 4;           // both K halves of one row group
    static constexpr int OFF_FRAG = kStages * StreamGeom<GB>::STAGE_BYTES;
    static constexpr int OFF_XS = OFF_FRAG + 2 * FRAG_BUF;
    static constexpr int OFF_OUT = OFF_XS + 2 * XS_BUF;
    static constexpr int TOTAL = OFF_OUT + 2 * OUT_BUF + 1024;  // + slack to align the ring
};

// Row permutation inside a warp's 16 rows: lane group g (= lane / 4) works on row rho(g)
// (and rho(g) + 8).  Chosen per load width so that the rows met by one shared-memory
// wavefront differ in the address bits the 128-byte swizzle XORs into the chunk index.
template <int LW>
__device__ __forceinline__ uint32_t rho(uint32_t g) {
    if constexpr (LW == 8) return ((g & 3u) << 1) | (g >> 2);   // 0 2 4 6 1 3 5 7
    if constexpr (LW == 16) return ((g & 1u) << 2) | (g >> 1);  // 0 4 1 5 2 6 3 7
    return g;
}

__device__ __forceinline__ void consumer_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

// scale / bias word (two 16-bit values) -> f32 of the low or high half; SD = 1 bf16, 0 f16
template <int SD>
__device__ __forceinline__ float sb_half(uint32_t w, int hi) {
    if constexpr (SD == 1) return __uint_as_float(hi ? (w & 0xFFFF0000u) : (w << 16));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(hi ? (w >> 16) : (w & 0xFFFFu))));
}

// Warp roles: 0..15 consumers (kh * 8 + rb), 16 producer, 17 writer.
// Head-of-next-weight prefetch.  A decoder knows which weight the following launch streams; the host can
// name it, and each producer, once its own last tile is requested, asks L2 for the first tiles of the ranges
// the next launch's CTAs will start on.  Those requests queue behind this launch's reads, so HBM keeps
// streaming through this launch's write-out tail, the launch gap and the next launch's prologue, which
// then finds its first tiles in L2.  Nothing waits on a prefetch and it has no destination in this CTA.
__device__ __forceinline__ void prefetch_next_head(const GemvParams &p, const CUtensorMap *nw, const CUtensorMap *ns,
                                                   const CUtensorMap *nb) {
    if (p.next_units == 0u) return;
    for (uint32_t c = blockIdx.x; c < p.next_ctas; c += gridDim.x) {
        const uint32_t b = range_begin(c, p.next_units, p.next_ctas);
        uint32_t e = range_begin(c + 1u, p.next_units, p.next_ctas);
        if (e > b + p.next_prefetch) e = b + p.next_prefetch;
        uint32_t rg = b / p.next_chunks, kc = b - rg * p.next_chunks;
        for (uint32_t u = b; u < e; ++u) {
#pragma unroll
            for (int pnl = 0; pnl < kPanels; ++pnl) tma_prefetch_2d(nw, kc * kChunkBytes + pnl * kPanelBytes, rg * kRows);
            const uint32_t sb_col = (kc * p.next_gps * 2u) & ~15u;
            tma_prefetch_2d(ns, sb_col, rg * kRows);
            tma_prefetch_2d(nb, sb_col, rg * kRows);
            if (++kc == p.next_chunks) kc = 0u, ++rg;
        }
    }
}

template <int GB, int BITS, int MT, bool XF32, int SD>
__global__ void __launch_bounds__(kThreads, 1)
gaf_gemv_stream_kernel(const GemvParams p, const __grid_constant__ CUtensorMap tmap_w,
                       const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap next_w, const __grid_constant__ CUtensorMap next_s,
                       const __grid_constant__ CUtensorMap next_b) {
    using Geo = StreamGeom<GB>;
    using Plan = SmemPlan<GB, MT, XF32>;
    constexpr int GPS = Geo::GPS, GPP = Geo::GPP, LW = Geo::LW, WPT = Geo::WPT;
    constexpr int XPB = 8 / BITS;                          // activations per packed byte
    constexpr float OFF = BITS == 4 ? 128.f : 2176.f;      // what the +128 offsets add per unit of sum(x)
    constexpr int NF = Plan::NF;                           // fragment sets per activation tile (hi, lo)
    constexpr int SBW = GPP * 2 / 4 > 0 ? GPP * 2 / 4 : 1;  // 32-bit words holding one row's scales of a warp's groups
    static_assert(WPT >= 1 && GPP >= 1, "unsupported group size");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[kStages];
    __shared__ __align__(8) uint64_t s_empty[kStages];
    __shared__ __align__(8) uint64_t s_out_full[2];   // consumers -> writer: a row group's sums are in the out buffer
    __shared__ __align__(8) uint64_t s_out_empty[2];  // writer -> consumers: the out buffer may be reused
    __shared__ volatile uint32_t s_abort;  // a consumer warp gave up a wait: everybody leaves at the next barrier

    // the ring starts at a 1024-byte boundary (8 rows x 128 bytes, the swizzle atom)
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        s_abort = 0u;
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), kConsumerWarps);
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_out_full[s]), kConsumerWarps);
            mbar_init(smem_u32(&s_out_empty[s]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t u_begin = range_begin(blockIdx.x, p.units, gridDim.x);
    const uint32_t u_end = range_begin(blockIdx.x + 1u, p.units, gridDim.x);
    if (u_begin >= u_end) return;
    const uint32_t rg_begin = u_begin / p.chunks;
    const uint32_t kc_begin = u_begin - rg_begin * p.chunks;

    if (warp == kConsumerWarps) {
        // ------------------------- producer warp (one lane works) -------------------------
        if (lane != 0) return;
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_s)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b)) : "memory");
        uint32_t issued = 0, rg = rg_begin, kc = kc_begin;
        bool ok = true;
        for (uint32_t u = u_begin; u < u_end; ++u, ++issued) {
            const uint32_t stage = issued % kStages;
            const uint32_t round = issued / kStages;
            if (round > 0) ok = mbar_wait(smem_u32(&s_empty[stage]), (round - 1u) & 1u, p.error_word, 0x1u);
            if (!ok) break;
            const uint32_t full = smem_u32(&s_full[stage]);
            {
                // rows past N and bytes past a row end are zero-filled by the copy engine,
                // so every unit delivers the same byte count
                const uint32_t base = ring + stage * Geo::STAGE_BYTES;
                mbar_arrive_expect_tx(full, Geo::STAGE_BYTES);
#pragma unroll
                for (int pnl = 0; pnl < kPanels; ++pnl)
                    tma_load_2d(base + pnl * kPanelSize, &tmap_w, kc * kChunkBytes + pnl * kPanelBytes, rg * kRows, full);
                const uint32_t sb_col = (kc * GPS * 2u) & ~15u;  // boxes start on 16-byte columns
                tma_load_2d(base + kWeightBytes, &tmap_s, sb_col, rg * kRows, full);
                tma_load_2d(base + kWeightBytes + Geo::SB_BYTES, &tmap_b, sb_col, rg * kRows, full);
            }
            if (++kc == p.chunks) kc = 0u, ++rg;
        }
        if (!ok) {
            // give copies already in flight a bounded time to land before the CTA's memory is released
            const uint32_t pending = issued < static_cast<uint32_t>(kStages) ? issued : static_cast<uint32_t>(kStages);
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t idx = issued - 1u - i;
                mbar_wait(smem_u32(&s_full[idx % kStages]), (idx / kStages) & 1u, p.error_word, 0x4u);
            }
        } else {
            prefetch_next_head(p, &next_w, &next_s, &next_b);
        }
        return;
    }

    const uint32_t g = lane >> 2;  // activation row inside a tile; accumulator row slot
    const uint32_t t = lane & 3;   // quarter of the group this lane holds
    const uint32_t wr = rho<LW>(g);  // weight row (of a warp's 16) behind accumulator rows g and g + 8

    if (warp == kConsumerWarps + 1) {
        // ------------------------- writer warp -------------------------
        // One round per row group this CTA touches: add the two K halves, then either write y
        // (the CTA saw the whole row group) or park the partial and take a ticket; the last
        // ticket holder adds all partials in slot order and writes y.  Nothing here is on the
        // consumers' critical path.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t rg_last_touched = (u_end - 1u) / p.chunks;
        uint32_t ob = 0, ophase = 0;
        bool tagged_ok = true;  // false once a wait for another CTA's partial sums ran out
        for (uint32_t rg = rg_begin; rg <= rg_last_touched; ++rg) {
            if (!mbar_wait(smem_u32(&s_out_full[ob]), ophase, p.error_word, 0x8u)) return;
            const uint32_t rg_first = rg * p.chunks, rg_last = rg_first + p.chunks - 1u;
            const bool whole = u_begin <= rg_first && rg_last < u_end;
            uint32_t slots = 1u, slot = 0u;
            if (!whole) {
                const uint32_t first_cta = unit_owner(rg_first, p.units, gridDim.x);
                slots = unit_owner(rg_last, p.units, gridDim.x) - first_cta + 1u;
                slot = blockIdx.x - first_cta;
            }
            float *mine = p.partials + (static_cast<size_t>(rg) * p.max_slots + slot) * (kRows * MT * 8);
            const uint32_t obuf = ring + Plan::OFF_OUT + ob * Plan::OUT_BUF + lane * (MT * 16u);
            auto store = [&](uint32_t m, uint32_t n, float val) {
                if (m < p.M && n < p.N) {
                    if constexpr (XF32)
                        static_cast<float *>(p.y)[static_cast<size_t>(m) * p.N + n] = val;
                    else
                        static_cast<__nv_bfloat16 *>(p.y)[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(val);
                }
            };
            // split row group with tagged partial sums: the CTA that owns the head (slot 0) collects
            const bool finisher = !whole && p.tagged != nullptr && slot == 0u;
            if (finisher && tagged_ok) {
                constexpr uint32_t kTag = 0x5A5A5A5Au;
                constexpr uint32_t RBC = MT == 1 ? 4u : 2u;  // row blocks per batch: every load in flight before the first check
                unsigned long long *base = p.tagged + static_cast<size_t>(rg) * p.max_slots * (kRows * MT * 8);
#pragma unroll 1
                for (uint32_t rb0 = 0; rb0 < kRowBlocks && tagged_ok; rb0 += RBC) {
                    float acc[RBC][MT][4];
#pragma unroll
                    for (uint32_t i = 0; i < RBC; ++i)
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            float b0, b1, b2, b3;
                            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                         : "=f"(acc[i][mt][0]), "=f"(acc[i][mt][1]), "=f"(acc[i][mt][2]), "=f"(acc[i][mt][3])
                                         : "r"(obuf + (rb0 + i) * (32u * MT * 16u) + mt * 16u));
                            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                         : "=f"(b0), "=f"(b1), "=f"(b2), "=f"(b3)
                                         : "r"(obuf + (kRowBlocks + rb0 + i) * (32u * MT * 16u) + mt * 16u));
                            acc[i][mt][0] += b0, acc[i][mt][1] += b1, acc[i][mt][2] += b2, acc[i][mt][3] += b3;
                        }
                    for (uint32_t sidx = 1; sidx < slots && tagged_ok; ++sidx) {  // fixed order: reproducible sums
                        unsigned long long *src = base + static_cast<size_t>(sidx) * (kRows * MT * 8);
                        unsigned long long wd[RBC][MT][4];
                        bool got = false;
                        for (uint32_t it = 0; it < kWaitLimit; ++it) {
                            bool all = true;
#pragma unroll
                            for (uint32_t i = 0; i < RBC; ++i)
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    const uint32_t r0 = (rb0 + i) * 16u + wr;
                                    const uint32_t o0 = r0 * (MT * 8) + mt * 8 + 2 * t, o1 = o0 + 8u * (MT * 8);
                                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(wd[i][mt][0]), "=l"(wd[i][mt][1]) : "l"(src + o0) : "memory");
                                    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(wd[i][mt][2]), "=l"(wd[i][mt][3]) : "l"(src + o1) : "memory");
                                }
#pragma unroll
                            for (uint32_t i = 0; i < RBC; ++i)
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                                    for (int q = 0; q < 4; ++q) all = all && static_cast<uint32_t>(wd[i][mt][q] >> 32) == kTag;
                            if (__all_sync(0xFFFFFFFFu, all)) {
                                got = true;
                                break;
                            }
                            if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
                        }
                        if (!got) {
                            if (lane == 0) atomicOr(p.error_word, 0x20u);
                            tagged_ok = false;
                            break;
                        }
#pragma unroll
                        for (uint32_t i = 0; i < RBC; ++i)
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                const uint32_t r0 = (rb0 + i) * 16u + wr;
                                const uint32_t o0 = r0 * (MT * 8) + mt * 8 + 2 * t, o1 = o0 + 8u * (MT * 8);
#pragma unroll
                                for (int q = 0; q < 4; ++q) acc[i][mt][q] += __uint_as_float(static_cast<uint32_t>(wd[i][mt][q]));
                                asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1,%2};" ::"l"(src + o0), "l"(0ull), "l"(0ull) : "memory");
                                asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1,%2};" ::"l"(src + o1), "l"(0ull), "l"(0ull) : "memory");
                            }
                    }
                    if (tagged_ok) {
#pragma unroll
                        for (uint32_t i = 0; i < RBC; ++i) {
                            const uint32_t n0 = rg * kRows + (rb0 + i) * 16u + wr, n1 = n0 + 8u;
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                store(mt * 8 + 2 * t, n0, acc[i][mt][0]);
                                store(mt * 8 + 2 * t + 1, n0, acc[i][mt][1]);
                                store(mt * 8 + 2 * t, n1, acc[i][mt][2]);
                                store(mt * 8 + 2 * t + 1, n1, acc[i][mt][3]);
                            }
                        }
                    }
                }
            }
            if (!finisher) {
#pragma unroll 2
                for (uint32_t rb = 0; rb < kRowBlocks; ++rb) {
                    const uint32_t r0 = rb * 16u + wr, r1 = r0 + 8u;
                    const uint32_t n0 = rg * kRows + r0, n1 = n0 + 8u;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        float a0, a1, a2, a3, b0, b1, b2, b3;
                        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                     : "=f"(a0), "=f"(a1), "=f"(a2), "=f"(a3)
                                     : "r"(obuf + rb * (32u * MT * 16u) + mt * 16u));
                        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                     : "=f"(b0), "=f"(b1), "=f"(b2), "=f"(b3)
                                     : "r"(obuf + (kRowBlocks + rb) * (32u * MT * 16u) + mt * 16u));
                        a0 += b0, a1 += b1, a2 += b2, a3 += b3;
                        if (whole) {
                            store(mt * 8 + 2 * t, n0, a0);
                            store(mt * 8 + 2 * t + 1, n0, a1);
                            store(mt * 8 + 2 * t, n1, a2);
                            store(mt * 8 + 2 * t + 1, n1, a3);
                        } else if (p.tagged != nullptr) {
                            // Partial sums that carry their own arrival tag ({fp32 value, tag} in one 64-bit
                            // word): the CTA that owns the head of the row group (slot 0; it gets there last)
                            // adds the other slots to its own sums in slot order and clears the words; nobody
                            // takes a ticket or fences.
                            constexpr uint32_t kTag = 0x5A5A5A5Au;
                            constexpr unsigned long long kTagHi = static_cast<unsigned long long>(kTag) << 32;
                            unsigned long long *base = p.tagged + static_cast<size_t>(rg) * p.max_slots * (kRows * MT * 8);
                            const uint32_t o0 = r0 * (MT * 8) + mt * 8 + 2 * t, o1 = r1 * (MT * 8) + mt * 8 + 2 * t;
                            if (slot != 0u) {
                                unsigned long long *dst = base + static_cast<size_t>(slot) * (kRows * MT * 8);
                                asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1,%2};" ::"l"(dst + o0), "l"(kTagHi | __float_as_uint(a0)),
                                             "l"(kTagHi | __float_as_uint(a1))
                                             : "memory");
                                asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1,%2};" ::"l"(dst + o1), "l"(kTagHi | __float_as_uint(a2)),
                                             "l"(kTagHi | __float_as_uint(a3))
                                             : "memory");
                            }
                        } else {
                            // slot layout [128 rows][MT*8]: this lane's values are 8-byte pairs
                            *reinterpret_cast<float2 *>(mine + r0 * (MT * 8) + mt * 8 + 2 * t) = make_float2(a0, a1);
                            *reinterpret_cast<float2 *>(mine + r1 * (MT * 8) + mt * 8 + 2 * t) = make_float2(a2, a3);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_out_empty[ob]));  // the consumers may refill this buffer
            if (!whole && p.tagged == nullptr) {
                // release the partial (all lanes' stores are ordered before lane 0's atomic by the warp
                // barrier) and learn whether the other owners of this row group are done
                unsigned int ticket = 0;
                if (lane == 0)
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + rg) : "memory");
                ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
                if (ticket == slots - 1u) {
                    const float *all = p.partials + static_cast<size_t>(rg) * p.max_slots * (kRows * MT * 8);
                    if (slots == 2u) {
                        // the usual case: a few row blocks at a time, every load issued before the first use
                        constexpr uint32_t RBC = MT == 1 ? 4u : 2u;
#pragma unroll 1
                        for (uint32_t rb0 = 0; rb0 < kRowBlocks; rb0 += RBC) {
                            float2 va[RBC][MT][2], vb[RBC][MT][2];
#pragma unroll
                            for (uint32_t i = 0; i < RBC; ++i)
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                                    for (int sidx = 0; sidx < 2; ++sidx) {
                                        const float *sp = all + static_cast<size_t>(sidx) * (kRows * MT * 8);
                                        const uint32_t r0 = (rb0 + i) * 16u + wr, r1 = r0 + 8u;
                                        va[i][mt][sidx] = __ldcg(reinterpret_cast<const float2 *>(sp + r0 * (MT * 8) + mt * 8 + 2 * t));
                                        vb[i][mt][sidx] = __ldcg(reinterpret_cast<const float2 *>(sp + r1 * (MT * 8) + mt * 8 + 2 * t));
                                    }
#pragma unroll
                            for (uint32_t i = 0; i < RBC; ++i) {
                                const uint32_t n0 = rg * kRows + (rb0 + i) * 16u + wr, n1 = n0 + 8u;
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    store(mt * 8 + 2 * t, n0, va[i][mt][0].x + va[i][mt][1].x);
                                    store(mt * 8 + 2 * t + 1, n0, va[i][mt][0].y + va[i][mt][1].y);
                                    store(mt * 8 + 2 * t, n1, vb[i][mt][0].x + vb[i][mt][1].x);
                                    store(mt * 8 + 2 * t + 1, n1, vb[i][mt][0].y + vb[i][mt][1].y);
                                }
                            }
                        }
                    } else {
#pragma unroll 1
                        for (uint32_t rb = 0; rb < kRowBlocks; ++rb) {
                            const uint32_t r0 = rb * 16u + wr, r1 = r0 + 8u;
                            const uint32_t n0 = rg * kRows + r0, n1 = n0 + 8u;
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
                                for (uint32_t sidx = 0; sidx < slots; ++sidx) {  // fixed order: reproducible sums
                                    const float *sp = all + static_cast<size_t>(sidx) * (kRows * MT * 8);
                                    const float2 xa = __ldcg(reinterpret_cast<const float2 *>(sp + r0 * (MT * 8) + mt * 8 + 2 * t));
                                    const float2 xb = __ldcg(reinterpret_cast<const float2 *>(sp + r1 * (MT * 8) + mt * 8 + 2 * t));
                                    a.x += xa.x, a.y += xa.y, b.x += xb.x, b.y += xb.y;
                                }
                                store(mt * 8 + 2 * t, n0, a.x);
                                store(mt * 8 + 2 * t + 1, n0, a.y);
                                store(mt * 8 + 2 * t, n1, b.x);
                                store(mt * 8 + 2 * t + 1, n1, b.y);
                            }
                        }
                    }
                    if (lane == 0) p.counters[rg] = 0u;  // ready for the next launch
                }
            }
            ob ^= 1u;
            if (ob == 0u) ophase ^= 1u;
        }
        return;
    }

    // --------------------------- consumer warps ---------------------------
    // warp = kh * 8 + rb: row block rb (16 of the unit's 128 rows), K half kh (one 128-byte panel)
    const uint32_t rb = warp & (kRowBlocks - 1);
    const uint32_t kh = warp / kRowBlocks;
    const uint8_t *xbase = static_cast<const uint8_t *>(p.x);
    const size_t x_elt = XF32 ? 4 : 2;

    // Activation fragments are stored only for the activation rows that exist (one tile: min(M, 8)).
    const uint32_t mg = MT == 1 ? (p.M < 8u ? p.M : 8u) : 8u;
    const uint32_t item_bytes = mg * 64u;                                 // one (group, word, tile, set)
    const uint32_t unit_frag_bytes = kFragItems * MT * NF * item_bytes;   // one unit
    uint32_t block_units = Plan::FRAG_BUF / unit_frag_bytes;              // units prepared together
    if (block_units > static_cast<uint32_t>(kMaxBlockUnits)) block_units = kMaxBlockUnits;
    // When the fragments of a whole row of K fit the two buffers taken together, they are built once, in the
    // order this CTA meets the K chunks, and every later row group reuses them: no rebuild, no CTA barrier.
    const bool whole_k = p.chunks <= static_cast<uint32_t>(kMaxBlockUnits) && p.chunks * unit_frag_bytes <= 2u * Plan::FRAG_BUF;
    const uint32_t block_len = whole_k ? p.chunks : block_units;
    const bool has_x = g < mg;

    // shared-memory offsets of this lane's pieces of a panel row, one per group of the panel
    // (swizzle: 16-byte chunk index XOR (row & 7); rows wr and wr + 8 share the XOR term)
    uint32_t swz[GPP];
#pragma unroll
    for (int q = 0; q < GPP; ++q) {
        const uint32_t ob = q * GB + t * LW;
        swz[q] = ring + (rb * 16u + wr) * kPanelBytes + kh * kPanelSize + ((((ob >> 4) ^ wr) & 7u) << 4) + (ob & 15u);
    }
    // this lane's rows in the scale / bias boxes of a stage (row pitch SBOX)
    const uint32_t sb_lane = ring + kWeightBytes + (rb * 16u + wr) * Geo::SBOX + kh * GPP * 2u;
    const uint32_t frag_lane = ring + Plan::OFF_FRAG + (g * 4u + t) * 16u;
    const uint32_t xs_lane = ring + Plan::OFF_XS + t * 8u;
    const uint32_t out_lane = ring + Plan::OFF_OUT + ((kh * kRowBlocks + rb) * 32u + lane) * (MT * 16u);

    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;

    // ---- activation fragments and group sums for a block of units, built once per CTA ----
    // (unit ub of the block, group gl) pairs are dealt round-robin to the 16 warps.
    // fragment (ub, gl, word j, tile mt, set f) -> buf + ub*unit_frag_bytes + (((gl*WPT + j)*MT + mt)*NF + f)*item_bytes
    auto prep_block = [&](uint32_t kc_first, uint32_t count, uint32_t buf) {
        for (uint32_t pi = warp; pi < count * GPS; pi += kConsumerWarps) {
            const uint32_t ub = pi / GPS, gl = pi % GPS;
            const uint32_t gi = ((kc_first + ub) % p.chunks) * GPS + gl;
            float xs[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) xs[mt][i] = 0.f;
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t m = mt * 8 + g;
                    uint32_t xh[4], xl[4];
                    const uint32_t kx = gi * p.group + (t * LW + 4 * j) * XPB;
                    load_x_frags<BITS, XF32>(xbase + static_cast<size_t>(m) * p.K * x_elt, kx, m < p.M && gi < p.groups,
                                             xh, xl);
                    if (has_x) {
                        const uint32_t dst = frag_lane + buf * Plan::FRAG_BUF + ub * unit_frag_bytes +
                                             (((gl * WPT + j) * MT + mt) * NF) * item_bytes;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(xh[0]), "r"(xh[1]),
                                     "r"(xh[2]), "r"(xh[3])
                                     : "memory");
                        if constexpr (XF32)
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + item_bytes), "r"(xl[0]),
                                         "r"(xl[1]), "r"(xl[2]), "r"(xl[3])
                                         : "memory");
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // group sums of x: all-ones A (for 8-bit, only the low-nibble slots)
                        mma_bf16_16816(xs[mt], kOnesBf16, kOnesBf16, BITS == 4 ? kOnesBf16 : 0u,
                                       BITS == 4 ? kOnesBf16 : 0u, xh[2 * h], xh[2 * h + 1]);
                        if constexpr (XF32)
                            mma_bf16_16816(xs[mt], kOnesBf16, kOnesBf16, BITS == 4 ? kOnesBf16 : 0u,
                                           BITS == 4 ? kOnesBf16 : 0u, xl[2 * h], xl[2 * h + 1]);
                    }
                }
            }
            if (g == 0) {  // every accumulator row holds the same sums
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t dst = xs_lane + buf * Plan::XS_BUF + ub * Plan::XS_UNIT + (gl * MT * 8 + mt * 8) * 4u;
                    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(dst), "f"(xs[mt][0]), "f"(xs[mt][1]) : "memory");
                }
            }
        }
    };

    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const uint32_t total = u_end - u_begin;
        prep_block(kc_begin, total < block_len ? total : block_len, 0u);
    }
    consumer_barrier();

    uint32_t rg = rg_begin, kc = kc_begin;
    uint32_t stage = 0, phase = 0;     // ring position
    uint32_t ub = 0, buf = 0;          // unit inside the fragment block, fragment buffer
    uint32_t ob = 0, ophase = 0;       // out buffer and its phase
    bool alive = true;                 // false once this warp gave up a wait
    for (uint32_t u = u_begin; u < u_end; ++u) {
        const bool more = u + 1u < u_end;
        uint32_t kc_n = kc + 1u, rg_n = rg;  // row group / K chunk of the next unit
        if (kc_n == p.chunks) kc_n = 0u, ++rg_n;

        // A warp must not leave before the barriers below (the others would wait for it forever):
        // on a timeout it raises s_abort and skips the arithmetic until everybody leaves together.
        bool landed = false;
        if (alive) {
            landed = mbar_wait(smem_u32(&s_full[stage]), phase, p.error_word, 0x2u);
            if (!landed) alive = false, s_abort = 1u;
        }

        const uint32_t off = kc * kChunkBytes + kh * kPanelBytes;
        const uint32_t bytes = off < p.row_bytes ? min(static_cast<uint32_t>(kPanelBytes), p.row_bytes - off) : 0u;
        const uint32_t ngroups = landed ? bytes / GB : 0u;  // groups of this warp's panel that exist
        const uint32_t stage_off = stage * Geo::STAGE_BYTES;
        const uint32_t fragb = frag_lane + buf * Plan::FRAG_BUF + ub * unit_frag_bytes + (kh * GPP * WPT * MT * NF) * item_bytes;
        const uint32_t xsb = xs_lane + buf * Plan::XS_BUF + ub * Plan::XS_UNIT + (kh * GPP * MT * 8) * 4u;

        // scales / biases of this warp's groups for rows wr and wr + 8: {s0, b0, s1, b1}[SBW words]
        uint32_t sb[4][SBW];
        if (ngroups) {
            const uint32_t a0 = stage_off + sb_lane + ((kc * GPS * 2u) & 15u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t a = a0 + (i & 1) * Geo::SB_BYTES + (i >> 1) * 8u * Geo::SBOX;
                if constexpr (GPP == 1) {
                    uint16_t v;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
                    sb[i][0] = v;
                } else if constexpr (SBW == 1) {
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sb[i][0]) : "r"(a));
                } else if constexpr (SBW == 2) {
                    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(sb[i][0]), "=r"(sb[i][1]) : "r"(a));
                } else {
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(sb[i][0]), "=r"(sb[i][1]), "=r"(sb[i][2]), "=r"(sb[i][3])
                                 : "r"(a));
                }
            }
        }

#pragma unroll
        for (int q = 0; q < GPP; ++q) {
            if (static_cast<uint32_t>(q) < ngroups) {
                uint32_t wa[WPT], wb[WPT];
                lds_row<WPT>(stage_off + swz[q], wr, wa);
                lds_row<WPT>(stage_off + swz[q] + 8u * kPanelBytes, wr, wb);
                float acc[MT][4];
#pragma unroll
                for (int j = 0; j < WPT; ++j) {
                    uint32_t pa[4], pb[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        pa[i] = ((wa[j] >> (4 * i)) & kNibMask) | kMagic128;
                        pb[i] = ((wb[j] >> (4 * i)) & kNibMask) | kMagic128;
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                        for (int f = 0; f < NF; ++f) {
                            uint32_t xf[4] = {0u, 0u, 0u, 0u};
                            if (has_x)
                                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                             : "=r"(xf[0]), "=r"(xf[1]), "=r"(xf[2]), "=r"(xf[3])
                                             : "r"(fragb + (((q * WPT + j) * MT + mt) * NF + f) * item_bytes));
                            if (j == 0 && f == 0)
                                mma_bf16_16816_z(acc[mt], pa[0], pb[0], pa[1], pb[1], xf[0], xf[1]);
                            else
                                mma_bf16_16816(acc[mt], pa[0], pb[0], pa[1], pb[1], xf[0], xf[1]);
                            mma_bf16_16816(acc[mt], pa[2], pb[2], pa[3], pb[3], xf[2], xf[3]);
                        }
                    }
                }
                const float s0 = sb_half<SD>(sb[0][q >> 1], q & 1), b0 = sb_half<SD>(sb[1][q >> 1], q & 1);
                const float s1 = sb_half<SD>(sb[2][q >> 1], q & 1), b1 = sb_half<SD>(sb[3][q >> 1], q & 1);
                const float b0o = fmaf(-OFF, s0, b0), b1o = fmaf(-OFF, s1, b1);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    float xs0, xs1;
                    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];"
                                 : "=f"(xs0), "=f"(xs1)
                                 : "r"(xsb + (q * MT * 8 + mt * 8) * 4u));
                    yacc[mt][0] = fmaf(s0, acc[mt][0], yacc[mt][0]);
                    yacc[mt][1] = fmaf(s0, acc[mt][1], yacc[mt][1]);
                    yacc[mt][2] = fmaf(s1, acc[mt][2], yacc[mt][2]);
                    yacc[mt][3] = fmaf(s1, acc[mt][3], yacc[mt][3]);
                    yacc[mt][0] = fmaf(b0o, xs0, yacc[mt][0]);
                    yacc[mt][1] = fmaf(b0o, xs1, yacc[mt][1]);
                    yacc[mt][2] = fmaf(b1o, xs0, yacc[mt][2]);
                    yacc[mt][3] = fmaf(b1o, xs1, yacc[mt][3]);
                }
            }
        }
        // this warp is done with the stage
        __syncwarp();
        if (landed && lane == 0) mbar_arrive(smem_u32(&s_empty[stage]));
        if (++stage == kStages) stage = 0u, phase ^= 1u;

        // ---- end of this CTA's share of the row group: hand the sums to the writer warp ----
        if ((kc + 1u == p.chunks) || !more) {
            if (alive && !mbar_wait(smem_u32(&s_out_empty[ob]), ophase ^ 1u, p.error_word, 0x10u)) alive = false, s_abort = 1u;
            if (alive) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(out_lane + ob * Plan::OUT_BUF + mt * 16u),
                                 "f"(yacc[mt][0]), "f"(yacc[mt][1]), "f"(yacc[mt][2]), "f"(yacc[mt][3])
                                 : "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_out_full[ob]));
            }
            ob ^= 1u;
            if (ob == 0u) ophase ^= 1u;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) yacc[mt][i] = 0.f;
        }

        // ---- end of a fragment block: build the next one in the other buffer, then everybody meets ----
        if (++ub == block_len) {
            ub = 0u;
            if (more && !whole_k) {
                const uint32_t left = u_end - (u + 1u);
                prep_block(kc_n, left < block_units ? left : block_units, buf ^ 1u);
                consumer_barrier();
                if (s_abort) return;
                buf ^= 1u;
            }
        }
        kc = kc_n, rg = rg_n;
    }
}

// ---------------------------------------------------------------------------
// Streaming GEMV for M <= 4 on the integer dot-product unit (M <= 2) or the int8 tensor-core MMA (M = 3, 4).
//
// With one or two activation rows the tensor-core formulation above wastes seven
// of its eight columns and is bound by instruction issue (unpack + fragment
// bookkeeping per 16 rows).  Here every lane owns whole weight rows instead:
//   * activations are turned, once per CTA and K block, into 13-bit integers per
//     group (x ~ xi * 2^(E-12), E from the group's largest |x|, |xi| <= 4095) and
//     split into two signed bytes xi = 64 * hi + lo;
//   * a packed word yields its even and odd nibbles as bytes with three integer
//     ops; four dp4a (u8 x s8 -> s32) per word accumulate sum(q * hi), sum(q * lo)
//     exactly;
//   * per group and row: y += s * 2^(E-12) * (64 * acc_hi + acc_lo) + b * sum(x).
// The quantisation error of x is at most 2^-13 of the group's largest |x| per
// element (bf16 inputs carry 2^-9 relative), far inside the 1e-2 budget.
// Same producer / ring / split-K protocol as the tensor-core kernel; warp =
// (group of the unit, block of rows), lane = row.
//
// M = 3, 4 (template MD = 4) keep the skeleton and the quantised activations but do the dot products on the
// int8 tensor-core MMA (m16n8k32, u8 x s8): a packed word's even / odd nibbles, as bytes, ARE the A registers
// (the k order inside an MMA is free, the activation bytes are laid out to match), and the eight columns are
// the (activation row, limb) pairs, so four rows cost what one costs.  A warp keeps its group's B registers
// for all its 16-row blocks; thread (g, t) of a block ends up with the sums of rows g, g + 8 for activation
// row t.
// ---------------------------------------------------------------------------
// float(64 * hi + lo) for |hi|, |lo| < 2^22 without conversion instructions (which issue at a quarter of
// the rate): adding 1.5 * 2^23 to the bit pattern is exact, and the sum stays below 2^24
__device__ __forceinline__ float limbs_to_float(int hi, int lo) {
    const float fh = __int_as_float(hi + 0x4B400000) - 12582912.f;
    const float fl = __int_as_float(lo + 0x4B400000) - 12582912.f;
    return fmaf(fh, 64.f, fl);
}
// int8 tensor-core MMA: D[16x8] += A[16x32] (u8, row) * B[32x8] (s8, col), s32 accumulate
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// the gate's activation: 1 = silu (core/src/compute/cuda/kernels/ops/reduction_ops.cu:46-57),
// 2 = tanh-form gelu (reduction_ops.cu:59-72)
__device__ __forceinline__ float gate_activation(float g, uint32_t act) {
    if (act == 2u) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.f + tanhf(inner));
    }
    return g / (1.f + __expf(-g));
}

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int GB, int MD, bool XF32, int NST, int BU, bool XQS = false, int BITS = 4>
struct DpPlan {
    static constexpr int GPS = kChunkBytes / GB;           // groups per unit
    static constexpr int WPG = GB / 4;                     // packed words per group and row
    // quantised activations of one group: per word and row 16 bytes (eight 4-bit codes x {hi, lo}) or 8 (four 8-bit codes)
    static constexpr int XQ_GROUP = WPG * MD * (BITS == 4 ? 16 : 8);
    static constexpr int XQ_UNIT = GPS * XQ_GROUP;         // 1 KB per activation row for any group size
    static constexpr int XI_UNIT = GPS * MD * 8;           // {2^(E-12), sum x} per group and activation row
    static constexpr int OUT_BUF = GPS * kRows * MD * 4;   // per-group partial sums of one row group
    static constexpr int NOB = MD > 4 ? 1 : 2;             // hand-over buffers to the writer warp (32 KB each at eight rows)
    // XQS: a stage also holds the unit's quantised activations (copied from global memory like the weights)
    static constexpr int XQS_UNIT = XQ_UNIT + XI_UNIT;     // a multiple of 16 bytes
    static constexpr int STAGE = XQS ? ((StreamGeom<GB>::STAGE_BYTES + XQS_UNIT + 1023) / 1024) * 1024 : StreamGeom<GB>::STAGE_BYTES;
    static constexpr int OFF_XQ = NST * STAGE;
    static constexpr int OFF_XI = OFF_XQ + 2 * BU * XQ_UNIT;
    static constexpr int OFF_OUT = OFF_XI + 2 * BU * XI_UNIT;
    static constexpr int TOTAL = OFF_OUT + NOB * OUT_BUF + 1024;
};

// NCW consumer warps, NST ring stages, BU units per activation block.  (A configuration with 8 warps and 2
// stages, two CTAs per SM, measured no better and was dropped.)
//
// NOPS = 2 runs two dependent linears in ONE launch (the FFN: gate|up, then down on silu(gate) * up): the
// copy warp walks straight on into the second weight while the first one's sums are still being collected,
// so the ring never drains between the two; the second operation's warps meet at a grid-wide arrival
// counter (every CTA's writer arrives when its share of the first output is stored) before they read that
// output.  In that mode the "next" tensor maps are the second weight's.
// NOPS = 0 runs a whole launch list (GemvOpList) the same way: the copy warp streams across all the weights of a
// decoder step without a pause, an operation waits at the arrival counter of its predecessor only when its
// activations are that predecessor's output (GemvParams::dep), and the per-launch costs (launch gap, ring ramp-up
// and drain, write-out tail) are paid once per list instead of once per weight.
template <int GB, int MD, bool XF32, int SD, int NCW, int NST, int BU, int NOPS, int BITS>
__global__ void __launch_bounds__((NCW + 2) * 32, 1)
gaf_gemv_dp4a_kernel(const GemvParams pa, const GemvParams pb, const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap next_w, const __grid_constant__ CUtensorMap next_s,
                     const __grid_constant__ CUtensorMap next_b, const GemvOpList list) {
    using Geo = StreamGeom<GB>;
    // launch lists (one activation row on the dp4a instance, up to four on the int8-MMA instance): activations
    // quantised once per launch, streamed into the stages
    constexpr bool XQS = NOPS == 0 && (MD == 1 || MD >= 4) && !XF32;
    using Plan = DpPlan<GB, MD, XF32, NST, BU, XQS, BITS>;
    static_assert(BITS == 4 || (BITS == 8 && MD <= 4), "8-bit codes: up to four rows");
    constexpr int GPS = Geo::GPS, WPG = Plan::WPG;
    constexpr int RW = kRows * GPS / NCW;  // rows per warp: 128 (G=32), 64 (G=64), 32 (G=128)
    constexpr int R = RW / 32;                        // rows per lane
    constexpr int CH = GB / 16;                       // 16-byte chunks per group and row
    constexpr bool IM = MD >= 4;                      // three to eight activation rows: int8 MMA instead of dp4a
    constexpr int NB = IM ? MD / 4 : 1;               // IM: sets of eight B columns (four activation rows x two limbs each)
    constexpr int MQ = MD > 4 ? 4 : MD;               // writer: activation rows handled together when it polls for partial sums
    constexpr int WPT = GB / 16;                      // IM: packed words per quad lane, group and row = MMAs per group
    constexpr int NRB = RW / 16;                      // IM: 16-row blocks per warp
    static_assert(R >= 1 && GPS <= NCW && GPS * (kRows / RW) == NCW, "unsupported group size");

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_full[NST];
    __shared__ __align__(8) uint64_t s_empty[NST];
    __shared__ __align__(8) uint64_t s_out_full[2];
    __shared__ __align__(8) uint64_t s_out_empty[2];
    __shared__ volatile uint32_t s_abort;

    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        s_abort = 0u;
#pragma unroll
        for (int s = 0; s < NST; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), NCW);
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_out_full[s]), NCW);
            mbar_init(smem_u32(&s_out_empty[s]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // one or two operations: every CTA has at least one unit of each (the host caps the grid at the smallest unit count).
    // A launch list may hold operations with fewer units than CTAs: a CTA without units of one still arrives at its counter
    if (NOPS != 0 && range_begin(blockIdx.x, pa.units, gridDim.x) >= range_begin(blockIdx.x + 1u, pa.units, gridDim.x)) return;
    const uint32_t nops = NOPS > 0 ? static_cast<uint32_t>(NOPS) : list.count;   // list mode: pa is the first operation
    unsigned int *const gbar = NOPS > 0 ? pa.grid_bar : list.grid_bar;

    if (warp == NCW) {
        // ------------------------- producer warp (one lane works) -------------------------
        if (lane != 0) return;
        uint32_t issued = 0;
        bool ok = true;
        bool xq_seen = !XQS || list.xq_pairs == 0u;
        uint32_t late_dst[NST], late_bar[NST], n_late = 0u;
        const uint8_t *late_src[NST];
        auto xq_copy = [&](uint32_t dst, const uint8_t *src, uint32_t bar) {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                         "l"(src), "n"(Plan::XQS_UNIT), "r"(bar)
                         : "memory");
        };
        // waits (bounded) until every CTA has written its share of the launch's quantised activations, orders the copies
        // (async proxy) after what was observed, and issues the copies that were put off
        auto flush_late = [&]() -> bool {
            bool there = false;
            for (uint32_t it = 0; it < kWaitLimit; ++it) {
                unsigned int v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gbar + nops) : "memory");
                if (v >= gridDim.x) {
                    there = true;
                    break;
                }
                if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
            }
            if (!there) {
                atomicOr(pa.error_word, 0x400u);
                return false;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            for (uint32_t i = 0; i < n_late; ++i) xq_copy(late_dst[i], late_src[i], late_bar[i]);
            n_late = 0u;
            xq_seen = true;
            return true;
        };
#pragma unroll 1
        for (uint32_t o = 0; o < nops; ++o) {
            GemvParams plist;
            if constexpr (NOPS == 0) plist = list.ops[o];
            const GemvParams &p = NOPS == 0 ? plist : (o == 0 ? pa : pb);
            const CUtensorMap *tw = NOPS == 0 ? list.maps + 3u * o : (o == 0 ? &tmap_w : &next_w);
            const CUtensorMap *ts = NOPS == 0 ? list.maps + 3u * o + 1u : (o == 0 ? &tmap_s : &next_s);
            const CUtensorMap *tb = NOPS == 0 ? list.maps + 3u * o + 2u : (o == 0 ? &tmap_b : &next_b);
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tw)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(ts)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tb)) : "memory");
            const uint32_t vcta = NOPS == 0 ? range_index(blockIdx.x, p.rot, gridDim.x) : blockIdx.x;
            const uint32_t u_begin = range_begin(vcta, p.units, gridDim.x);
            const uint32_t u_end = range_begin(vcta + 1u, p.units, gridDim.x);
            uint32_t rg = u_begin / p.chunks;
            uint32_t kc = u_begin - rg * p.chunks;
            for (uint32_t u = u_begin; u < u_end && ok; ++u) {
                const uint32_t stage = issued % NST;
                const uint32_t round = issued / NST;
                if constexpr (XQS) {
                    // the ring is full of weights whose activations are still missing (or the very first such stage when
                    // the ring is already turning): now the counter has to be there
                    if (!xq_seen && (n_late == static_cast<uint32_t>(NST) || (round > 0 && n_late != 0u))) ok = flush_late();
                    if (!ok) break;
                }
                if (round > 0) ok = mbar_wait(smem_u32(&s_empty[stage]), (round - 1u) & 1u, p.error_word, 0x1u);
                if (!ok) break;
                const uint32_t full = smem_u32(&s_full[stage]);
                {
                    const uint32_t base = ring + stage * Plan::STAGE;
                    const bool with_x = XQS && p.xq != nullptr;
                    mbar_arrive_expect_tx(full, Geo::STAGE_BYTES + (with_x ? Plan::XQS_UNIT : 0));
#pragma unroll
                    for (int pnl = 0; pnl < kPanels; ++pnl)
                        tma_load_2d(base + pnl * kPanelSize, tw, kc * kChunkBytes + pnl * kPanelBytes, rg * kRows, full);
                    const uint32_t sb_col = (kc * GPS * 2u) & ~15u;
                    tma_load_2d(base + kWeightBytes, ts, sb_col, rg * kRows, full);
                    tma_load_2d(base + kWeightBytes + Geo::SB_BYTES, tb, sb_col, rg * kRows, full);
                    if (with_x) {
                        const uint8_t *src = p.xq + static_cast<size_t>(kc) * Plan::XQS_UNIT;
                        if (xq_seen) {
                            xq_copy(base + Geo::STAGE_BYTES, src, full);
                        } else {
                            // the quantised activations are still being written (start of the launch): the weights of
                            // this stage are on their way; its activations follow once the grid-wide counter is there
                            late_dst[n_late] = base + Geo::STAGE_BYTES, late_src[n_late] = src, late_bar[n_late] = full;
                            ++n_late;
                        }
                    }
                }
                ++issued;
                if (++kc == p.chunks) kc = 0u, ++rg;
            }
        }
        if constexpr (XQS) {
            if (ok && !xq_seen && n_late != 0u) ok = flush_late();
        }
        if (!ok) {
            s_abort = 1u;
            const uint32_t pending = issued < static_cast<uint32_t>(NST) ? issued : static_cast<uint32_t>(NST);
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t idx = issued - 1u - i;
                mbar_wait(smem_u32(&s_full[idx % NST]), (idx / NST) & 1u, pa.error_word, 0x4u);
            }
        } else if constexpr (NOPS == 1) {
            prefetch_next_head(pa, &next_w, &next_s, &next_b);
        }
        return;
    }

    if (warp == NCW + 1) {
        // ------------------------- writer warp -------------------------
        // lane owns rows lane, lane + 32, lane + 64, lane + 96 of the row group
        asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t ob = 0, ophase = 0;
        // fused all-reduce: the exchange epoch of the launch's k-th fused operation is (epoch at launch start) + 1 + k;
        // the epoch word itself moves once, at the very end of the launch, by the number of fused operations
        uint32_t fbase = 0u, nfused = 0u;
        uint32_t *fctl_launch = nullptr;
        FusedOp late = {};                       // an exchange whose wait was put off to the end of the following operation
        uint32_t late_rg[8] = {}, late_n = 0xFFFFFFFFu;
#pragma unroll 1
        for (uint32_t o = 0; o < nops; ++o) {
        GemvParams plist;
        if constexpr (NOPS == 0) plist = list.ops[o];
        const GemvParams &p = NOPS == 0 ? plist : (o == 0 ? pa : pb);
        const uint32_t vcta = NOPS == 0 ? range_index(blockIdx.x, p.rot, gridDim.x) : blockIdx.x;
        const uint32_t u_begin = range_begin(vcta, p.units, gridDim.x);
        const uint32_t u_end = range_begin(vcta + 1u, p.units, gridDim.x);
        const uint32_t rg_begin = u_begin / p.chunks;
        // (a CTA without units of this operation: u_begin = u_end = units, the loop below is empty)
        const uint32_t rg_last_touched = (u_end - 1u) / p.chunks;

        // Fused all-reduce (row-parallel weight under tensor parallelism): the final sums of a row group are
        // not written to y but pushed, as fp32, into slot `my rank` of every rank's exchange region; once all
        // of this CTA's row groups are pushed, it waits for the peers' words of the same row groups, adds the
        // ranks in rank order and writes y.  Early row groups therefore cross NVLink while later ones are
        // still being computed.
        const bool fused = MD <= 4 && p.fuse_size != 0u;   // (the sum over ranks rides in launches of up to four rows)
        uint8_t *my_region = fused ? p.fuse_region[p.fuse_rank] : nullptr;
        uint32_t *fctl = reinterpret_cast<uint32_t *>(my_region + kFusedCtlOff);  // {epoch, done}
        uint32_t fepoch = 0u, fphase = 0u;
        if (fused) {
            if (fctl_launch == nullptr) {
                fctl_launch = fctl;
                fbase = __ldcg(fctl);  // every CTA of this launch reads the same value: it moves only when the whole launch is through
            }
            fepoch = fbase + 1u + nfused;
            fphase = fepoch & static_cast<uint32_t>(kFusedPhases - 1);   // four data phases: an exchange may still be read while the next two are written
            ++nfused;
        }
        constexpr uint32_t kPend = 8;
        uint32_t pend[kPend] = {};
        uint32_t npend = 0u;
        bool peers_ok = true;

        auto store = [&](uint32_t m, uint32_t n, float val) {
            if (m < p.M && n < p.N) {
                if (XF32 || p.y_f32)
                    static_cast<float *>(p.y)[static_cast<size_t>(m) * p.N + n] = val;
                else
                    static_cast<__nv_bfloat16 *>(p.y)[static_cast<size_t>(m) * p.N + n] = __float2bfloat16_rn(val);
            }
        };
        // Exchange words are {fp32 value, launch epoch} in 64 bits, written with one store: a reader that sees
        // the epoch has the value, so there is no flag, no fence and no second NVLink hop (the same idea as
        // the split-K words above, and as the "LL" protocols of collective libraries).
        // wait for every rank's words of row group rg, add them in rank order, write y
        auto finish = [&](const FusedOp &f, uint32_t rg) {
            if constexpr (MD <= 4) {
            const unsigned long long *data = reinterpret_cast<const unsigned long long *>(
                f.region + kFusedDataOff + static_cast<size_t>(f.phase) * kPeerMaxRanks * kPeerSlotBytes);
            float acc[4][MD];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int m = 0; m < MD; ++m) acc[i][m] = 0.f;
            for (uint32_t r = 0; r < f.size; ++r) {
                const unsigned long long *src = data + r * (kPeerSlotBytes / 8u);
                unsigned long long word[4][MD];
                bool got = false;
                for (uint32_t it = 0; it < kPeerPollLimit; ++it) {
                    bool all = true;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t n = rg * kRows + lane + 32u * i;
#pragma unroll
                        for (int m = 0; m < MD; ++m) {
                            if (static_cast<uint32_t>(m) < f.M && n < f.N) {
                                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];"
                                             : "=l"(word[i][m])
                                             : "l"(src + static_cast<size_t>(m) * f.N + n)
                                             : "memory");
                                all = all && static_cast<uint32_t>(word[i][m] >> 32) == f.epoch;
                            } else {
                                word[i][m] = 0ull;
                            }
                        }
                    }
                    if (__all_sync(0xFFFFFFFFu, all)) {
                        got = true;
                        break;
                    }
                    if (it > 64) __nanosleep(it > 4096 ? 1000 : 32);
                }
                if (!got) {
                    if (lane == 0) atomicOr(pa.error_word, 0x200u);
                    peers_ok = false;
                    return;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int m = 0; m < MD; ++m) acc[i][m] += __uint_as_float(static_cast<uint32_t>(word[i][m]));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int m = 0; m < MD; ++m) {
                    const uint32_t n = rg * kRows + lane + 32u * i;
                    if (static_cast<uint32_t>(m) < f.M && n < f.N) {
                        if (XF32 || f.y_f32)
                            static_cast<float *>(f.y)[static_cast<size_t>(m) * f.N + n] = acc[i][m];
                        else
                            static_cast<__nv_bfloat16 *>(f.y)[static_cast<size_t>(m) * f.N + n] = __float2bfloat16_rn(acc[i][m]);
                    }
                }
            }
        };
        const FusedOp cur = {p.y, my_region, p.N, p.M, p.y_f32, p.fuse_size, fepoch, fphase};
        // final sums of row group rg (this rank's share of K): to y, or to the peers
        auto emit = [&](uint32_t rg, const float (&v)[4][MD]) {
            if (!fused) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int m = 0; m < MD; ++m) store(m, rg * kRows + lane + 32u * i, v[i][m]);
                return;
            }
            const size_t slot = kFusedDataOff + (static_cast<size_t>(fphase) * kPeerMaxRanks + p.fuse_rank) * kPeerSlotBytes;
            for (uint32_t j = 0; j < p.fuse_size; ++j) {
                uint32_t r = p.fuse_rank + j;
                if (r >= p.fuse_size) r -= p.fuse_size;
                unsigned long long *dst = reinterpret_cast<unsigned long long *>(p.fuse_region[r] + slot);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t n = rg * kRows + lane + 32u * i;
#pragma unroll
                    for (int m = 0; m < MD; ++m)
                        if (static_cast<uint32_t>(m) < p.M && n < p.N) {
                            const unsigned long long word =
                                (static_cast<unsigned long long>(fepoch) << 32) | __float_as_uint(v[i][m]);
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + static_cast<size_t>(m) * p.N + n), "l"(word)
                                         : "memory");
                        }
                }
            }
            if (npend == kPend) {  // rare: many short row groups per CTA; settle the oldest first
                if (peers_ok) finish(cur, pend[0]);
#pragma unroll
                for (uint32_t i = 0; i + 1u < kPend; ++i) pend[i] = pend[i + 1u];
                --npend;
            }
            pend[npend++] = rg;
        };

        for (uint32_t rg = rg_begin; rg <= rg_last_touched; ++rg) {
            if (!mbar_wait(smem_u32(&s_out_full[ob]), ophase, p.error_word, 0x8u)) return;
            const uint32_t rg_first = rg * p.chunks, rg_last = rg_first + p.chunks - 1u;
            const bool whole = u_begin <= rg_first && rg_last < u_end;
            uint32_t slots = 1u, slot = 0u;
            if (!whole) {
                const uint32_t first_cta = unit_owner(rg_first, p.units, gridDim.x);
                slots = unit_owner(rg_last, p.units, gridDim.x) - first_cta + 1u;
                slot = vcta - first_cta;
            }
            // scratch slot layout [128 rows][8]: the same footprint as the tensor-core kernel's single tile
            float *mine = p.partials + (static_cast<size_t>(rg) * p.max_slots + slot) * (kRows * 8);
            const uint32_t obuf = ring + Plan::OFF_OUT + ob * Plan::OUT_BUF;
            float sum[4][MD];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t row = lane + 32u * i;
                if constexpr (MD > 4) {
                    // four activation rows per load; groups added in the same fixed order
#pragma unroll
                    for (int m4 = 0; m4 < MD; m4 += 4) {
                        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                        for (int gq = 0; gq < GPS; ++gq) {
                            float v0, v1, v2, v3;
                            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                                         : "=f"(v0), "=f"(v1), "=f"(v2), "=f"(v3)
                                         : "r"(obuf + ((gq * kRows + row) * MD + m4) * 4u));
                            a0 += v0, a1 += v1, a2 += v2, a3 += v3;
                        }
                        sum[i][m4] = a0, sum[i][m4 + 1] = a1, sum[i][m4 + 2] = a2, sum[i][m4 + 3] = a3;
                    }
                } else {
#pragma unroll
                for (int m = 0; m < MD; ++m) {
                    float a = 0.f;
#pragma unroll
                    for (int gq = 0; gq < GPS; ++gq) {  // fixed order over the unit's groups
                        float v;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(obuf + ((gq * kRows + row) * MD + m) * 4u));
                        a += v;
                    }
                    sum[i][m] = a;
                }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_out_empty[ob]));
            {
                if (whole) {
                    emit(rg, sum);
                } else if (p.tagged != nullptr) {
                    // Partial sums that carry their own arrival tag: {fp32 value, tag} in one 64-bit word, so
                    // a reader that sees the tag has the value (no flag, no ticket, no fence).  The CTA that
                    // owns the head of the row group (it gets there last, at the end of its range) collects:
                    // own sums + the other slots in slot order, and sets the words back to zero.
                    constexpr uint32_t kTag = 0x5A5A5A5Au;
                    unsigned long long *slots_base = p.tagged + static_cast<size_t>(rg) * p.max_slots * (kRows * MD);
                    if (slot != 0u) {
                        unsigned long long *dst = slots_base + static_cast<size_t>(slot) * (kRows * MD);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int m = 0; m < MD; ++m) {
                                const unsigned long long word =
                                    (static_cast<unsigned long long>(kTag) << 32) | __float_as_uint(sum[i][m]);
                                asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst + (lane + 32u * i) * MD + m), "l"(word) : "memory");
                            }
                    } else {
                        bool got = true;
                        for (uint32_t sidx = 1; sidx < slots && got; ++sidx) {  // fixed order: reproducible sums
                            unsigned long long *src = slots_base + static_cast<size_t>(sidx) * (kRows * MD);
#pragma unroll
                            for (int cb = 0; cb < MD / MQ; ++cb) {   // MQ activation rows at a time (register budget)
                            unsigned long long word[4][MQ];
                            got = false;
                            for (uint32_t it = 0; it < kWaitLimit; ++it) {
                                bool all = true;
#pragma unroll
                                for (int i = 0; i < 4; ++i)
#pragma unroll
                                    for (int m = 0; m < MQ; ++m) {
                                        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word[i][m]) : "l"(src + (lane + 32u * i) * MD + cb * MQ + m) : "memory");
                                        all = all && static_cast<uint32_t>(word[i][m] >> 32) == kTag;
                                    }
                                if (__all_sync(0xFFFFFFFFu, all)) {
                                    got = true;
                                    break;
                                }
                                if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
                            }
                            if (!got) {
                                if (lane == 0) atomicOr(p.error_word, 0x20u);
                                break;
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i)
#pragma unroll
                                for (int m = 0; m < MQ; ++m) {
                                    sum[i][cb * MQ + m] += __uint_as_float(static_cast<uint32_t>(word[i][m]));
                                    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(src + (lane + 32u * i) * MD + cb * MQ + m), "l"(0ull) : "memory");
                                }
                            }
                        }
                        if (got) emit(rg, sum);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int m = 0; m < MD; ++m) mine[(lane + 32u * i) * 8 + m] = sum[i][m];
                    __syncwarp();
                    unsigned int ticket = 0;
                    if (lane == 0)
                        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.counters + rg) : "memory");
                    ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
                    if (ticket == slots - 1u) {
                        const float *all = p.partials + static_cast<size_t>(rg) * p.max_slots * (kRows * 8);
                        float tot[4][MD];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int m = 0; m < MD; ++m) tot[i][m] = 0.f;
                        for (uint32_t sidx = 0; sidx < slots; ++sidx) {  // fixed order: reproducible sums
#pragma unroll
                            for (int i = 0; i < 4; ++i)
#pragma unroll
                                for (int m = 0; m < MD; ++m)
                                    tot[i][m] += __ldcg(all + static_cast<size_t>(sidx) * (kRows * 8) + (lane + 32u * i) * 8 + m);
                        }
                        emit(rg, tot);
                        if (lane == 0) p.counters[rg] = 0u;
                    }
                }
            }
            if constexpr (Plan::NOB == 2) {
                ob ^= 1u;
                if (ob == 0u) ophase ^= 1u;
            } else {
                ophase ^= 1u;
            }
        }
        // this CTA's share of operation `op`'s output is stored (or handed to the head owner, who stores it
        // before it arrives here itself): arrive at the operation's grid-wide counter.  After the last
        // operation the counter only finds the last CTA, which zeroes all of them for the next launch.
        auto arrive_op = [&](uint32_t op) {
            if (NOPS != 1) {
                __syncwarp();
                if (lane == 0) {
                    unsigned int t;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(t) : "l"(gbar + op) : "memory");
                    if (op == nops - 1u && t == gridDim.x - 1u)
                        for (uint32_t i = 0; i <= nops; ++i) gbar[i] = 0u;   // [nops]: the quantised-activations counter
                }
            }
        };
        // an exchange put off at the end of the previous operation: by now its words have had this whole operation's
        // streaming time to cross NVLink
        if (late_n != 0xFFFFFFFFu) {
            for (uint32_t i = 0; i < late_n; ++i)
                if (peers_ok) finish(late, late_rg[i]);
            arrive_op(o - 1u);
            late_n = 0xFFFFFFFFu;
        }
        bool put_off = false;
        if (fused) {
            // Launch lists: when the next operation does not read what this launch writes, this operation's wait for
            // the peers moves to the end of the next one (and with it the arrival at its counter), so the NVLink
            // latency hides behind that operation's streaming instead of stalling the write-out here.
            if constexpr (NOPS == 0) put_off = o + 1u < nops && list.ops[o + 1u].dep == 0u;
            if (put_off) {
                late = cur;
                late_n = npend;
#pragma unroll
                for (uint32_t i = 0; i < kPend; ++i) late_rg[i] = pend[i];
            } else {
                for (uint32_t i = 0; i < npend; ++i)
                    if (peers_ok) finish(cur, pend[i]);
            }
        }
        if (!put_off) arrive_op(o);
        }  // operations
        if (fctl_launch != nullptr) {
            // the exchange epoch moves once per launch, when the launch's last CTA is through all its operations
            __syncwarp();
            if (lane == 0) {
                __threadfence();
                const uint32_t t = atomicAdd(fctl_launch + 1, 1u);
                if (t == gridDim.x - 1u) {
                    fctl_launch[1] = 0u;
                    __threadfence();
                    fctl_launch[0] = fbase + nfused;
                }
            }
        }
        return;
    }

    // --------------------------- consumer warps ---------------------------
    const uint32_t gq = warp % GPS;          // group of the unit this warp works on
    const uint32_t rbase = (warp / GPS) * RW;  // first of its rows
    constexpr uint32_t block_units = BU;

    // shared-memory offsets of this lane's rows: first 16-byte chunk of the group, swizzled
    uint32_t woff[R], sboff[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const uint32_t row = rbase + lane + 32u * i;
        const uint32_t ob = gq * GB;              // byte offset of the group inside the unit's 256 bytes
        const uint32_t pnl = ob / kPanelBytes, inp = ob % kPanelBytes;
        woff[i] = ring + pnl * kPanelSize + row * kPanelBytes + ((((inp >> 4) ^ row) & 7u) << 4);
        sboff[i] = ring + kWeightBytes + row * Geo::SBOX + gq * 2u;
    }
    const uint32_t xq_warp = ring + Plan::OFF_XQ + gq * Plan::XQ_GROUP;
    const uint32_t xi_warp = ring + Plan::OFF_XI + gq * MD * 8u;
    const uint32_t out_warp = ring + Plan::OFF_OUT + gq * (kRows * MD * 4u);

    float yacc[R][MD];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int m = 0; m < MD; ++m) yacc[i][m] = 0.f;

    // int8-MMA variant: quad layout of the MMA fragments.  Accumulator rows g, g + 8 of a 16-row block are
    // weight rows wr, wr + 8 (wr = rho(g): the permutation that keeps the swizzled loads conflict free).
    const uint32_t qg = lane >> 2, qt = lane & 3;
    const uint32_t wr = rho<GB / 4>(qg);
    uint32_t aoff[IM ? NRB : 1], sbim[IM ? NRB : 1];
    float yim[IM ? NRB : 1][2 * NB];
    if constexpr (IM) {
#pragma unroll
        for (int rb = 0; rb < NRB; ++rb) {
            const uint32_t row = rbase + rb * 16u + wr;
            const uint32_t obyte = gq * GB + qt * (GB / 4);   // this lane's bytes of the group inside the unit row
            const uint32_t pnl = obyte / kPanelBytes, inp = obyte % kPanelBytes;
            aoff[rb] = ring + pnl * kPanelSize + row * kPanelBytes + ((((inp >> 4) ^ row) & 7u) << 4) + (inp & 15u);
            sbim[rb] = ring + kWeightBytes + row * Geo::SBOX + gq * 2u;
#pragma unroll
            for (int c2 = 0; c2 < 2 * NB; ++c2) yim[rb][c2] = 0.f;
        }
    }

    uint32_t stage = 0, phase = 0;   // ring position and out-buffer position run on across operations
    uint32_t ob = 0, ophase = 0;
    bool alive = true;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (XQS) {
        // ---- the launch's activations, quantised ONCE: the (operation, K chunk) pairs are dealt round-robin to the
        // CTAs, each writes its pairs' quantised units to global memory, then arrives at a grid-wide counter; the copy
        // warps wait for that counter before their first copy of such a unit.  Afterwards an operation's activations
        // arrive with its weights, stage by stage: no per-CTA rebuild, no CTA barrier between operations.
        if (list.xq_pairs != 0u) {
            constexpr int G = GB * 8 / BITS, PER = G / 32;
            // task = (pair, group of the unit, activation row): one warp each, dealt over all consumer warps of the grid
            const uint32_t ntasks = list.xq_pairs * GPS * MD, stride = gridDim.x * NCW;
#pragma unroll 1
            for (uint32_t task = blockIdx.x * NCW + warp; task < ntasks; task += stride) {
                const uint32_t m = task % MD, gl = (task / MD) % GPS, j = task / (MD * GPS);
                const XqPair pr = list.xq_tab[j];
                const __nv_bfloat16 *qx = static_cast<const __nv_bfloat16 *>(pr.x);
                uint8_t *dst = pr.dst;
                const uint32_t kc = pr.kc, qgroups = pr.groups, qK = pr.K, qM = pr.M;
                const uint32_t gi = kc * GPS + gl;
                const bool live = gi < qgroups && m < qM;   // rows the instance has room for but the call does not use: zeros
                float xv[PER];
#pragma unroll
                for (int e = 0; e < PER; ++e)
                    xv[e] = live ? __bfloat162float(qx[static_cast<size_t>(m) * qK + static_cast<size_t>(gi) * G + lane * PER + e]) : 0.f;
                uint32_t abits = 0u;
#pragma unroll
                for (int e = 0; e < PER; ++e) abits = max(abits, __float_as_uint(xv[e]) & 0x7FFFFFFFu);
                abits = __reduce_max_sync(0xFFFFFFFFu, abits);
                const uint32_t eb = abits >> 23;   // same rule as the per-CTA quantiser below
                const bool nz = eb >= 27u && eb < 255u;
                const float up = nz ? __uint_as_float((265u - eb) << 23) : 0.f;
                const float down = nz ? __uint_as_float((eb - 11u) << 23) : 0.f;
                int isum = 0;
#pragma unroll
                for (int e = 0; e < PER; ++e) {
                    int xi = __float_as_int(fmaf(xv[e], up, 12582912.f)) - 0x4B400000;
                    xi = max(-4095, min(4095, xi));
                    isum += xi;
                    const uint32_t k = lane * PER + e;
                    const uint32_t wj = k >> 3, odd = k & 1u, bytepos = (k & 7u) >> 1;
                    if constexpr (IM && BITS == 8) {
                        const uint32_t w8 = k >> 2, t8 = w8 / WPT, wl = w8 % WPT;   // (the layout the per-CTA quantiser writes)
                        uint8_t *a = dst + gl * Plan::XQ_GROUP + ((wl >> 1) * NB + m / 4u) * 256u + ((2u * (m % 4u)) * 4u + t8) * 8u +
                                     (wl & 1u) * 4u + (k & 3u);
                        a[0] = static_cast<uint8_t>((xi >> 6) & 0xFF);
                        a[32] = static_cast<uint8_t>(xi & 63);
                    } else if constexpr (IM) {
                        // B registers of MMA (wj % WPT) for the quad lane (wj / WPT): 8 bytes {even, odd} per (column, quad
                        // lane), column 2m = hi limb, 2m + 1 = lo limb (the layout the per-CTA quantiser writes)
                        uint8_t *a = dst + gl * Plan::XQ_GROUP + ((wj % WPT) * NB + m / 4u) * 256u + ((2u * (m % 4u)) * 4u + wj / WPT) * 8u +
                                     odd * 4u + bytepos;
                        a[0] = static_cast<uint8_t>((xi >> 6) & 0xFF);
                        a[32] = static_cast<uint8_t>(xi & 63);
                    } else if constexpr (BITS == 8) {
                        uint8_t *a = dst + gl * Plan::XQ_GROUP + ((k >> 2) * MD + m) * 8u + (k & 3u);   // {hi, lo} x 4 bytes per word of four codes
                        a[0] = static_cast<uint8_t>((xi >> 6) & 0xFF);
                        a[4] = static_cast<uint8_t>(xi & 63);
                    } else {
                        uint8_t *a = dst + gl * Plan::XQ_GROUP + (wj * MD + m) * 16u + odd * 4u + bytepos;   // {even hi, odd hi, even lo, odd lo} x 4 bytes
                        a[0] = static_cast<uint8_t>((xi >> 6) & 0xFF);
                        a[8] = static_cast<uint8_t>(xi & 63);
                    }
                }
                isum = __reduce_add_sync(0xFFFFFFFFu, isum);
                if (lane == 0)
                    *reinterpret_cast<float2 *>(dst + Plan::XQ_UNIT + (gl * MD + m) * 8u) = make_float2(down, static_cast<float>(isum) * down);
            }
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (warp == 0 && lane == 0) {
                __threadfence();
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gbar + nops) : "memory");
            }
        }
    }
#pragma unroll 1
    for (uint32_t o = 0; o < nops; ++o) {
    GemvParams plist;
    if constexpr (NOPS == 0) plist = list.ops[o];
    const GemvParams &p = NOPS == 0 ? plist : (o == 0 ? pa : pb);
    const uint8_t *xbase = static_cast<const uint8_t *>(p.x);
    const uint32_t vcta = NOPS == 0 ? range_index(blockIdx.x, p.rot, gridDim.x) : blockIdx.x;
    const uint32_t u_begin = range_begin(vcta, p.units, gridDim.x);
    const uint32_t u_end = range_begin(vcta + 1u, p.units, gridDim.x);
    const uint32_t rg_begin = u_begin / p.chunks;
    const uint32_t kc_begin = u_begin - rg_begin * p.chunks;
    // opx: this operation's activations were quantised at the start of the launch and arrive with every stage: no
    // block to build, nothing to wait for between operations
    const bool opx = XQS && p.xq != nullptr;
    if (NOPS != 1 && !opx) {
        if (o > 0) {
            // all warps are done reading the previous operation's activation blocks, and (when this operation reads
            // what the previous one wrote) the previous operation's output is complete on every CTA
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (p.dep != 0u && warp == 0 && lane == 0) {
                bool ok = false;
                for (uint32_t it = 0; it < kWaitLimit; ++it) {
                    unsigned int v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(gbar + (o - 1u)) : "memory");
                    if (v >= gridDim.x) {
                        ok = true;
                        break;
                    }
                    if (it > 32) __nanosleep(it > 4096 ? 256 : 32);
                }
                if (!ok) {
                    atomicOr(pa.error_word, 0x40u);
                    s_abort = 1u;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (s_abort) return;
        }
    }

    // ---- quantised activations for a block of units: (unit, group, activation row) triples over the warps ----
    // Two passes so that all of a warp's global loads are in flight together.
    auto prep_block = [&](auto act_c, uint32_t kc_first, uint32_t count, uint32_t buf) {
        constexpr bool ACT = decltype(act_c)::value;  // compile-time: the plain path keeps its loads branch-free
        if constexpr (IM && BITS == 4 && !ACT && !XF32) {
            // Four activation rows: a lane takes one packed word's worth (8 consecutive elements, one 16-byte
            // load) of one (unit, group, activation row); the G/8 lanes of a row reduce among themselves.  The
            // word's {even, odd} byte pairs are exactly one lane's B registers of one MMA.
            constexpr int G = GB * 2, WG = G / 8;              // words per group: 4, 8, 16
            constexpr int TASKS = BU * GPS * MD * WG;          // per block, at most
            constexpr int IT = (TASKS + NCW * 32 - 1) / (NCW * 32);
            const uint32_t ntask = count * GPS * MD * WG;
            const uint32_t gmask = ((WG == 32 ? 0u : (1u << WG)) - 1u) << (lane & ~(WG - 1));
            uint4 v[IT];
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const uint32_t id = (it * NCW + warp) * 32u + lane;
                const uint32_t wd = id % WG, m = (id / WG) % MD, gl = (id / (WG * MD)) % GPS, ubk = id / (WG * MD * GPS);
                const uint32_t gi = ((kc_first + ubk) % p.chunks) * GPS + gl;
                v[it] = make_uint4(0u, 0u, 0u, 0u);
                if (id < ntask && m < p.M && gi < p.groups)
                    v[it] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(xbase) +
                                                             static_cast<size_t>(m) * p.K + static_cast<size_t>(gi) * G + wd * 8u);
            }
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const uint32_t id = (it * NCW + warp) * 32u + lane;
                const uint32_t wd = id % WG, m = (id / WG) % MD, gl = (id / (WG * MD)) % GPS, ubk = id / (WG * MD * GPS);
                const uint32_t w4[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
                uint32_t amax = 0u;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t a = w4[e] & 0x7FFF7FFFu;  // two bf16 magnitudes: they order like integers
                    amax = max(amax, max(a & 0xFFFFu, a >> 16));
                }
                amax = __reduce_max_sync(gmask, amax);
                const uint32_t eb = amax >> 7;                     // biased exponent of the group's largest |x|
                const bool nz = eb >= 27u && eb < 255u;
                const float up = nz ? __uint_as_float((265u - eb) << 23) : 0.f;    // 2^(12 - E), E = eb - 126
                const float down = nz ? __uint_as_float((eb - 11u) << 23) : 0.f;   // 2^(E - 12)
                int isum = 0;
                uint32_t ehi = 0u, ohi = 0u, elo = 0u, olo = 0u;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int xe = __float_as_int(fmaf(__uint_as_float(w4[e] << 16), up, 12582912.f)) - 0x4B400000;          // element 2e
                    int xo = __float_as_int(fmaf(__uint_as_float(w4[e] & 0xFFFF0000u), up, 12582912.f)) - 0x4B400000;  // 2e + 1
                    xe = max(-4095, min(4095, xe));
                    xo = max(-4095, min(4095, xo));
                    isum += xe + xo;
                    ehi |= (static_cast<uint32_t>(xe >> 6) & 0xFFu) << (8 * e);
                    elo |= (static_cast<uint32_t>(xe) & 63u) << (8 * e);
                    ohi |= (static_cast<uint32_t>(xo >> 6) & 0xFFu) << (8 * e);
                    olo |= (static_cast<uint32_t>(xo) & 63u) << (8 * e);
                }
                isum = __reduce_add_sync(gmask, isum);
                if (id < ntask) {
                    const uint32_t qb = ring + Plan::OFF_XQ + (buf * BU + ubk) * Plan::XQ_UNIT + gl * Plan::XQ_GROUP;
                    // MMA (wd % WPT), column set m / 4: 256 bytes = 8 columns x 4 quad lanes x {even, odd} words
                    const uint32_t a = qb + ((wd % WPT) * NB + m / 4u) * 256u + ((2u * (m % 4u)) * 4u + wd / WPT) * 8u;
                    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(ehi), "r"(ohi) : "memory");
                    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a + 32u), "r"(elo), "r"(olo) : "memory");
                    if (wd == 0u) {
                        const uint32_t xa = ring + Plan::OFF_XI + (buf * BU + ubk) * Plan::XI_UNIT + (gl * MD + m) * 8u;
                        asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(xa), "f"(down), "f"(static_cast<float>(isum) * down) : "memory");
                    }
                }
            }
            return;
        }
        constexpr int G = GB * 8 / BITS;                   // elements per group
        constexpr int PER = G / 32;                        // elements per lane: 1 (G=32), 2, 4
        constexpr int TPW = (BU * GPS * MD + NCW - 1) / NCW;  // triples per warp, at most
        float xv[TPW][PER];
        const uint32_t ntask = count * GPS * MD;
#pragma unroll
        for (int tk = 0; tk < TPW; ++tk) {
            const uint32_t pi = warp + tk * NCW;
            const uint32_t m = pi % MD, gl = (pi / MD) % GPS, ub = pi / (MD * GPS);
            const uint32_t gi = ((kc_first + ub) % p.chunks) * GPS + gl;
            const bool live = pi < ntask && m < p.M && gi < p.groups;
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const size_t idx = static_cast<size_t>(m) * p.K + static_cast<size_t>(gi) * G + lane * PER + e;
                float v = 0.f;
                if (live) {
                    if constexpr (ACT) {
                        // x = silu(gate) * up, gate and up the two halves of the previous operation's fp32 output
                        // (written by other SMs during this launch: read through L2)
                        const size_t gidx = static_cast<size_t>(m) * 2u * p.K + static_cast<size_t>(gi) * G + lane * PER + e;
                        const float gt = __ldcg(reinterpret_cast<const float *>(xbase) + gidx);
                        const float up = __ldcg(reinterpret_cast<const float *>(xbase) + gidx + p.K);
                        v = gate_activation(gt, p.act) * up;
                    } else if constexpr (XF32) {
                        v = reinterpret_cast<const float *>(xbase)[idx];
                    } else {
                        v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(xbase)[idx]);
                    }
                }
                xv[tk][e] = v;
            }
        }
#pragma unroll
        for (int tk = 0; tk < TPW; ++tk) {
            const uint32_t pi = warp + tk * NCW;
            if (pi >= ntask) break;
            const uint32_t m = pi % MD, gl = (pi / MD) % GPS, ub = pi / (MD * GPS);
            // largest |x| of the group: non-negative floats order like their bit patterns
            uint32_t abits = 0u;
#pragma unroll
            for (int e = 0; e < PER; ++e) abits = max(abits, __float_as_uint(xv[tk][e]) & 0x7FFFFFFFu);
            abits = __reduce_max_sync(0xFFFFFFFFu, abits);
            // amax = 1.f * 2^(eb - 127) < 2^E with E = eb - 126; xi = rint(x * 2^(12-E)), |xi| <= 4095.
            // Groups whose largest value is below 2^-100 (or not finite) count as zero.
            const uint32_t eb = abits >> 23;
            const bool nz = eb >= 27u && eb < 255u;
            const float up = nz ? __uint_as_float((265u - eb) << 23) : 0.f;    // 2^(12 - E)
            const float down = nz ? __uint_as_float((eb - 11u) << 23) : 0.f;   // 2^(E - 12)
            const uint32_t qb = ring + Plan::OFF_XQ + (buf * BU + ub) * Plan::XQ_UNIT + gl * Plan::XQ_GROUP;
            int isum = 0;
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                int xi = __float_as_int(fmaf(xv[tk][e], up, 12582912.f)) - 0x4B400000;  // rint without a conversion instruction
                xi = max(-4095, min(4095, xi));
                isum += xi;
                const int hi = xi >> 6, lo = xi & 63;
                // element k of the group -> word k/8, even/odd nibble word, byte (k%8)/2
                const uint32_t k = lane * PER + e;
                const uint32_t wj = k >> 3, odd = k & 1u, bytepos = (k & 7u) >> 1;
                // 16 bytes per (word, activation row): {even hi, odd hi, even lo, odd lo} x 4 bytes
                if constexpr (IM && BITS == 8) {
                    // 8-bit codes: a lane's WPT words of the group row feed WPT / 2 MMAs, two words each (A registers
                    // {a0, a1} = word 2 jj of rows g / g + 8, {a2, a3} = word 2 jj + 1); element k = byte k % 4 of word k / 4
                    const uint32_t w8 = k >> 2, t8 = w8 / WPT, wl = w8 % WPT;
                    const uint32_t a = qb + ((wl >> 1) * NB + m / 4u) * 256u + ((2u * (m % 4u)) * 4u + t8) * 8u + (wl & 1u) * 4u + (k & 3u);
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(hi & 0xFF) : "memory");
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a + 32u), "r"(lo & 0xFF) : "memory");
                } else if constexpr (IM) {
                    // B registers of MMA (wj % WPT) for the quad lane (wj / WPT): 8 bytes {even, odd} per
                    // (column, quad lane), column 2m = hi limb, 2m + 1 = lo limb
                    const uint32_t a = qb + ((wj % WPT) * NB + m / 4u) * 256u + ((2u * (m % 4u)) * 4u + wj / WPT) * 8u + odd * 4u + bytepos;
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(hi & 0xFF) : "memory");
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a + 32u), "r"(lo & 0xFF) : "memory");
                } else if constexpr (BITS == 8) {
                    // element k of the group -> word k / 4, byte k % 4: 8 bytes per (word, activation row): {hi, lo} x 4
                    const uint32_t a = qb + ((k >> 2) * MD + m) * 8u + (k & 3u);
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(hi & 0xFF) : "memory");
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a + 4u), "r"(lo & 0xFF) : "memory");
                } else {
                    const uint32_t a = qb + (wj * MD + m) * 16u + odd * 4u + bytepos;
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(hi & 0xFF) : "memory");
                    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a + 8u), "r"(lo & 0xFF) : "memory");
                }
            }
            // sum of the quantised activations (exact in integers): the bias term then matches the
            // dot products, y = sum_k (s q_k + b) * xq_k
            isum = __reduce_add_sync(0xFFFFFFFFu, isum);
            const float ssum = static_cast<float>(isum) * down;
            if (lane == 0) {
                const uint32_t a = ring + Plan::OFF_XI + (buf * BU + ub) * Plan::XI_UNIT + (gl * MD + m) * 8u;
                asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(a), "f"(down), "f"(ssum) : "memory");
            }
        }
    };

    // When a row of K fits the two activation buffers taken together (K / 512 <= 2 BU), they are filled here
    // with every K chunk, in the order this CTA meets them; later row groups reuse them and nothing is rebuilt.
    const bool whole_k = opx || p.chunks <= 2u * block_units;
    const uint32_t block_len = whole_k ? p.chunks : block_units;
    if (!opx) {
        const uint32_t total = u_end - u_begin;
        const uint32_t first = total < block_len ? total : block_len;
        const uint32_t head = first < block_units ? first : block_units;
        if (NOPS != 1 && p.act != 0u) {
            prep_block(std::true_type{}, kc_begin, head, 0u);
            if (first > head) prep_block(std::true_type{}, (kc_begin + head) % p.chunks, first - head, 1u);
        } else {
            prep_block(std::false_type{}, kc_begin, head, 0u);
            if (first > head) prep_block(std::false_type{}, (kc_begin + head) % p.chunks, first - head, 1u);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    }
    uint32_t rg = rg_begin, kc = kc_begin;
    uint32_t ub = 0, buf = 0;
    for (uint32_t u = u_begin; u < u_end; ++u) {
        const bool more = u + 1u < u_end;
        uint32_t kc_n = kc + 1u, rg_n = rg;
        if (kc_n == p.chunks) kc_n = 0u, ++rg_n;

        bool landed = false;
        if (alive) {
            landed = mbar_wait(smem_u32(&s_full[stage]), phase, p.error_word, 0x2u);
            if (!landed) alive = false, s_abort = 1u;
        }
        const bool exists = kc * GPS + gq < p.groups;  // the last K chunk of a row may hold fewer groups
        if constexpr (IM) {
            if (landed && exists) {
                const uint32_t stage_off = stage * Plan::STAGE;
                const uint32_t xq = (opx ? ring + stage_off + Geo::STAGE_BYTES + gq * Plan::XQ_GROUP
                                         : xq_warp + (buf * BU + ub) * Plan::XQ_UNIT) + lane * 8u;
                constexpr int NMMA = BITS == 4 ? WPT : WPT / 2;   // MMAs per group: 32 codes each
                uint32_t bfr[NB][NMMA][2];  // this group's B registers, kept for all row blocks
#pragma unroll
                for (int cs = 0; cs < NB; ++cs)
#pragma unroll
                    for (int j = 0; j < NMMA; ++j)
                        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(bfr[cs][j][0]), "=r"(bfr[cs][j][1]) : "r"(xq + (j * NB + cs) * 256u));
                float ex[NB], xs[NB];  // activation rows 4 cs + qt
#pragma unroll
                for (int cs = 0; cs < NB; ++cs)
                    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];"
                                 : "=f"(ex[cs]), "=f"(xs[cs])
                                 : "r"((opx ? ring + stage_off + Geo::STAGE_BYTES + Plan::XQ_UNIT + gq * MD * 8u
                                            : xi_warp + (buf * BU + ub) * Plan::XI_UNIT) + (cs * 4u + qt) * 8u));
                const uint32_t sbo = (kc * GPS * 2u) & 15u;
#pragma unroll
                for (int rb = 0; rb < NRB; ++rb) {
                    uint32_t wa[WPT], wb[WPT];
                    lds_row<WPT>(stage_off + aoff[rb], wr, wa);
                    lds_row<WPT>(stage_off + aoff[rb] + 8u * kPanelBytes, wr, wb);
                    int c[NB][4];
#pragma unroll
                    for (int cs = 0; cs < NB; ++cs) c[cs][0] = c[cs][1] = c[cs][2] = c[cs][3] = 0;
                    if constexpr (BITS == 8) {
                        // the code bytes ARE the A registers: no unpacking at all
#pragma unroll
                        for (int j = 0; j < NMMA; ++j)
#pragma unroll
                            for (int cs = 0; cs < NB; ++cs)
                                mma_u8s8_16832(c[cs], wa[2 * j], wb[2 * j], wa[2 * j + 1], wb[2 * j + 1], bfr[cs][j][0], bfr[cs][j][1]);
                    } else {
#pragma unroll
                    for (int j = 0; j < WPT; ++j) {
                        const uint32_t a0 = wa[j] & 0x0F0F0F0Fu, a1 = wb[j] & 0x0F0F0F0Fu;
                        const uint32_t a2 = (wa[j] >> 4) & 0x0F0F0F0Fu, a3 = (wb[j] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                        for (int cs = 0; cs < NB; ++cs) mma_u8s8_16832(c[cs], a0, a1, a2, a3, bfr[cs][j][0], bfr[cs][j][1]);
                    }
                    }
                    uint16_t s0r, b0r, s1r, b1r;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s0r) : "r"(stage_off + sbim[rb] + sbo));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(b0r) : "r"(stage_off + sbim[rb] + sbo + Geo::SB_BYTES));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s1r) : "r"(stage_off + sbim[rb] + sbo + 8u * Geo::SBOX));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(b1r) : "r"(stage_off + sbim[rb] + sbo + 8u * Geo::SBOX + Geo::SB_BYTES));
                    const float s0 = sb_half<SD>(s0r, 0), b0 = sb_half<SD>(b0r, 0);
                    const float s1 = sb_half<SD>(s1r, 0), b1 = sb_half<SD>(b1r, 0);
                    // columns 2 qt (hi) and 2 qt + 1 (lo): y += s 2^(E-12) (64 hi + lo) + b 2^(E-12) sum(xi)
#pragma unroll
                    for (int cs = 0; cs < NB; ++cs) {
                        yim[rb][2 * cs] = fmaf(limbs_to_float(c[cs][0], c[cs][1]), s0 * ex[cs], fmaf(b0, xs[cs], yim[rb][2 * cs]));
                        yim[rb][2 * cs + 1] = fmaf(limbs_to_float(c[cs][2], c[cs][3]), s1 * ex[cs], fmaf(b1, xs[cs], yim[rb][2 * cs + 1]));
                    }
                }
            }
        } else
        if (landed && exists) {
            const uint32_t stage_off = stage * Plan::STAGE;
            // packed codes of this lane's rows
            uint32_t w[R][WPG];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int c = 0; c < CH; ++c)
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(w[i][4 * c]), "=r"(w[i][4 * c + 1]), "=r"(w[i][4 * c + 2]), "=r"(w[i][4 * c + 3])
                                 : "r"(stage_off + (woff[i] ^ (static_cast<uint32_t>(c) << 4))));
            int ahi[R][MD], alo[R][MD];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int m = 0; m < MD; ++m) ahi[i][m] = 0, alo[i][m] = 0;
            // quantised activations: of this unit, beside its weights in the stage (opx), or of the CTA's current block
            const uint32_t xq = opx ? ring + stage_off + Geo::STAGE_BYTES + gq * Plan::XQ_GROUP
                                    : xq_warp + (buf * BU + ub) * Plan::XQ_UNIT;
#pragma unroll
            for (int j = 0; j < WPG; ++j) {
                if constexpr (BITS == 8) {
                    // a packed word IS four unsigned bytes: two dot products per word and row, no unpacking at all
                    uint32_t x_hi[MD], x_lo[MD];
#pragma unroll
                    for (int m = 0; m < MD; ++m)
                        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(x_hi[m]), "=r"(x_lo[m]) : "r"(xq + (j * MD + m) * 8u));
#pragma unroll
                    for (int i = 0; i < R; ++i)
#pragma unroll
                        for (int m = 0; m < MD; ++m) {
                            ahi[i][m] = dp4a_u8s8(w[i][j], x_hi[m], ahi[i][m]);
                            alo[i][m] = dp4a_u8s8(w[i][j], x_lo[m], alo[i][m]);
                        }
                } else {
                uint32_t xe_hi[MD], xo_hi[MD], xe_lo[MD], xo_lo[MD];
#pragma unroll
                for (int m = 0; m < MD; ++m)
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(xe_hi[m]), "=r"(xo_hi[m]), "=r"(xe_lo[m]), "=r"(xo_lo[m])
                                 : "r"(xq + (j * MD + m) * 16u));
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const uint32_t even = w[i][j] & 0x0F0F0F0Fu, odd = (w[i][j] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                    for (int m = 0; m < MD; ++m) {
                        ahi[i][m] = dp4a_u8s8(even, xe_hi[m], ahi[i][m]);
                        ahi[i][m] = dp4a_u8s8(odd, xo_hi[m], ahi[i][m]);
                        alo[i][m] = dp4a_u8s8(even, xe_lo[m], alo[i][m]);
                        alo[i][m] = dp4a_u8s8(odd, xo_lo[m], alo[i][m]);
                    }
                }
                }
            }
            float ex[MD], xs[MD];
            const uint32_t xi = opx ? ring + stage_off + Geo::STAGE_BYTES + Plan::XQ_UNIT + gq * MD * 8u
                                    : xi_warp + (buf * BU + ub) * Plan::XI_UNIT;
#pragma unroll
            for (int m = 0; m < MD; ++m)
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(ex[m]), "=f"(xs[m]) : "r"(xi + m * 8u));
            const uint32_t sbo = (kc * GPS * 2u) & 15u;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                uint16_t sraw, braw;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sraw) : "r"(stage_off + sboff[i] + sbo));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(braw) : "r"(stage_off + sboff[i] + sbo + Geo::SB_BYTES));
                const float s = sb_half<SD>(sraw, 0), b = sb_half<SD>(braw, 0);
#pragma unroll
                for (int m = 0; m < MD; ++m) {
                    const float v = limbs_to_float(ahi[i][m], alo[i][m]);
                    yacc[i][m] = fmaf(v, s * ex[m], yacc[i][m]);
                    yacc[i][m] = fmaf(b, xs[m], yacc[i][m]);
                }
            }
        }
        __syncwarp();
        if (landed && lane == 0) mbar_arrive(smem_u32(&s_empty[stage]));
        if (++stage == NST) stage = 0u, phase ^= 1u;

        // ---- end of this CTA's share of the row group: hand the sums to the writer warp ----
        if ((kc + 1u == p.chunks) || !more) {
            if (alive && !mbar_wait(smem_u32(&s_out_empty[ob]), ophase ^ 1u, p.error_word, 0x10u)) alive = false, s_abort = 1u;
            if (alive) {
                if constexpr (IM) {
#pragma unroll
                    for (int rb = 0; rb < NRB; ++rb) {
                        const uint32_t row = rbase + rb * 16u + wr;
#pragma unroll
                        for (int cs = 0; cs < NB; ++cs) {
                            asm volatile("st.shared.f32 [%0], %1;" ::"r"(out_warp + ob * Plan::OUT_BUF + (row * MD + cs * 4u + qt) * 4u), "f"(yim[rb][2 * cs]) : "memory");
                            asm volatile("st.shared.f32 [%0], %1;" ::"r"(out_warp + ob * Plan::OUT_BUF + ((row + 8u) * MD + cs * 4u + qt) * 4u), "f"(yim[rb][2 * cs + 1]) : "memory");
                            yim[rb][2 * cs] = yim[rb][2 * cs + 1] = 0.f;
                        }
                    }
                } else {
#pragma unroll
                for (int i = 0; i < R; ++i)
#pragma unroll
                    for (int m = 0; m < MD; ++m)
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(out_warp + ob * Plan::OUT_BUF +
                                                                        ((rbase + lane + 32u * i) * MD + m) * 4u),
                                     "f"(yacc[i][m])
                                     : "memory");
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_out_full[ob]));
            }
            if constexpr (Plan::NOB == 2) {
                ob ^= 1u;
                if (ob == 0u) ophase ^= 1u;
            } else {
                ophase ^= 1u;
            }
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int m = 0; m < MD; ++m) yacc[i][m] = 0.f;
        }

        if (++ub == block_len) {
            ub = 0u;
            if (more && !whole_k) {
                const uint32_t left = u_end - (u + 1u);
                if (NOPS != 1 && p.act != 0u)
                    prep_block(std::true_type{}, kc_n, left < block_units ? left : block_units, buf ^ 1u);
                else
                    prep_block(std::false_type{}, kc_n, left < block_units ? left : block_units, buf ^ 1u);
                asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
                if (s_abort) return;
                buf ^= 1u;
            }
        }
        kc = kc_n, rg = rg_n;
    }
    }  // operations
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

// Embedding rows: block = one requested row, threads walk its packed words.
// (quant * scale + bias) * multiplier, as core/src/compute/cuda/kernels/ops/quant_ops.cu:43.
__global__ void __launch_bounds__(256)
gaf_gather_dequant_f32_kernel(const uint8_t *packed, const uint16_t *scales, const uint16_t *biases,
                              const uint32_t *ids, float multiplier, float *out, uint32_t N, uint32_t K,
                              uint32_t group, uint32_t bits, uint32_t sdtype, uint32_t row_bytes, uint32_t groups) {
    const uint32_t n = ids[blockIdx.x];
    if (n >= N) return;  // ids are validated on the host; never read outside the table
    const uint32_t vpw = 32u / bits;
    const uint32_t words = K / vpw;
    const uint32_t mask = bits == 4 ? 0xFu : 0xFFu;
    float *orow = out + static_cast<size_t>(blockIdx.x) * K;
    for (uint32_t wi = threadIdx.x; wi < words; wi += blockDim.x) {
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
        for (uint32_t j = 0; j < vpw; ++j)
            orow[k0 + j] = fmaf(static_cast<float>((word >> (j * bits)) & mask), s, b) * multiplier;
    }
}

// SwiGLU between two separately launched linears: h = silu(gate) * up on bf16 rows [gate | up]
// (core/src/inference/backend/cpu/kernels/ffn.zig:213-266; CUDA: reduction_ops.cu:46-72).
__global__ void __launch_bounds__(256)
gaf_swiglu_bf16_kernel(const __nv_bfloat16 *gu, __nv_bfloat16 *h, uint32_t M, uint32_t d_ff, uint32_t act) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<size_t>(M) * d_ff) return;
    const size_t m = i / d_ff, j = i - m * d_ff;
    const float g = __bfloat162float(gu[m * 2u * d_ff + j]);
    const float u = __bfloat162float(gu[m * 2u * d_ff + d_ff + j]);
    h[i] = __float2bfloat16_rn(gate_activation(g, act) * u);
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
struct GemvPlan {
    uint32_t rgs, chunks, units, ctas, max_slots;
};

constexpr int kMaxDevices = 64;

// The opt-in to more than 48 KB of dynamic shared memory is a property of (function, device): set it the first
// time a kernel instance is launched on each device of the process.
template <typename Kern>
cudaError_t opt_in_shared_memory(Kern kern, int bytes, bool (&configured)[kMaxDevices]) {
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (configured[dev]) return cudaSuccess;
    if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); e != cudaSuccess) return e;
    configured[dev] = true;
    return cudaSuccess;
}

GemvPlan plan_gemv(const WeightView &w, const GemvTuning &tune, int sm_count) {
    GemvPlan pl;
    pl.rgs = (w.N + kRows - 1u) / kRows;
    pl.chunks = (w.row_bytes + kChunkBytes - 1u) / kChunkBytes;
    pl.units = pl.rgs * pl.chunks;
    uint32_t ctas = tune.ctas > 0 ? static_cast<uint32_t>(tune.ctas) : static_cast<uint32_t>(sm_count);
    // CTAs of one launch wait on one another (split-K collection, the two-operation launch): all must be resident
    if (ctas > static_cast<uint32_t>(sm_count)) ctas = static_cast<uint32_t>(sm_count);
    if (ctas > pl.units) ctas = pl.units;
    if (ctas < 1u) ctas = 1u;
    pl.ctas = ctas;
    // a row group of `chunks` units is cut by at most ceil(chunks / q) + 1 contiguous ranges of >= q units
    const uint32_t q = pl.units / ctas;
    pl.max_slots = (pl.chunks + q - 1u) / q + 1u;
    return pl;
}

template <int GB, int BITS, int MT, bool XF32, int SD>
cudaError_t launch_stream(const GemvParams &p, const WeightView &w, const WeightView *next, uint32_t ctas, bool pdl,
                          cudaStream_t stream) {
    auto kern = gaf_gemv_stream_kernel<GB, BITS, MT, XF32, SD>;
    using Plan = SmemPlan<GB, MT, XF32>;
    if constexpr (Plan::TOTAL > 227 * 1024) return cudaErrorNotSupported;  // see gemv_mma_max_rows
    static bool configured[kMaxDevices] = {};  // per instantiation and device: the attribute belongs to the function on one device
    if (cudaError_t e = opt_in_shared_memory(kern, Plan::TOTAL, configured); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Plan::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    const WeightView &nx = next ? *next : w;
    return cudaLaunchKernelEx(&cfg, kern, p, w.tmap, w.tmap_s, w.tmap_b, nx.tmap, nx.tmap_s, nx.tmap_b);
}

template <int GB, int MD, bool XF32, int SD, int NCW, int NST, int BU, int NOPS = 1, int BITS = 4>
cudaError_t launch_dp4a(const GemvParams &p, const WeightView &w, const WeightView *next, uint32_t ctas, bool pdl,
                        cudaStream_t stream, const GemvParams *second = nullptr, const GemvOpList *list = nullptr) {
    auto kern = gaf_gemv_dp4a_kernel<GB, MD, XF32, SD, NCW, NST, BU, NOPS, BITS>;
    using Plan = DpPlan<GB, MD, XF32, NST, BU, (NOPS == 0 && (MD == 1 || MD >= 4) && !XF32), BITS>;
    static bool configured[kMaxDevices] = {};
    if (cudaError_t e = opt_in_shared_memory(kern, Plan::TOTAL, configured); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3((NCW + 2) * 32);
    cfg.dynamicSmemBytes = Plan::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    // two operations: `next` is the second weight (its maps travel in the next-weight slots)
    const WeightView &nx = next ? *next : w;
    GemvOpList none;
    memset(&none, 0, sizeof none);
    return cudaLaunchKernelEx(&cfg, kern, p, second ? *second : p, w.tmap, w.tmap_s, w.tmap_b, nx.tmap, nx.tmap_s, nx.tmap_b,
                              list ? *list : none);
}

// a whole launch list in one launch (all operations: gaf4, one group size, one scales dtype, the same M <= 4)
template <int GB>
cudaError_t dispatch_list(const GemvParams &first, const WeightView &w0, const GemvOpList &list, uint32_t ctas, uint32_t M,
                          bool pdl, cudaStream_t stream, bool imma_small) {
    const bool bf = first.sdtype == 1u;
    constexpr int NST1 = GB == 16 ? 3 : 4;
    if constexpr (GB != 16) {
        if (w0.bits == 8u) {
            if (M == 1 && !imma_small)
                return bf ? launch_dp4a<GB, 1, false, 1, kConsumerWarps, 4, 8, 0, 8>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list)
                          : launch_dp4a<GB, 1, false, 0, kConsumerWarps, 4, 8, 0, 8>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list);
            if (M <= 4)
                return bf ? launch_dp4a<GB, 4, false, 1, kConsumerWarps, 3, 8, 0, 8>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list)
                          : launch_dp4a<GB, 4, false, 0, kConsumerWarps, 3, 8, 0, 8>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list);
            return cudaErrorNotSupported;
        }
    }
    if ((imma_small && M == 1) || M == 2) M = 4;   // the int8-MMA instance (built for four rows) with fewer rows in use
    if (M == 1)
        return bf ? launch_dp4a<GB, 1, false, 1, kConsumerWarps, NST1, 8, 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list)
                  : launch_dp4a<GB, 1, false, 0, kConsumerWarps, NST1, 8, 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list);
    if (M == 3 || M == 4)
        return bf ? launch_dp4a<GB, 4, false, 1, kConsumerWarps, 3, (GB == 16 ? 4 : 8), 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list)
                  : launch_dp4a<GB, 4, false, 0, kConsumerWarps, 3, (GB == 16 ? 4 : 8), 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list);
    if constexpr (GB != 16) {
        // five to eight rows: two sets of MMA columns; activation blocks of two units for the operations that still
        // quantise per CTA, one hand-over buffer to the writer warp
        if (M >= 5 && M <= 8)
            return bf ? launch_dp4a<GB, 8, false, 1, kConsumerWarps, 3, 2, 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list)
                      : launch_dp4a<GB, 8, false, 0, kConsumerWarps, 3, 2, 0>(first, w0, nullptr, ctas, pdl, stream, nullptr, &list);
    }
    return cudaErrorNotSupported;
}

// gate|up then down in one launch (M = 1, both weights of one group size)
template <int GB>
cudaError_t dispatch_ffn(const GemvParams &p1, const GemvParams &p2, const WeightView &w1, const WeightView &w2,
                         uint32_t ctas, uint32_t M, bool pdl, cudaStream_t stream) {
    const bool bf = p1.sdtype == 1u;
    constexpr int NST1 = GB == 16 ? 3 : 4;
    if (M == 1)
        return bf ? launch_dp4a<GB, 1, false, 1, kConsumerWarps, NST1, 8, 2>(p1, w1, &w2, ctas, pdl, stream, &p2)
                  : launch_dp4a<GB, 1, false, 0, kConsumerWarps, NST1, 8, 2>(p1, w1, &w2, ctas, pdl, stream, &p2);
    return cudaErrorNotSupported;
}

template <int GB>
cudaError_t dispatch_dp4a(const GemvParams &p, const WeightView &w, const WeightView *next, uint32_t ctas, uint32_t M,
                          bool pdl, cudaStream_t stream) {
    const bool bf = p.sdtype == 1u;
    // Ring depth: four stages for one activation row where shared memory allows (group sizes 64 / 128),
    // three otherwise.  (Five stages measured no better: the kernel is issue-bound before it is latency-bound.)
    constexpr int NST1 = GB == 16 ? 3 : 4;
    if (M == 1)
        return bf ? launch_dp4a<GB, 1, false, 1, kConsumerWarps, NST1, 8>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 1, false, 0, kConsumerWarps, NST1, 8>(p, w, next, ctas, pdl, stream);
    if (M == 2)
        return bf ? launch_dp4a<GB, 2, false, 1, kConsumerWarps, 3, 8>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 2, false, 0, kConsumerWarps, 3, 8>(p, w, next, ctas, pdl, stream);
    if (M == 3 || M == 4)  // int8-MMA variant, three stages, activation blocks of eight units (four for 32-element groups)
        return bf ? launch_dp4a<GB, 4, false, 1, kConsumerWarps, 3, (GB == 16 ? 4 : 8)>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 4, false, 0, kConsumerWarps, 3, (GB == 16 ? 4 : 8)>(p, w, next, ctas, pdl, stream);
    return cudaErrorNotSupported;
}

// 8-bit codes, one or two bf16 activation rows: the integer dot-product kernel on the bytes as they are
// (groups of 32 and 64 codes: the row split of the kernel needs at least four groups per unit)
template <int GB>
cudaError_t dispatch_dp4a8(const GemvParams &p, const WeightView &w, const WeightView *next, uint32_t ctas, uint32_t M,
                           bool pdl, cudaStream_t stream) {
    const bool bf = p.sdtype == 1u;
    if (M == 1)
        return bf ? launch_dp4a<GB, 1, false, 1, kConsumerWarps, 4, 8, 1, 8>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 1, false, 0, kConsumerWarps, 4, 8, 1, 8>(p, w, next, ctas, pdl, stream);
    if (M == 2)
        return bf ? launch_dp4a<GB, 2, false, 1, kConsumerWarps, 3, 8, 1, 8>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 2, false, 0, kConsumerWarps, 3, 8, 1, 8>(p, w, next, ctas, pdl, stream);
    if (M == 3 || M == 4)   // int8 MMA on the code bytes as they are
        return bf ? launch_dp4a<GB, 4, false, 1, kConsumerWarps, 3, 8, 1, 8>(p, w, next, ctas, pdl, stream)
                  : launch_dp4a<GB, 4, false, 0, kConsumerWarps, 3, 8, 1, 8>(p, w, next, ctas, pdl, stream);
    return cudaErrorNotSupported;
}

template <int GB, int BITS>
cudaError_t dispatch_stream(const GemvParams &p, const WeightView &tmap, const WeightView *next, uint32_t ctas, int mt,
                            bool xf32, bool pdl,
                            cudaStream_t stream) {
    const bool bf = p.sdtype == 1u;
#define TGAF_CASE(MTv, XFv)                                                                          \
    if (mt == MTv && xf32 == XFv)                                                                    \
        return bf ? launch_stream<GB, BITS, MTv, XFv, 1>(p, tmap, next, ctas, pdl, stream)                 \
                  : launch_stream<GB, BITS, MTv, XFv, 0>(p, tmap, next, ctas, pdl, stream);
    TGAF_CASE(1, false)
    TGAF_CASE(2, false)
    TGAF_CASE(1, true)
    TGAF_CASE(2, true)
#undef TGAF_CASE
    return cudaErrorNotSupported;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

// Tensor map of the packed matrix as bytes [N][row_bytes], tile 128 rows x 128 bytes, 128-byte swizzle.
cudaError_t make_packed_tmap(const WeightView &w, CUtensorMap *out) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    if (reinterpret_cast<uintptr_t>(w.packed) % 16u != 0 || w.row_bytes % 16u != 0) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {w.row_bytes, w.N};
    const cuuint64_t strides[1] = {w.row_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kPanelBytes), static_cast<cuuint32_t>(kRows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w.packed), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Tensor map of a scale / bias array as bytes [N][groups * 2], tile 128 rows x max(16, groups-per-unit * 2) bytes.
static cudaError_t make_sb_tmap(const WeightView &w, const uint16_t *base, CUtensorMap *out) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return cudaErrorNotSupported;
    const uint32_t gb = w.group * w.bits / 8u;
    if (gb == 0 || kChunkBytes % gb != 0) return cudaErrorNotSupported;
    const uint32_t gps = kChunkBytes / gb;
    const uint32_t sbox = gps * 2u > 16u ? gps * 2u : 16u;
    const uint64_t pitch = static_cast<uint64_t>(w.groups) * 2u;
    if (reinterpret_cast<uintptr_t>(base) % 16u != 0 || pitch % 16u != 0) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {pitch, w.N};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {sbox, static_cast<cuuint32_t>(kRows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint16_t *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

void attach_packed_tmap(WeightView &w) {
    w.has_tmap = make_packed_tmap(w, &w.tmap) == cudaSuccess && make_sb_tmap(w, w.scales, &w.tmap_s) == cudaSuccess &&
                 make_sb_tmap(w, w.biases, &w.tmap_b) == cudaSuccess;
}

bool gemv_mma_eligible(const WeightView &w, const void *x, const void *y, bool x_f32) {
    if (!w.has_tmap) return false;
    const uint32_t gb = w.group * w.bits / 8u;
    // group sizes 32 / 64 / 128 of either code width (what the converter produces)
    if (w.bits == 4 ? (gb != 16u && gb != 32u && gb != 64u) : (gb != 32u && gb != 64u && gb != 128u)) return false;
    if (w.row_bytes != w.K * w.bits / 8u) return false;
    // TMA needs a 16-byte aligned base and row pitch
    if (reinterpret_cast<uintptr_t>(w.packed) % 16u != 0 || w.row_bytes % 16u != 0) return false;
    if (reinterpret_cast<uintptr_t>(w.scales) % 2u != 0 || reinterpret_cast<uintptr_t>(w.biases) % 2u != 0) return false;
    // activation rows are read 16 bytes at a time
    const size_t xrow = static_cast<size_t>(w.K) * (x_f32 ? 4u : 2u);
    if (reinterpret_cast<uintptr_t>(x) % 16u != 0 || xrow % 16u != 0) return false;
    if (reinterpret_cast<uintptr_t>(y) % (x_f32 ? 4u : 2u) != 0) return false;
    return true;
}

// The all-reduce can ride in the write-out of the M <= 4 kernel when the peers' regions are mapped and the
// fp32 tile [M][N] fits an exchange slot.
bool gemv_fused_eligible(const WeightView &w, uint32_t M, bool x_f32, const GemvTuning &tune) {
    if (!tune.fuse || !tune.fuse->ok || tune.fuse->size == 0u || tune.fuse->size > static_cast<uint32_t>(kPeerMaxRanks)) return false;
    if (w.bits != 4u || M == 0u || M > 4u || x_f32 || tune.no_dp4a) return false;
    if (static_cast<size_t>(M) * w.N * 8u > kPeerSlotBytes) return false;  // {value, epoch} words
    return true;
}

size_t gemv_mma_scratch_bytes(const WeightView &w, uint32_t M, const GemvTuning &tune, int sm_count) {
    const GemvPlan pl = plan_gemv(w, tune, sm_count);
    const uint32_t mrows = M <= 8u ? 8u : 16u;
    return static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * mrows * sizeof(float);
}

size_t gemv_tagged_bytes(const WeightView &w, uint32_t M, bool x_f32, const GemvTuning &tune, int sm_count) {
    if (M == 0u || M > 16u) return 0;
    const GemvPlan pl = plan_gemv(w, tune, sm_count);
    const uint32_t gb = w.group * w.bits / 8u;
    const bool integer_path = ((w.bits == 4u && M <= 4u) || (w.bits == 8u && M <= 4u && (gb == 32u || gb == 64u))) && !x_f32 &&
                              !tune.no_dp4a && gb != 0u;
    const uint32_t cols = integer_path ? (M <= 2u ? M : 4u) : (M <= 8u ? 8u : 16u);
    return static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * cols * 8u;
}

// Activation rows one launch of the fast path takes: 16, except where two tiles do not fit in shared memory
// (4-bit codes in groups of 32 with fp32 activations: hi + lo fragments double the block).
uint32_t gemv_mma_max_rows(const WeightView &w, bool x_f32) {
    return (w.bits == 4u && w.group == 32u && x_f32) ? 8u : 16u;
}

size_t gemv_mma_counter_count(const WeightView &w) {
    return static_cast<size_t>((w.N + kRows - 1u) / kRows);
}

// the fields every GEMV launch fills the same way
static GemvParams base_params(const WeightView &w, const void *x, void *y, uint32_t M, const GemvPlan &pl,
                              unsigned int *d_error_word) {
    GemvParams p;
    memset(&p, 0, sizeof p);
    p.packed = w.packed;
    p.scales = w.scales;
    p.biases = w.biases;
    p.x = x;
    p.y = y;
    p.error_word = d_error_word;
    p.N = w.N;
    p.K = w.K;
    p.M = M;
    p.groups = w.groups;
    p.row_bytes = w.row_bytes;
    p.group = w.group;
    p.sdtype = w.sdtype;
    p.chunks = pl.chunks;
    p.units = pl.units;
    p.max_slots = pl.max_slots;
    return p;
}

cudaError_t gemv_mma(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                     const Scratch &scratch, const GemvTuning &tune, cudaStream_t stream, int sm_count,
                     unsigned int *d_error_word) {
    if (M == 0 || M > gemv_mma_max_rows(w, x_f32)) return cudaErrorNotSupported;
    if (!gemv_mma_eligible(w, x, y, x_f32)) return cudaErrorNotSupported;
    const GemvPlan pl = plan_gemv(w, tune, sm_count);
    const int mt = M <= 8u ? 1 : 2;
    const size_t need = static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * (mt * 8) * sizeof(float);
    if (need > scratch.partial_bytes || gemv_mma_counter_count(w) > scratch.counter_count)
        return cudaErrorMemoryAllocation;
    const uint32_t gb = w.group * w.bits / 8u;
    GemvParams p = base_params(w, x, y, M, pl, d_error_word);
    p.partials = scratch.partials;
    p.counters = scratch.counters;
    // optional hint: the weight the following launch will stream (same unit geometry on either GEMV kernel)
    const WeightView *next = nullptr;
    p.next_units = p.next_chunks = p.next_ctas = p.next_gps = p.next_prefetch = 0u;
    if (tune.next && tune.prefetch_units > 0 && tune.next->has_tmap) {
        const uint32_t ngb = tune.next->group * tune.next->bits / 8u;
        if (ngb != 0u && kChunkBytes % ngb == 0u) {
            const GemvPlan np = plan_gemv(*tune.next, tune, sm_count);
            next = tune.next;
            p.next_units = np.units;
            p.next_chunks = np.chunks;
            p.next_ctas = np.ctas;
            p.next_gps = kChunkBytes / ngb;
            p.next_prefetch = static_cast<uint32_t>(tune.prefetch_units);
        }
    }
    const bool pdl = tune.pdl != 0;
    for (int r = 0; r < kPeerMaxRanks; ++r) p.fuse_region[r] = nullptr;
    p.fuse_rank = 0u;
    p.fuse_size = 0u;
    if (tune.fuse) {
        if (!gemv_fused_eligible(w, M, x_f32, tune)) return cudaErrorNotSupported;
        for (int r = 0; r < kPeerMaxRanks; ++r) p.fuse_region[r] = static_cast<uint8_t *>(tune.fuse->region[r]);
        p.fuse_rank = tune.fuse->rank;
        p.fuse_size = tune.fuse->size;
    }
    if (w.bits == 4 && M <= 4u && !x_f32 && !tune.no_dp4a) {
        const uint32_t md = M <= 2u ? M : 4u;  // activation rows the kernel instance is built for
        if (scratch.tagged && static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * md * 8u <= scratch.tagged_bytes)
            p.tagged = scratch.tagged;
        // one or two bf16 activation rows: the integer dot-product formulation (its 13-bit activations
        // are ample next to bf16 inputs; f32 callers keep the hi + lo tensor-core path and its 1e-3 accuracy)
        if (gb == 16u) return dispatch_dp4a<16>(p, w, next, pl.ctas, M, pdl, stream);
        if (gb == 32u) return dispatch_dp4a<32>(p, w, next, pl.ctas, M, pdl, stream);
        if (gb == 64u) return dispatch_dp4a<64>(p, w, next, pl.ctas, M, pdl, stream);
    }
    if (w.bits == 8 && M <= 4u && !x_f32 && !tune.no_dp4a && (gb == 32u || gb == 64u)) {
        const uint32_t md8 = M <= 2u ? M : 4u;
        if (scratch.tagged && static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * md8 * 8u <= scratch.tagged_bytes)
            p.tagged = scratch.tagged;
        if (gb == 32u) return dispatch_dp4a8<32>(p, w, next, pl.ctas, M, pdl, stream);
        return dispatch_dp4a8<64>(p, w, next, pl.ctas, M, pdl, stream);
    }
    // tensor-core formulation: tagged partial sums [row group][slot][128][8 or 16] when the scratch has room
    if (scratch.tagged && static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * (mt * 8) * 8u <= scratch.tagged_bytes)
        p.tagged = scratch.tagged;
    if (w.bits == 4) {
        if (gb == 16u) return dispatch_stream<16, 4>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
        if (gb == 32u) return dispatch_stream<32, 4>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
        if (gb == 64u) return dispatch_stream<64, 4>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
    } else {
        if (gb == 32u) return dispatch_stream<32, 8>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
        if (gb == 64u) return dispatch_stream<64, 8>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
        if (gb == 128u) return dispatch_stream<128, 8>(p, w, next, pl.ctas, mt, x_f32, pdl, stream);
    }
    return cudaErrorNotSupported;
}

// ---------------------------------------------------------------------------
// SwiGLU FFN for M = 1 in one launch: y = (silu(x Wg^T) * (x Wu^T)) Wd^T with Wg, Wu stacked as one weight
// [2 d_ff, d_model] (gate rows first) and Wd [d_model, d_ff].  `mid` is fp32 [M][2 d_ff] device scratch.
// ---------------------------------------------------------------------------
bool gemv_ffn_eligible(const WeightView &w1, const WeightView &w2, const void *x, const void *y, uint32_t M,
                       const GemvTuning &tune) {
    // one activation row only: with two, the two-launch path measured faster (0.41 vs 0.47 ms on the 8B stack)
    if (M != 1u || tune.no_dp4a) return false;
    if (w1.bits != 4u || w2.bits != 4u || w1.group != w2.group || w1.sdtype != w2.sdtype) return false;
    if (w1.N != 2u * w2.K) return false;
    if (!gemv_mma_eligible(w1, x, y, false)) return false;
    // the second operand is the fp32 scratch, always aligned; its weight must be on the fast path too
    if (!w2.has_tmap || w2.row_bytes != w2.K * w2.bits / 8u) return false;
    return true;
}

size_t gemv_ffn_tagged_bytes(const WeightView &w1, const WeightView &w2, uint32_t M, const GemvTuning &tune, int sm_count) {
    GemvTuning t = tune;
    const GemvPlan a = plan_gemv(w1, t, sm_count), b = plan_gemv(w2, t, sm_count);
    t.ctas = static_cast<int>(a.ctas < b.ctas ? a.ctas : b.ctas);
    const GemvPlan pa = plan_gemv(w1, t, sm_count), pb = plan_gemv(w2, t, sm_count);
    return (static_cast<size_t>(pa.rgs) * pa.max_slots + static_cast<size_t>(pb.rgs) * pb.max_slots) * kRows * M * 8u;
}

cudaError_t gemv_ffn_swiglu(const WeightView &w1, const WeightView &w2, const void *x, float *mid, void *y, uint32_t M,
                            uint32_t act, const Scratch &scratch, unsigned int *grid_bar, const GemvTuning &tune,
                            cudaStream_t stream, int sm_count, unsigned int *d_error_word) {
    if (!gemv_ffn_eligible(w1, w2, x, y, M, tune)) return cudaErrorNotSupported;
    GemvTuning t = tune;
    const GemvPlan a = plan_gemv(w1, t, sm_count), b = plan_gemv(w2, t, sm_count);
    t.ctas = static_cast<int>(a.ctas < b.ctas ? a.ctas : b.ctas);  // one grid: every CTA has units of both weights
    const GemvPlan pl1 = plan_gemv(w1, t, sm_count), pl2 = plan_gemv(w2, t, sm_count);
    const size_t need1 = static_cast<size_t>(pl1.rgs) * pl1.max_slots * kRows * M;  // 64-bit words
    const size_t need2 = static_cast<size_t>(pl2.rgs) * pl2.max_slots * kRows * M;
    if (!scratch.tagged || (need1 + need2) * 8u > scratch.tagged_bytes || !grid_bar) return cudaErrorMemoryAllocation;
    GemvParams p1 = base_params(w1, x, mid, M, pl1, d_error_word);
    p1.tagged = scratch.tagged;
    p1.y_f32 = 1u;
    p1.grid_bar = grid_bar;
    GemvParams p2 = base_params(w2, mid, y, M, pl2, d_error_word);
    p2.tagged = scratch.tagged + need1;
    p2.act = act;
    p2.dep = 1u;
    p2.grid_bar = grid_bar;
    if (tune.fuse && gemv_fused_eligible(w2, M, false, tune)) {  // tensor parallel: the sum over ranks rides in the down projection
        for (int r = 0; r < kPeerMaxRanks; ++r) p2.fuse_region[r] = static_cast<uint8_t *>(tune.fuse->region[r]);
        p2.fuse_rank = tune.fuse->rank;
        p2.fuse_size = tune.fuse->size;
    } else if (tune.fuse) {
        return cudaErrorNotSupported;
    }
    const uint32_t gb = w1.group * w1.bits / 8u;
    const bool pdl = tune.pdl != 0;
    if (gb == 16u) return dispatch_ffn<16>(p1, p2, w1, w2, pl1.ctas, M, pdl, stream);
    if (gb == 32u) return dispatch_ffn<32>(p1, p2, w1, w2, pl1.ctas, M, pdl, stream);
    if (gb == 64u) return dispatch_ffn<64>(p1, p2, w1, w2, pl1.ctas, M, pdl, stream);
    return cudaErrorNotSupported;
}

// ---------------------------------------------------------------------------
// Launch list: several linears (M <= 4, gaf4, one group size and scales dtype) in ONE launch of the M <= 4 kernel.
// The caller fills `params` / `maps` (host arrays of `count` / 3 * count entries) through gemv_list_plan, copies them
// to the device once, and launches with gemv_list_launch as often as it likes.
// ---------------------------------------------------------------------------
// activation rows the list's kernel instance is built for: 1 (integer dot products), 4 or 8 (int8 MMA; two rows run
// on the four-row instance, which measured faster in a list than the two-row dot-product one)
static uint32_t list_instance_rows(uint32_t M, const GemvTuning &tune) {
    if (M == 1u && !tune.imma_small) return 1u;
    return M <= 4u ? 4u : 8u;
}

bool gemv_list_eligible(const WeightView *const *ws, uint32_t count, uint32_t M, const GemvTuning &tune) {
    if (count == 0u || count > 256u || M == 0u || M > 8u || tune.no_dp4a || tune.force_generic) return false;
    const WeightView &w0 = *ws[0];
    const uint32_t gb0 = w0.group * w0.bits / 8u;
    if (w0.bits == 8u) {
        // 8-bit codes: up to four activation rows, groups of 32 and 64 codes
        if (M > 4u || (gb0 != 32u && gb0 != 64u)) return false;
    } else {
        if (gb0 != 16u && gb0 != 32u && gb0 != 64u) return false;
        if (M > 4u && gb0 == 16u) return false;   // five to eight rows: groups of 64 and 128 codes only (shared memory)
    }
    for (uint32_t i = 0; i < count; ++i) {
        const WeightView &w = *ws[i];
        if ((w.bits != 4u && w.bits != 8u) || w.bits != w0.bits || w.group != w0.group || w.sdtype != w0.sdtype || !w.has_tmap) return false;
        if (w.row_bytes != w.K * w.bits / 8u) return false;
    }
    return true;
}

// One grid for the whole list.  Up to four rows: as many CTAs as the largest operation can use; in an operation with
// fewer units than that some CTAs have none (they pass straight on to the next one).  Five to eight rows: the
// smallest unit count, so that every operation keeps the units per CTA the once-per-launch activations want.
uint32_t gemv_list_ctas(const WeightView *const *ws, uint32_t count, uint32_t M, const GemvTuning &tune, int sm_count) {
    uint32_t lo = 0xFFFFFFFFu, hi = 1u;
    for (uint32_t i = 0; i < count; ++i) {
        const GemvPlan pl = plan_gemv(*ws[i], tune, sm_count);
        if (pl.ctas < lo) lo = pl.ctas;
        if (pl.ctas > hi) hi = pl.ctas;
    }
    return M <= 4u ? hi : lo;
}

// tagged split-K words the whole list needs (64-bit words), operation by operation
size_t gemv_list_tagged_words(const WeightView *const *ws, uint32_t count, uint32_t M, const GemvTuning &tune, int sm_count) {
    GemvTuning t = tune;
    t.ctas = static_cast<int>(gemv_list_ctas(ws, count, M, tune, sm_count));
    const uint32_t md = list_instance_rows(M, tune);
    size_t words = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const GemvPlan pl = plan_gemv(*ws[i], t, sm_count);
        words += static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * md;
    }
    return words;
}

// A planned launch list: host copy of the first operation's parameters (the kernel takes them by value), the
// device tables (tensor maps, parameters, arrival counters) in one allocation.
struct GemvList {
    GemvParams first;
    WeightView w0;
    void *d_blob;
    const GemvParams *d_params;
    const CUtensorMap *d_maps;
    const XqPair *d_tab;
    unsigned int *d_bar;
    size_t bar_bytes;
    uint32_t count, ctas, M;
    uint32_t xq_pairs;  // (operation, K chunk) pairs quantised at the start of every launch
    bool imma_small;   // M <= 2 on the int8-MMA instance (the tagged words are then laid out for four rows)
};

cudaError_t gemv_list_create(const WeightView *const *ws, const void *const *xs, void *const *ys, const uint8_t *deps,
                             const PeerComm *const *fuse, uint32_t count, uint32_t M, unsigned long long *tagged,
                             const GemvTuning &tune, int sm_count, unsigned int *d_error_word, cudaStream_t stream,
                             GemvList **out) {
    *out = nullptr;
    if (!gemv_list_eligible(ws, count, M, tune)) return cudaErrorNotSupported;
    // five to eight rows: an operation that quantises per CTA (it reads what the launch writes, or it is too small for the
    // once-per-launch form) would do so in blocks of two units - all the shared memory left beside the eight-row stages -
    // which measured slower than separate launches: such lists run call by call
    if (M > 4u && deps)
        for (uint32_t i = 0; i < count; ++i)
            if (deps[i]) return cudaErrorNotSupported;
    GemvTuning t = tune;
    t.ctas = static_cast<int>(gemv_list_ctas(ws, count, M, tune, sm_count));
    const uint32_t md = list_instance_rows(M, tune);
    const size_t map_bytes = static_cast<size_t>(count) * 3u * sizeof(CUtensorMap);
    const size_t par_bytes = (static_cast<size_t>(count) * sizeof(GemvParams) + 255u) & ~size_t(255);
    const size_t bar_bytes = (static_cast<size_t>(count + 1u) * sizeof(unsigned int) + 255u) & ~size_t(255);   // + the activations counter
    // One activation row on the integer-dot instance: operations whose activations nothing in this launch writes get them
    // quantised once per launch into global memory, [K chunk][1 KB of limb bytes + {scale, sum} per group]
    const uint32_t gb0 = ws[0]->group * ws[0]->bits / 8u;
    // per activation row the instance is built for: the limb bytes of a unit's 512 (4-bit) or 256 (8-bit) activations
    // and a {scale, sum} pair per group
    const size_t xqs_unit = ((ws[0]->bits == 4u ? 1024u : 512u) + (gb0 ? (kChunkBytes / gb0) * 8u : 0u)) * md;
    const bool use_xq = gb0 != 0u;
    size_t xq_bytes = 0;
    // (operations that give every CTA at least two units - with the unit ranges rotating and the launch-start
    // quantisation dealt over the whole grid that measured faster than, or as fast as, letting each CTA quantise the
    // block or two it needs, down to the shards of eight tensor-parallel ranks; above four rows, whose instance has room
    // for per-CTA blocks of two units only, at least four units)
    auto wants_xq = [&](uint32_t i, const GemvPlan &pl) {
        if (!use_xq || (deps && deps[i])) return false;
        const uint32_t per_cta = pl.units / static_cast<uint32_t>(t.ctas);
        return per_cta >= (M <= 4u ? 2u : 4u);
    };
    for (uint32_t i = 0; i < count; ++i) {
        const GemvPlan pl = plan_gemv(*ws[i], t, sm_count);
        if (wants_xq(i, pl)) xq_bytes += static_cast<size_t>(pl.chunks) * xqs_unit;
        else if (M > 4u) return cudaErrorNotSupported;   // five to eight rows: only operations that take the once-per-launch form
    }
    xq_bytes = (xq_bytes + 255u) & ~size_t(255);
    uint32_t total_pairs = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const GemvPlan pl = plan_gemv(*ws[i], t, sm_count);
        if (wants_xq(i, pl)) total_pairs += pl.chunks;
    }
    const size_t tab_bytes = (static_cast<size_t>(total_pairs) * sizeof(XqPair) + 255u) & ~size_t(255);
    uint8_t *host = static_cast<uint8_t *>(malloc(map_bytes + par_bytes + tab_bytes));
    if (!host) return cudaErrorMemoryAllocation;
    XqPair *tab = reinterpret_cast<XqPair *>(host + map_bytes + par_bytes);
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(host);
    GemvParams *params = reinterpret_cast<GemvParams *>(host + map_bytes);
    size_t words = 0, xq_off = 0;
    uint32_t xq_pairs = 0, rot = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const WeightView &w = *ws[i];
        if (!gemv_mma_eligible(w, xs[i], ys[i], false)) {
            free(host);
            return cudaErrorNotSupported;
        }
        const GemvPlan pl = plan_gemv(w, t, sm_count);
        GemvParams q = base_params(w, xs[i], ys[i], M, pl, d_error_word);
        q.tagged = tagged + words;
        words += static_cast<size_t>(pl.rgs) * pl.max_slots * kRows * md;
        q.dep = deps && deps[i] ? 1u : 0u;
        // the ranges with one unit more start where the previous operation's stopped
        q.rot = rot;
        rot = (rot + static_cast<uint32_t>(t.ctas) - pl.units % static_cast<uint32_t>(t.ctas)) % static_cast<uint32_t>(t.ctas);
        if (wants_xq(i, pl)) {
            // the address is an offset for now: the blob it lives in is allocated below
            q.xq = reinterpret_cast<uint8_t *>(xq_off + 1u);
            q.xq_pair0 = xq_pairs;
            xq_off += static_cast<size_t>(pl.chunks) * xqs_unit;
            xq_pairs += pl.chunks;
        }
        if (fuse && fuse[i]) {
            GemvTuning tf = t;
            tf.fuse = fuse[i];
            if (!gemv_fused_eligible(w, M, false, tf)) {
                free(host);
                return cudaErrorNotSupported;
            }
            for (int r = 0; r < kPeerMaxRanks; ++r) q.fuse_region[r] = static_cast<uint8_t *>(fuse[i]->region[r]);
            q.fuse_rank = fuse[i]->rank;
            q.fuse_size = fuse[i]->size;
        }
        params[i] = q;
        memcpy(&maps[3u * i], &w.tmap, sizeof(CUtensorMap));
        memcpy(&maps[3u * i + 1u], &w.tmap_s, sizeof(CUtensorMap));
        memcpy(&maps[3u * i + 2u], &w.tmap_b, sizeof(CUtensorMap));
    }
    GemvList *l = new (std::nothrow) GemvList();
    if (!l) {
        free(host);
        return cudaErrorMemoryAllocation;
    }
    // device blob: tensor maps, parameters, pair table, counters, quantised activations
    cudaError_t e = cudaMalloc(&l->d_blob, map_bytes + par_bytes + tab_bytes + bar_bytes + xq_bytes);
    if (e == cudaSuccess) {
        uint8_t *xq_base = static_cast<uint8_t *>(l->d_blob) + map_bytes + par_bytes + tab_bytes + bar_bytes;
        uint32_t np = 0;
        for (uint32_t i = 0; i < count; ++i) {
            if (!params[i].xq) continue;
            params[i].xq = xq_base + (reinterpret_cast<uintptr_t>(params[i].xq) - 1u);
            for (uint32_t kc = 0; kc < params[i].chunks; ++kc, ++np) {
                tab[np].x = params[i].x;
                tab[np].dst = params[i].xq + static_cast<size_t>(kc) * xqs_unit;
                tab[np].kc = kc, tab[np].groups = params[i].groups, tab[np].K = params[i].K, tab[np].M = params[i].M;
            }
        }
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(l->d_blob, host, map_bytes + par_bytes + tab_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(static_cast<uint8_t *>(l->d_blob) + map_bytes + par_bytes + tab_bytes, 0, bar_bytes, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);   // the host copy goes away below
    l->first = params[0];
    l->w0 = *ws[0];
    free(host);
    if (e != cudaSuccess) {
        if (l->d_blob) cudaFree(l->d_blob);
        delete l;
        return e;
    }
    l->d_maps = static_cast<const CUtensorMap *>(l->d_blob);
    l->d_params = reinterpret_cast<const GemvParams *>(static_cast<uint8_t *>(l->d_blob) + map_bytes);
    l->d_tab = reinterpret_cast<const XqPair *>(static_cast<uint8_t *>(l->d_blob) + map_bytes + par_bytes);
    l->d_bar = reinterpret_cast<unsigned int *>(static_cast<uint8_t *>(l->d_blob) + map_bytes + par_bytes + tab_bytes);
    l->bar_bytes = bar_bytes;
    l->count = count;
    l->ctas = static_cast<uint32_t>(t.ctas);
    l->M = M;
    l->xq_pairs = xq_pairs;
    l->imma_small = tune.imma_small != 0 || M == 2u;
    *out = l;
    return cudaSuccess;
}

cudaError_t gemv_list_launch(const GemvList *l, const GemvTuning &tune, cudaStream_t stream) {
    GemvOpList list;
    list.ops = l->d_params;
    list.maps = l->d_maps;
    list.count = l->count;
    list.grid_bar = l->d_bar;
    list.xq_pairs = l->xq_pairs;
    list.xq_tab = l->d_tab;
    const uint32_t gb = l->w0.group * l->w0.bits / 8u;
    const bool pdl = tune.pdl != 0;
    const bool im = l->imma_small;
    if (gb == 16u) return dispatch_list<16>(l->first, l->w0, list, l->ctas, l->M, pdl, stream, im);
    if (gb == 32u) return dispatch_list<32>(l->first, l->w0, list, l->ctas, l->M, pdl, stream, im);
    if (gb == 64u) return dispatch_list<64>(l->first, l->w0, list, l->ctas, l->M, pdl, stream, im);
    return cudaErrorNotSupported;
}

// after a launch was abandoned (a bounded wait ran out): the arrival counters may be anywhere
cudaError_t gemv_list_reset(GemvList *l) { return cudaMemset(l->d_bar, 0, l->bar_bytes); }

void gemv_list_destroy(GemvList *l) {
    if (!l) return;
    if (l->d_blob) cudaFree(l->d_blob);
    delete l;
}

// ---------------------------------------------------------------------------
// Streaming GEMV on a fixed scratch that lives in the library image.
//
// Some hosts must not allocate once they are serving: they hand the rest of the
// device's memory to their own KV-cache / arena at start-up, and cudaMalloc or
// cudaFree later would synchronise the whole device in the middle of a token
// step, or simply fail.  For them the split-K scratch (partial sums + arrival
// counters) of this variant is a file-scope device array of a fixed size; every
// GPU that loads the library carries it until the process exits.
//
// In host code the array's name is only a stand-in for the symbol, not a device
// address; the address is looked up once per device, with that device current,
// by cudaGetSymbolAddress (first call on a device: make it before any stream
// capture).  All calls on a device share the array and it keeps whatever the
// last call left: the counters are cleared on the stream before each launch, the
// partial sums are always written before they are read.  Two calls that overlap
// on the GPU (different streams) would race on it.
// ---------------------------------------------------------------------------
constexpr size_t kStaticPartialBytes = size_t(8) << 20;  // fp32 partial sums
constexpr size_t kStaticCounters = 8192;                 // one per 128-row group
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticCounters * sizeof(unsigned int);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void *g_static_ptr[kMaxDevices];  // device address of g_static_scratch, per device (0 = not looked up yet)

size_t gemv_static_scratch_capacity() { return kStaticPartialBytes; }

cudaError_t gemv_mma_static(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                            const GemvTuning &tune, cudaStream_t stream, int sm_count, int device,
                            unsigned int *d_error_word, size_t *needed_bytes) {
    if (needed_bytes) *needed_bytes = 0;
    if (M == 0 || M > 16u) return cudaErrorNotSupported;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!gemv_mma_eligible(w, x, y, x_f32)) return cudaErrorNotSupported;
    const size_t need = gemv_mma_scratch_bytes(w, M, tune, sm_count);
    if (needed_bytes) *needed_bytes = need;
    if (need > kStaticPartialBytes || gemv_mma_counter_count(w) > kStaticCounters) return cudaErrorMemoryAllocation;
    if (!g_static_ptr[device]) {
        // set-up, once per device: `device` must be the current device here
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_ptr[device] = ptr;
    }
    unsigned char *base = static_cast<unsigned char *>(g_static_ptr[device]);
    Scratch sc;
    sc.partials = reinterpret_cast<float *>(base);
    sc.partial_bytes = kStaticPartialBytes;
    sc.counters = reinterpret_cast<unsigned int *>(base + kStaticPartialBytes);
    sc.counter_count = kStaticCounters;
    sc.tagged = nullptr;
    sc.tagged_bytes = 0;
    // the counters must start at zero; the previous call (or an abandoned one) may have left anything
    cudaError_t e = cudaMemsetAsync(sc.counters, 0, gemv_mma_counter_count(w) * sizeof(unsigned int), stream);
    if (e != cudaSuccess) return e;
    GemvTuning t = tune;
    t.pdl = 0;  // the memset before the launch is a full dependency anyway
    t.next = nullptr;
    t.fuse = nullptr;
    return gemv_mma(w, x, y, M, x_f32, sc, t, stream, sm_count, d_error_word);
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

cudaError_t gather_dequant_f32(const WeightView &w, const uint32_t *d_ids, uint32_t count, float multiplier,
                               float *out, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    gaf_gather_dequant_f32_kernel<<<count, 256, 0, stream>>>(w.packed, w.scales, w.biases, d_ids, multiplier, out, w.N,
                                                            w.K, w.group, w.bits, w.sdtype, w.row_bytes, w.groups);
    return cudaGetLastError();
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

// y[m, n] += bias[n] (core/src/inference/backend/cpu/executor/model.zig:134-136, addBiasRows); bf16 y is
// widened, added in fp32 and rounded once
template <bool F32>
__global__ void __launch_bounds__(256)
gaf_add_bias_rows_kernel(void *y, const float *bias, uint32_t M, uint32_t N) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<size_t>(M) * N) return;
    const float b = bias[i % N];
    if constexpr (F32)
        static_cast<float *>(y)[i] += b;
    else
        static_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16_rn(__bfloat162float(static_cast<__nv_bfloat16 *>(y)[i]) + b);
}

cudaError_t add_bias_rows(void *y, const float *bias, uint32_t M, uint32_t N, bool f32, cudaStream_t stream) {
    const size_t n = static_cast<size_t>(M) * N;
    if (n == 0) return cudaSuccess;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    if (f32)
        gaf_add_bias_rows_kernel<true><<<blocks, 256, 0, stream>>>(y, bias, M, N);
    else
        gaf_add_bias_rows_kernel<false><<<blocks, 256, 0, stream>>>(y, bias, M, N);
    return cudaGetLastError();
}

cudaError_t swiglu_bf16(const void *gate_up, void *h, uint32_t M, uint32_t d_ff, uint32_t act, cudaStream_t stream) {
    const size_t n = static_cast<size_t>(M) * d_ff;
    if (n == 0) return cudaSuccess;
    gaf_swiglu_bf16_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(gate_up), static_cast<__nv_bfloat16 *>(h), M, d_ff, act);
    return cudaGetLastError();
}

}  // namespace tgaf
