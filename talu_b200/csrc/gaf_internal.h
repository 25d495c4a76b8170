// Internal interface between the C ABI (gaf_api.cu) and the kernel files.
// Not installed; the public surface is include/talu_gaf.h.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tgaf {

// A weight as the kernels see it: this rank's slice, canonical layout,
// row pitches in bytes (they differ from the dense pitch only for wrapped
// buffers; uploaded weights are repacked densely per rank).
struct WeightView {
    const uint8_t *packed;   // [N][row_bytes]
    const uint16_t *scales;  // [N][groups]
    const uint16_t *biases;  // [N][groups]
    uint32_t N;              // local output features
    uint32_t K;              // local input features
    uint32_t group;          // elements per group
    uint32_t bits;           // 4 or 8
    uint32_t sdtype;         // 0 = f16, 1 = bf16
    uint32_t row_bytes;      // K * bits / 8
    uint32_t groups;         // K / group
    CUtensorMap tmap;        // packed matrix as bytes [N][row_bytes] for the streaming GEMV
    CUtensorMap tmap_s;      // scales as bytes [N][groups * 2]
    CUtensorMap tmap_b;      // biases as bytes [N][groups * 2]
    bool has_tmap;           // false: a base or a row pitch is not 16-byte aligned (generic kernel only)
};

// Split-K scratch owned by a context.
struct Scratch {
    float *partials;          // [row group][slot][128][8 or 16]
    size_t partial_bytes;
    unsigned int *counters;   // [row group][8], self-resetting
    size_t counter_count;
    // M <= 4 kernel: partial sums that carry their own arrival tag, u64 {value, tag} [row group][slot][128][M];
    // all tags are zero between launches (null: the kernel uses partials + counters instead)
    unsigned long long *tagged;
    size_t tagged_bytes;
};

struct GemvTuning {
    int ctas;           // persistent CTAs of the streaming GEMV (0 = one per SM)
    int pdl;            // launch with programmatic stream serialization
    int force_generic;  // use the shape-agnostic kernel even when the fast path applies
    int imma_small;     // launch lists: M <= 2 on the int8 tensor-core instance instead of the integer dot-product one (A/B aid)
    int no_dp4a;        // keep M <= 2 on the tensor-core formulation (for A/B comparisons)
    int wait_limit;     // polls (with back-off) a device-side wait on another CTA or rank makes before it gives up (0 = default)
    int prefetch_units; // units at the head of each CTA range of the hinted next weight to pull into L2
    const WeightView *next;  // the weight the following launch will stream (one-shot hint; may be null)
    const struct PeerComm *fuse;  // sum the outputs over the ranks inside the GEMV (per call; may be null)
};

// y[M,N] = x[M,K] * W^T for M <= 16 on the tensor-core GEMV path.
// x / y are bf16 when x_f32 == 0, f32 otherwise.  Returns cudaSuccess or the
// launch error; returns cudaErrorNotSupported when the shape is not eligible
// for the fast path (the caller then uses gemv_generic).
cudaError_t gemv_mma(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                     const Scratch &scratch, const GemvTuning &tune, cudaStream_t stream,
                     int sm_count, unsigned int *d_error_word);
bool gemv_mma_eligible(const WeightView &w, const void *x, const void *y, bool x_f32);
// fills w.tmap / w.has_tmap from the other fields
void attach_packed_tmap(WeightView &w);
cudaError_t make_packed_tmap(const WeightView &w, CUtensorMap *out);
// scratch the fast path needs for this problem
// SwiGLU FFN (stacked gate|up weight, then down) for M = 1 in one launch; `mid` is fp32 [M][2 d_ff] scratch and
// `grid_bar` two zeroed counters.  cudaErrorNotSupported when the pair is not eligible.
bool gemv_ffn_eligible(const WeightView &w1, const WeightView &w2, const void *x, const void *y, uint32_t M,
                       const GemvTuning &tune);
size_t gemv_ffn_tagged_bytes(const WeightView &w1, const WeightView &w2, uint32_t M, const GemvTuning &tune, int sm_count);
cudaError_t gemv_ffn_swiglu(const WeightView &w1, const WeightView &w2, const void *x, float *mid, void *y, uint32_t M,
                            uint32_t act, const Scratch &scratch, unsigned int *grid_bar, const GemvTuning &tune,
                            cudaStream_t stream, int sm_count, unsigned int *d_error_word);
// h[m][j] = act(gu[m][j]) * gu[m][d_ff + j], bf16 in / out (the step between the two linears when they run apart);
// act: 1 = silu, 2 = tanh-form gelu
cudaError_t swiglu_bf16(const void *gate_up, void *h, uint32_t M, uint32_t d_ff, uint32_t act, cudaStream_t stream);
// y[m][n] += bias[n] in place (y f32 or bf16, bias f32 on the device)
cudaError_t add_bias_rows(void *y, const float *bias, uint32_t M, uint32_t N, bool f32, cudaStream_t stream);
bool gemv_fused_eligible(const WeightView &w, uint32_t M, bool x_f32, const GemvTuning &tune);
size_t gemv_mma_scratch_bytes(const WeightView &w, uint32_t M, const GemvTuning &tune, int sm_count);
size_t gemv_mma_counter_count(const WeightView &w);
uint32_t gemv_mma_max_rows(const WeightView &w, bool x_f32);
// bytes of Scratch::tagged the M <= 4 kernel needs for this weight (0 when that kernel does not apply)
size_t gemv_tagged_bytes(const WeightView &w, uint32_t M, bool x_f32, const GemvTuning &tune, int sm_count);

// Launch list: `count` linears (gaf4 weights of one group size and scales dtype, the same M <= 4 bf16 rows) in ONE
// launch of the M <= 4 kernel; the copy warps stream across all the weights without a pause.  deps[i] = 1: x of
// operation i is written by an earlier operation of the list (it then waits for operation i - 1 to be complete on the
// whole grid); fuse[i] != null: y of operation i is summed over the ranks inside the launch.  `tagged`: zeroed 64-bit
// words, gemv_list_tagged_words of them, owned by the caller for the life of the list.
struct GemvList;
bool gemv_list_eligible(const WeightView *const *ws, uint32_t count, uint32_t M, const GemvTuning &tune);
size_t gemv_list_tagged_words(const WeightView *const *ws, uint32_t count, uint32_t M, const GemvTuning &tune, int sm_count);
cudaError_t gemv_list_create(const WeightView *const *ws, const void *const *xs, void *const *ys, const uint8_t *deps,
                             const struct PeerComm *const *fuse, uint32_t count, uint32_t M, unsigned long long *tagged,
                             const GemvTuning &tune, int sm_count, unsigned int *d_error_word, cudaStream_t stream,
                             GemvList **out);
cudaError_t gemv_list_launch(const GemvList *l, const GemvTuning &tune, cudaStream_t stream);
cudaError_t gemv_list_reset(GemvList *l);
void gemv_list_destroy(GemvList *l);

// Same kernel on the library's fixed device-resident scratch: allocates nothing.
// cudaErrorMemoryAllocation: the problem needs more scratch than the fixed array holds
// (*needed_bytes tells how much); cudaErrorNotSupported: shape not eligible for the fast path.
cudaError_t gemv_mma_static(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                            const GemvTuning &tune, cudaStream_t stream, int sm_count, int device,
                            unsigned int *d_error_word, size_t *needed_bytes);
size_t gemv_static_scratch_capacity();

// Any shape the reference accepts, any M.  f32 arithmetic, per-element dequant.
cudaError_t gemv_generic(const WeightView &w, const void *x, void *y, uint32_t M, bool x_f32,
                         cudaStream_t stream);

// out f32 [N,K] = fmaf(q, scale, bias), bit-exact.
cudaError_t dequant_f32(const WeightView &w, float *out, cudaStream_t stream);

// out f32 [count, K]: row i = dequant(row ids[i]) * multiplier; ids on the device, all < N.
cudaError_t gather_dequant_f32(const WeightView &w, const uint32_t *d_ids, uint32_t count, float multiplier,
                               float *out, cudaStream_t stream);

// Dequant-GEMM on tcgen05 for M > 16 (bf16 in/out; 4- and 8-bit codes).  cudaErrorNotSupported when not eligible.
// `ws`: fp32 workspace of gemm_tc_workspace_bytes (one partial tile per CTA, for tiles whose K blocks are shared
// between CTAs); `flags`: gemm_tc_flag_count words, zero between launches.  cudaErrorMemoryAllocation when
// either is too small.
cudaError_t gemm_tc(const WeightView &w, const void *x_bf16, void *y_bf16, uint32_t M,
                    cudaStream_t stream, int sm_count, unsigned int *d_error_word, float *ws, size_t ws_bytes,
                    unsigned int *flags, size_t flag_count);
bool gemm_tc_eligible(const WeightView &w, uint32_t M, uint32_t min_m = 17u);
size_t gemm_tc_workspace_bytes(int sm_count);
size_t gemm_tc_flag_count(int sm_count);

// ---- all-reduce over NVLink peer memory (gaf_peer.cu) ----
constexpr int kPeerMaxRanks = 8;                      // ranks of one node
constexpr int kPeerCtas = 16;                         // CTAs of the all-reduce kernel (always all launched)
constexpr int kPeerThreads = 256;
constexpr size_t kPeerSlotBytes = size_t(1) << 20;    // one rank's tile as 64-bit words: 131072 values (16 rows x 8192)

// Region layout (one cudaMalloc per rank, mapped by every rank of the node):
//   all-reduce kernel: per-CTA call counters, data [2 phases][ranks][slot] of 64-bit words {fp32 value, epoch}
//   fused GEMV + all-reduce: {epoch, done} words, data [4 phases][ranks][slot] holding a rank's partial tile as
//   64-bit words {fp32 value, launch epoch} [activation row][N]
constexpr size_t kPeerEpochOff = 4096;
constexpr size_t kFusedCtlOff = size_t(128) << 10;
constexpr size_t kPeerDataOff = size_t(256) << 10;
constexpr size_t kFusedDataOff = kPeerDataOff + 2 * size_t(kPeerMaxRanks) * kPeerSlotBytes;
constexpr int kFusedPhases = 4;                       // data phases of the exchange fused into the GEMV write-out
constexpr size_t kPeerRegionBytes = kFusedDataOff + kFusedPhases * size_t(kPeerMaxRanks) * kPeerSlotBytes;

struct PeerComm {
    void *region[kPeerMaxRanks];  // every rank's region as mapped into this process; [rank] is cudaMalloc'ed here
    uint32_t rank, size;
    bool ok;                      // all ranks mapped all regions
};

size_t peer_region_bytes();
// In-place sum of d_buf[count] (bf16 or f32) over the ranks.  cudaErrorNotSupported when the tile does not
// fit a slot or the peer mapping is unavailable (the caller then uses NCCL).
// wait_limit: polls per awaited word before a rank gives up (0 = the default of several seconds).
// expect_absent_rank: diagnostic - also wait for the words of rank `size`, which nobody writes, so that the
// bounded wait runs out by design (size < kPeerMaxRanks only).
cudaError_t peer_allreduce(const PeerComm &pc, void *d_buf, size_t count, bool f32, bool pdl, cudaStream_t stream,
                           unsigned int *d_error_word, uint32_t wait_limit = 0, bool expect_absent_rank = false);

}  // namespace tgaf
