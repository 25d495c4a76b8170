// Sideload payload for talu's CUDA backend on B200 (kernels_sm_100.cubin).
//
// talu resolves each kernel op first in a sideloaded cubin named by a manifest
// (core/src/compute/cuda/manifest.zig:5-112, sideload.zig:24-140, registry.zig:77-103)
// and launches it with geometry its host code fixes.  For the grouped-affine
// matvec that is block 256, grid (ceil(out_dim / 8), batch_rows), no dynamic
// shared memory, f32 activations and outputs, and this parameter list
// (core/src/compute/cuda/kernels/ops/quant_ops.cu:46-57, argument order
// gaffine_u4_matvec.zig:74-84).  Inside that contract: one warp per output
// feature, 16-byte loads of the packed row (32 codes per lane and step), the
// deferred form y = sum_g (s * sum q x + b * sum x) with one scale / bias fetch per
// step, activations through the read-only path (the eight warps of a block share
// them in L1).  Bad shapes return silently, as the reference kernel does
// (quant_ops.cu:63-67).
#include <cuda_fp16.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ float sb_to_f32(uint16_t raw, uint32_t tag) {
    // tags of gaffine_u4_matvec.zig:13-14: 0 = f16, 1 = bf16
    return tag == 0u ? __half2float(__ushort_as_half(raw)) : __uint_as_float(static_cast<uint32_t>(raw) << 16);
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256)
talu_gaffine_u4_matvec_f32(const float *__restrict__ input, const uint32_t *__restrict__ packed_weight,
                           const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases,
                           float *__restrict__ out, uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                           uint32_t scales_dtype_tag, uint32_t batch_rows) {
    if (in_dim == 0u || out_dim == 0u || group_size == 0u || batch_rows == 0u) return;
    if ((in_dim & 7u) != 0u || (group_size & 7u) != 0u || in_dim % group_size != 0u || scales_dtype_tag > 1u) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t m = blockIdx.y;
    if (n >= out_dim || m >= batch_rows) return;
    const uint32_t words = in_dim >> 3;
    const uint32_t groups = in_dim / group_size;
    const uint32_t *prow = packed_weight + static_cast<size_t>(n) * words;
    const uint16_t *srow = scales + static_cast<size_t>(n) * groups;
    const uint16_t *brow = biases + static_cast<size_t>(n) * groups;
    const float *x = input + static_cast<size_t>(m) * in_dim;
    float acc = 0.f;
    // 16-byte steps when the row, the activations and the group size allow it (32 codes never straddle a group)
    const bool vec = (words & 3u) == 0u && (group_size & 31u) == 0u && ((reinterpret_cast<uintptr_t>(prow) & 15u) == 0u) &&
                     ((reinterpret_cast<uintptr_t>(x) & 15u) == 0u);
    if (vec) {
        for (uint32_t v = lane; v < (words >> 2); v += 32u) {
            const uint4 w4 = __ldg(reinterpret_cast<const uint4 *>(prow) + v);
            const uint32_t k0 = v * 32u;
            const uint32_t gi = k0 / group_size;
            const float s = sb_to_f32(srow[gi], scales_dtype_tag), b = sb_to_f32(brow[gi], scales_dtype_tag);
            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
            float qx = 0.f, sx = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 xa = __ldg(reinterpret_cast<const float4 *>(x + k0 + 8 * i));
                const float4 xb = __ldg(reinterpret_cast<const float4 *>(x + k0 + 8 * i + 4));
                const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    qx = fmaf(static_cast<float>((ws[i] >> (4 * j)) & 0xFu), xs[j], qx);
                    sx += xs[j];
                }
            }
            acc = fmaf(s, qx, fmaf(b, sx, acc));
        }
    } else {
        for (uint32_t wi = lane; wi < words; wi += 32u) {
            const uint32_t word = prow[wi];
            const uint32_t k0 = wi * 8u;
            const uint32_t gi = k0 / group_size;
            const float s = sb_to_f32(srow[gi], scales_dtype_tag), b = sb_to_f32(brow[gi], scales_dtype_tag);
            float qx = 0.f, sx = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float xv = x[k0 + j];
                qx = fmaf(static_cast<float>((word >> (4 * j)) & 0xFu), xv, qx);
                sx += xv;
            }
            acc = fmaf(s, qx, fmaf(b, sx, acc));
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0u) out[static_cast<size_t>(m) * out_dim + n] = acc;
}
