// Sideload payload for talu's CUDA backend on B200 (kernels_sm_100.cubin).
//
// talu resolves each kernel op first in a sideloaded cubin named by a manifest
// (core/src/compute/cuda/manifest.zig:5-112, sideload.zig:24-140, registry.zig:77-103)
// and launches it with geometry its host code fixes.  For the grouped-affine
// matvec that is block 256, grid (ceil(out_dim / 8), batch_rows), no dynamic
// shared memory, f32 activations and outputs, and this parameter list
// (core/src/compute/cuda/kernels/ops/quant_ops.cu:46-57, argument order
// gaffine_u4_matvec.zig:74-84).  The two fused decode kernels the reference
// launches when rows == 1 (engine.zig:4476-4553) have the same contract with
// grid.x = ceil((sum of the output dims) / 8): talu_gaffine_u4_matvec_qkv_f32
// (quant_ops.cu:127-152, geometry gaffine_u4_matvec_qkv.zig:193-198) and
// talu_gaffine_u4_matvec_gate_up_f32 (quant_ops.cu:221-239,
// gaffine_u4_matvec_gate_up.zig:79-85).  Inside that contract: one warp per output
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

// One output feature by one warp: y = sum_g (s_g * sum_k q x + b_g * sum_k x), all lanes return the sum.
// The caller has checked in_dim % 8 == 0, group_size % 8 == 0, in_dim % group_size == 0.
__device__ __forceinline__ float dot_row_warp(const float *__restrict__ x, const uint32_t *__restrict__ packed_weight,
                                              const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases,
                                              uint32_t in_dim, uint32_t n, uint32_t group_size, uint32_t tag, uint32_t lane) {
    const uint32_t words = in_dim >> 3;
    const uint32_t groups = in_dim / group_size;
    const uint32_t *prow = packed_weight + static_cast<size_t>(n) * words;
    const uint16_t *srow = scales + static_cast<size_t>(n) * groups;
    const uint16_t *brow = biases + static_cast<size_t>(n) * groups;
    float acc = 0.f;
    // 16-byte steps when the row, the activations and the group size allow it (32 codes never straddle a group)
    const bool vec = (words & 3u) == 0u && (group_size & 31u) == 0u && ((reinterpret_cast<uintptr_t>(prow) & 15u) == 0u) &&
                     ((reinterpret_cast<uintptr_t>(x) & 15u) == 0u);
    if (vec) {
        for (uint32_t v = lane; v < (words >> 2); v += 32u) {
            const uint4 w4 = __ldg(reinterpret_cast<const uint4 *>(prow) + v);
            const uint32_t k0 = v * 32u;
            const uint32_t gi = k0 / group_size;
            const float s = sb_to_f32(srow[gi], tag), b = sb_to_f32(brow[gi], tag);
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
            const float s = sb_to_f32(srow[gi], tag), b = sb_to_f32(brow[gi], tag);
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
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    return acc;
}

__device__ __forceinline__ bool group_ok(uint32_t in_dim, uint32_t group_size, uint32_t tag) {
    return group_size != 0u && (group_size & 7u) == 0u && in_dim % group_size == 0u && tag <= 1u;
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256)
talu_gaffine_u4_matvec_f32(const float *__restrict__ input, const uint32_t *__restrict__ packed_weight,
                           const uint16_t *__restrict__ scales, const uint16_t *__restrict__ biases,
                           float *__restrict__ out, uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                           uint32_t scales_dtype_tag, uint32_t batch_rows) {
    if (in_dim == 0u || out_dim == 0u || batch_rows == 0u || (in_dim & 7u) != 0u) return;
    if (!group_ok(in_dim, group_size, scales_dtype_tag)) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t m = blockIdx.y;
    if (n >= out_dim || m >= batch_rows) return;
    const float acc = dot_row_warp(input + static_cast<size_t>(m) * in_dim, packed_weight, scales, biases, in_dim, n,
                                   group_size, scales_dtype_tag, lane);
    if (lane == 0u) out[static_cast<size_t>(m) * out_dim + n] = acc;
}

// q | k | v in one launch: warp index over the three output ranges in turn (quant_ops.cu:127-219)
extern "C" __global__ void __launch_bounds__(256)
talu_gaffine_u4_matvec_qkv_f32(const float *__restrict__ input, const uint32_t *__restrict__ q_packed_weight,
                               const uint16_t *__restrict__ q_scales, const uint16_t *__restrict__ q_biases,
                               float *__restrict__ q_out, uint32_t q_out_dim, uint32_t q_group_size,
                               uint32_t q_scales_dtype_tag, const uint32_t *__restrict__ k_packed_weight,
                               const uint16_t *__restrict__ k_scales, const uint16_t *__restrict__ k_biases,
                               float *__restrict__ k_out, uint32_t k_out_dim, uint32_t k_group_size,
                               uint32_t k_scales_dtype_tag, const uint32_t *__restrict__ v_packed_weight,
                               const uint16_t *__restrict__ v_scales, const uint16_t *__restrict__ v_biases,
                               float *__restrict__ v_out, uint32_t v_out_dim, uint32_t v_group_size,
                               uint32_t v_scales_dtype_tag, uint32_t in_dim, uint32_t batch_rows) {
    const uint32_t m = blockIdx.y;
    if (m >= batch_rows || in_dim == 0u || (in_dim & 7u) != 0u) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const float *x = input + static_cast<size_t>(m) * in_dim;
    if (idx < q_out_dim) {
        if (!group_ok(in_dim, q_group_size, q_scales_dtype_tag)) return;
        const float acc = dot_row_warp(x, q_packed_weight, q_scales, q_biases, in_dim, idx, q_group_size, q_scales_dtype_tag, lane);
        if (lane == 0u) q_out[static_cast<size_t>(m) * q_out_dim + idx] = acc;
    } else if (idx - q_out_dim < k_out_dim) {
        if (!group_ok(in_dim, k_group_size, k_scales_dtype_tag)) return;
        const uint32_t n = idx - q_out_dim;
        const float acc = dot_row_warp(x, k_packed_weight, k_scales, k_biases, in_dim, n, k_group_size, k_scales_dtype_tag, lane);
        if (lane == 0u) k_out[static_cast<size_t>(m) * k_out_dim + n] = acc;
    } else if (idx - q_out_dim - k_out_dim < v_out_dim) {
        if (!group_ok(in_dim, v_group_size, v_scales_dtype_tag)) return;
        const uint32_t n = idx - q_out_dim - k_out_dim;
        const float acc = dot_row_warp(x, v_packed_weight, v_scales, v_biases, in_dim, n, v_group_size, v_scales_dtype_tag, lane);
        if (lane == 0u) v_out[static_cast<size_t>(m) * v_out_dim + n] = acc;
    }
}

// gate | up in one launch (quant_ops.cu:221-286)
extern "C" __global__ void __launch_bounds__(256)
talu_gaffine_u4_matvec_gate_up_f32(const float *__restrict__ input, const uint32_t *__restrict__ gate_packed_weight,
                                   const uint16_t *__restrict__ gate_scales, const uint16_t *__restrict__ gate_biases,
                                   float *__restrict__ gate_out, uint32_t gate_out_dim, uint32_t gate_group_size,
                                   uint32_t gate_scales_dtype_tag, const uint32_t *__restrict__ up_packed_weight,
                                   const uint16_t *__restrict__ up_scales, const uint16_t *__restrict__ up_biases,
                                   float *__restrict__ up_out, uint32_t up_out_dim, uint32_t up_group_size,
                                   uint32_t up_scales_dtype_tag, uint32_t in_dim, uint32_t batch_rows) {
    const uint32_t m = blockIdx.y;
    if (m >= batch_rows || in_dim == 0u || (in_dim & 7u) != 0u) return;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const float *x = input + static_cast<size_t>(m) * in_dim;
    if (idx < gate_out_dim) {
        if (!group_ok(in_dim, gate_group_size, gate_scales_dtype_tag)) return;
        const float acc = dot_row_warp(x, gate_packed_weight, gate_scales, gate_biases, in_dim, idx, gate_group_size,
                                       gate_scales_dtype_tag, lane);
        if (lane == 0u) gate_out[static_cast<size_t>(m) * gate_out_dim + idx] = acc;
    } else if (idx - gate_out_dim < up_out_dim) {
        if (!group_ok(in_dim, up_group_size, up_scales_dtype_tag)) return;
        const uint32_t n = idx - gate_out_dim;
        const float acc = dot_row_warp(x, up_packed_weight, up_scales, up_biases, in_dim, n, up_group_size,
                                       up_scales_dtype_tag, lane);
        if (lane == 0u) up_out[static_cast<size_t>(m) * up_out_dim + n] = acc;
    }
}
