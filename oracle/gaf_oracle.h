/*
 * CPU oracle for talu's grouped-affine (gaf4 / gaf8) quantized matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * CPU algorithm, used as the checker in tests, in the smoke check and as the
 * timed CPU baseline of the benchmark.  The product (the CUDA library) never
 * links, loads or calls it.
 *
 * Parity status: the reference (Zig 0.15) cannot be compiled where this was
 * written, so the restatement is pinned against every known-answer test that
 * the reference's own unit tests hold for this path (nibble/byte order, scale
 * decode, dequant rows, dot products, matmul results, CUDA self-test vectors).
 * The exact codes an arbitrary fp32 row quantizes to are NOT pinned by any
 * reference test ("parity unpinned" for the quantizer on random data): there
 * the restatement follows core/src/converter/grouped_affine.zig:448-501 line by
 * line.
 *
 * Layout (reference: core/src/converter/grouped_affine.zig:565-593):
 *   packed  u32 [N, K/vpw]   value j of a word sits at bits [j*bits,(j+1)*bits)
 *   scales  u16 [N, K/G]     bf16 (or f16) bit patterns
 *   biases  u16 [N, K/G]
 *   w[n,k] = f32(q[n,k]) * f32(scale[n,k/G]) + f32(bias[n,k/G])
 */
#ifndef GAF_ORACLE_H
#define GAF_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* scales dtype tags follow the reference's CUDA wrapper
 * (core/src/compute/cuda/gaffine_u4_matvec.zig:13-14): 0 = f16, 1 = bf16. */
#define GAF_SCALES_F16 0
#define GAF_SCALES_BF16 1

/* status codes */
#define GAF_OK 0
#define GAF_ERR_INVALID_ARGUMENT 1

/* core/src/converter/root.zig:504-507, core/src/dtype.zig:345-348: truncation. */
uint16_t gaf_f32_to_bf16_trunc(float v);
/* round-to-nearest-even bf16, used only to build bf16 activations / outputs. */
uint16_t gaf_f32_to_bf16_rne(float v);
/* core/src/dtype.zig:278-281 */
float gaf_bf16_to_f32(uint16_t v);
/* core/src/dtype.zig:165-167 */
float gaf_f16_to_f32(uint16_t v);
/* core/src/compute/cpu/quant/grouped_affine_quant.zig:12-20 */
float gaf_scale_bias_to_f32(int sdtype, uint16_t v);

/* core/src/compute/cpu/quant/grouped_affine_quant.zig:24-34 */
void gaf_extract_nibbles(uint32_t word, float out[8]);
/* core/src/compute/cpu/quant/grouped_affine_quant.zig:60-68 */
void gaf_extract_bytes(uint32_t word, float out[4]);
/* core/src/compute/cpu/simd/arch/root.zig:61-79 */
void gaf_extract32_nibbles(const uint8_t in[16], uint8_t out[32]);

/* Shape rules shared by the converter, loader and CUDA wrapper
 * (grouped_affine.zig:515-524, transforms.zig:158-185,
 *  gaffine_u4_matvec.zig:99-113). Returns GAF_OK or GAF_ERR_INVALID_ARGUMENT. */
int gaf_validate_shape(size_t N, size_t K, size_t group, int bits, int sdtype);

/* quantizeRowSlice, core/src/converter/grouped_affine.zig:448-501.
 * nthreads <= 1 runs inline; the result does not depend on nthreads. */
int gaf_quantize(const float *src, size_t N, size_t K, size_t group, int bits,
                 uint32_t *packed, uint16_t *scales, uint16_t *biases,
                 int nthreads);

/* decodeGroupedAffineU4Row / U8Row, core/src/compute/cpu/quant_decode.zig:64-130
 * (scalar twin: core/src/models/load/transforms.zig:651-714). */
int gaf_dequant_f32(const void *packed, const void *scales, const void *biases,
                    int sdtype, size_t N, size_t K, size_t group, int bits,
                    float *out, int nthreads);

/* gatherDecodeGroupedAffineU4Rows / U8Rows, core/src/compute/cpu/quant_decode.zig:133-210, with the
 * multiplier of the reference's CUDA embedding kernel
 * (core/src/compute/cuda/kernels/ops/quant_ops.cu:12-44): out[i, :] = dequant(row ids[i]) * multiplier.
 * Returns GAF_ERR_INVALID_TOKEN when an id is >= N (the reference's error.InvalidTokenId). */
#define GAF_ERR_INVALID_TOKEN 2
int gaf_gather_dequant_f32(const void *packed, const void *scales, const void *biases, int sdtype,
                           size_t N, size_t K, size_t group, int bits, const uint32_t *ids, size_t count,
                           float multiplier, float *out);

/* matmulGaffineU4Prefill / matmulGaffineU8Prefill,
 * core/src/compute/cpu/matmul_prefill.zig:28-480 and :488-864.
 * a f32 [M,K], out f32 [M,N].  nthreads = 0 picks the reference's policy
 * (gaf_reference_thread_count). */
int gaf_matmul_f32(const float *a, size_t M, size_t K, const void *packed,
                   const void *scales, const void *biases, int sdtype,
                   size_t N, size_t group, int bits, float *out, int nthreads);

/* float64 ground truth: out[m,n] = sum_k a[m,k] * (q*s + b) in double. */
int gaf_matmul_f64(const float *a, size_t M, size_t K, const void *packed,
                   const void *scales, const void *biases, int sdtype,
                   size_t N, size_t group, int bits, double *out, int nthreads);

/* gaffineU4DotProductOpt / gaffineU8DotProductOpt,
 * core/src/compute/cpu/matmul_primitives.zig:784-895, :977-1033
 * (scales / biases already f32). */
float gaf_dot_u4(const float *a, const void *w, const float *scales_f32,
                 const float *biases_f32, size_t group, size_t k_div_group);
float gaf_dot_u8(const float *a, const void *w, const float *scales_f32,
                 const float *biases_f32, size_t group, size_t k_div_group);

/* Reference CUDA kernel semantics (per-element dequant then fma, f32 in/out):
 * core/src/compute/cuda/kernels/ops/quant_ops.cu:46-93.  Scalar restatement,
 * used to check the self-test vectors the reference's CUDA backend holds. */
int gaf_matvec_cuda_semantics_f32(const float *input, const uint32_t *packed,
                                  const uint16_t *scales, const uint16_t *biases,
                                  float *out, uint32_t in_dim, uint32_t out_dim,
                                  uint32_t group_size, uint32_t sdtype,
                                  uint32_t batch_rows);

/* core/src/system/parallel.zig:20-52,278-306: THREADS env, else
 * min(physical, 8 + physical/4) with physical = logical/2 on x86. */
int gaf_reference_thread_count(void);
int gaf_logical_cpu_count(void);

/* helpers for the bf16 activation/ output convention of the GPU path */
void gaf_bf16_to_f32_array(const uint16_t *in, float *out, size_t n);
void gaf_f32_to_bf16_rne_array(const float *in, uint16_t *out, size_t n);

#ifdef __cplusplus
}
#endif
#endif
