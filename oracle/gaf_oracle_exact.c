/*
 * CPU oracle, exact part: conversions, quantizer, dequant, float64 truth and
 * a scalar restatement of the reference CUDA kernel's arithmetic.
 * TEST INFRASTRUCTURE ONLY - see gaf_oracle.h.
 *
 * Compile without fp contraction (-ffp-contract=off): the quantizer and the
 * dequant must give the same bits on every machine.
 */
#define _GNU_SOURCE
#include "gaf_oracle.h"
#include "gaf_pool.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------ */
/* conversions                                                         */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
}
static inline float bits_f32(uint32_t b) {
    float v;
    memcpy(&v, &b, 4);
    return v;
}

uint16_t gaf_f32_to_bf16_trunc(float v) { return (uint16_t)(f32_bits(v) >> 16); }

uint16_t gaf_f32_to_bf16_rne(float v) {
    uint32_t b = f32_bits(v);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((b >> 16) | 0x0040u); /* NaN */
    uint32_t lsb = (b >> 16) & 1u;
    b += 0x7FFFu + lsb;
    return (uint16_t)(b >> 16);
}

float gaf_bf16_to_f32(uint16_t v) { return bits_f32((uint32_t)v << 16); }

float gaf_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: man * 2^-24 */
        float f = (float)man * 0x1p-24f;
        return (sign ? -f : f);
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

float gaf_scale_bias_to_f32(int sdtype, uint16_t v) {
    return sdtype == GAF_SCALES_F16 ? gaf_f16_to_f32(v) : gaf_bf16_to_f32(v);
}

void gaf_bf16_to_f32_array(const uint16_t *in, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = gaf_bf16_to_f32(in[i]);
}
void gaf_f32_to_bf16_rne_array(const float *in, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = gaf_f32_to_bf16_rne(in[i]);
}

/* ------------------------------------------------------------------ */
/* unpack helpers                                                      */
/* ------------------------------------------------------------------ */

void gaf_extract_nibbles(uint32_t word, float out[8]) {
    /* byte i -> [low nibble, high nibble], bytes in little-endian order */
    for (int i = 0; i < 4; ++i) {
        uint32_t byte = (word >> (8 * i)) & 0xFFu;
        out[2 * i] = (float)(byte & 0x0Fu);
        out[2 * i + 1] = (float)(byte >> 4);
    }
}

void gaf_extract_bytes(uint32_t word, float out[4]) {
    for (int i = 0; i < 4; ++i) out[i] = (float)((word >> (8 * i)) & 0xFFu);
}

void gaf_extract32_nibbles(const uint8_t in[16], uint8_t out[32]) {
    for (int i = 0; i < 16; ++i) {
        out[2 * i] = in[i] & 0x0F;
        out[2 * i + 1] = in[i] >> 4;
    }
}

/* ------------------------------------------------------------------ */
/* shape rules                                                         */
/* ------------------------------------------------------------------ */

int gaf_validate_shape(size_t N, size_t K, size_t group, int bits, int sdtype) {
    if (bits != 4 && bits != 8) return GAF_ERR_INVALID_ARGUMENT;
    size_t vpw = bits == 4 ? 8 : 4;
    if (N == 0 || K == 0 || group == 0) return GAF_ERR_INVALID_ARGUMENT;
    if (K % vpw != 0 || group % vpw != 0) return GAF_ERR_INVALID_ARGUMENT;
    if (K % group != 0) return GAF_ERR_INVALID_ARGUMENT;
    if (sdtype != GAF_SCALES_F16 && sdtype != GAF_SCALES_BF16) return GAF_ERR_INVALID_ARGUMENT;
    /* MAX_SUPPORTED_GAFFINE_GROUPS, core/src/models/op_types.zig:333 */
    if (K / group > 1024) return GAF_ERR_INVALID_ARGUMENT;
    return GAF_OK;
}

/* ------------------------------------------------------------------ */
/* quantizer: core/src/converter/grouped_affine.zig:448-501            */
/* ------------------------------------------------------------------ */

typedef struct {
    const float *src;
    uint32_t *packed;
    uint16_t *scales;
    uint16_t *biases;
    size_t K, group;
    int bits;
} quant_ctx_t;

static void quantize_rows(size_t r0, size_t r1, void *vctx) {
    const quant_ctx_t *c = (const quant_ctx_t *)vctx;
    const size_t vpw = c->bits == 4 ? 8 : 4;
    const float maxq = c->bits == 4 ? 15.0f : 255.0f;
    const size_t words_per_row = c->K / vpw;
    const size_t groups = c->K / c->group;
    const size_t words_per_group = c->group / vpw;

    for (size_t r = r0; r < r1; ++r) {
        const float *row = c->src + r * c->K;
        uint32_t *prow = c->packed + r * words_per_row;
        for (size_t g = 0; g < groups; ++g) {
            const float *gv = row + g * c->group;
            float lo = gv[0], hi = gv[0];
            for (size_t i = 0; i < c->group; ++i) {
                if (gv[i] < lo) lo = gv[i];
                if (gv[i] > hi) hi = gv[i];
            }
            const float range = hi - lo;
            const float scale = range > 0 ? range / maxq : 0.0f;
            const float bias = lo;
            c->scales[r * groups + g] = gaf_f32_to_bf16_trunc(scale);
            c->biases[r * groups + g] = gaf_f32_to_bf16_trunc(bias);

            for (size_t w = 0; w < words_per_group; ++w) {
                uint32_t word = 0;
                for (size_t j = 0; j < vpw; ++j) {
                    uint32_t q = 0;
                    if (scale > 0) {
                        /* codes come from the UNROUNDED f32 scale / bias */
                        float norm = (gv[w * vpw + j] - bias) / scale;
                        float rq = roundf(norm); /* half away from zero, like @round */
                        rq = fminf(maxq, rq);
                        rq = fmaxf(0.0f, rq);
                        q = (uint32_t)rq;
                    }
                    word |= q << (j * (size_t)c->bits);
                }
                prow[g * words_per_group + w] = word;
            }
        }
    }
}

int gaf_quantize(const float *src, size_t N, size_t K, size_t group, int bits,
                 uint32_t *packed, uint16_t *scales, uint16_t *biases, int nthreads) {
    /* the converter has no K/G <= 1024 limit (only the loader has), and leaves a
     * tensor unquantized when K is not a multiple of the group or of the word
     * width (grouped_affine.zig:522-524): here that is an error return. */
    if (bits != 4 && bits != 8) return GAF_ERR_INVALID_ARGUMENT;
    const size_t vpw = bits == 4 ? 8 : 4;
    if (N == 0 || K == 0 || group == 0) return GAF_ERR_INVALID_ARGUMENT;
    if (K % group != 0 || K % vpw != 0 || group % vpw != 0) return GAF_ERR_INVALID_ARGUMENT;
    quant_ctx_t c = {src, packed, scales, biases, K, group, bits};
    gaf_parallel_for(N, quantize_rows, &c, nthreads);
    return GAF_OK;
}

/* ------------------------------------------------------------------ */
/* dequant: core/src/compute/cpu/quant_decode.zig:64-130               */
/* ------------------------------------------------------------------ */

typedef struct {
    const uint8_t *packed;
    const uint8_t *scales;
    const uint8_t *biases;
    int sdtype;
    size_t K, group;
    int bits;
    float *out_f32;
    double *out_f64;
    const float *a;
    size_t M, N;
} dq_ctx_t;

static inline uint32_t load_u32(const uint8_t *p) {
    uint32_t v;
    memcpy(&v, p, 4);
    return v;
}
static inline uint16_t load_u16(const uint8_t *p) {
    uint16_t v;
    memcpy(&v, p, 2);
    return v;
}

static void dequant_rows(size_t r0, size_t r1, void *vctx) {
    const dq_ctx_t *c = (const dq_ctx_t *)vctx;
    const size_t vpw = c->bits == 4 ? 8 : 4;
    const uint32_t mask = c->bits == 4 ? 0xFu : 0xFFu;
    const size_t words_per_row = c->K / vpw;
    const size_t groups = c->K / c->group;
    const size_t words_per_group = c->group / vpw;
    for (size_t r = r0; r < r1; ++r) {
        const uint8_t *prow = c->packed + r * words_per_row * 4;
        float *orow = c->out_f32 + r * c->K;
        for (size_t g = 0; g < groups; ++g) {
            const float s = gaf_scale_bias_to_f32(c->sdtype, load_u16(c->scales + (r * groups + g) * 2));
            const float b = gaf_scale_bias_to_f32(c->sdtype, load_u16(c->biases + (r * groups + g) * 2));
            for (size_t w = 0; w < words_per_group; ++w) {
                const uint32_t word = load_u32(prow + (g * words_per_group + w) * 4);
                for (size_t j = 0; j < vpw; ++j) {
                    const float q = (float)((word >> (j * (size_t)c->bits)) & mask);
                    /* the reference uses a fused multiply-add (quant_decode.zig:88-96)
                     * and a plain q*s+b (transforms.zig:704,708); q*s is exact in
                     * f32, so both give the same bits. */
                    orow[g * c->group + w * vpw + j] = fmaf(q, s, b);
                }
            }
        }
    }
}

int gaf_dequant_f32(const void *packed, const void *scales, const void *biases,
                    int sdtype, size_t N, size_t K, size_t group, int bits,
                    float *out, int nthreads) {
    int rc = gaf_validate_shape(N, K, group, bits, sdtype);
    if (rc != GAF_OK) return rc;
    dq_ctx_t c;
    memset(&c, 0, sizeof c);
    c.packed = (const uint8_t *)packed;
    c.scales = (const uint8_t *)scales;
    c.biases = (const uint8_t *)biases;
    c.sdtype = sdtype;
    c.K = K;
    c.group = group;
    c.bits = bits;
    c.out_f32 = out;
    gaf_parallel_for(N, dequant_rows, &c, nthreads);
    return GAF_OK;
}

int gaf_gather_dequant_f32(const void *packed, const void *scales, const void *biases, int sdtype,
                           size_t N, size_t K, size_t group, int bits, const uint32_t *ids, size_t count,
                           float multiplier, float *out) {
    int rc = gaf_validate_shape(N, K, group, bits, sdtype);
    if (rc != GAF_OK) return rc;
    const size_t vpw = bits == 4 ? 8 : 4;
    const size_t groups = K / group;
    for (size_t i = 0; i < count; ++i) {
        if (ids[i] >= N) return GAF_ERR_INVALID_TOKEN;
        dq_ctx_t c;
        memset(&c, 0, sizeof c);
        c.packed = (const uint8_t *)packed + (size_t)ids[i] * (K / vpw) * 4;
        c.scales = (const uint8_t *)scales + (size_t)ids[i] * groups * 2;
        c.biases = (const uint8_t *)biases + (size_t)ids[i] * groups * 2;
        c.sdtype = sdtype;
        c.K = K;
        c.group = group;
        c.bits = bits;
        c.out_f32 = out + i * K;
        dequant_rows(0, 1, &c);
        for (size_t k = 0; k < K; ++k) out[i * K + k] *= multiplier;
    }
    return GAF_OK;
}

/* ------------------------------------------------------------------ */
/* float64 truth                                                       */
/* ------------------------------------------------------------------ */

static void truth_rows(size_t n0, size_t n1, void *vctx) {
    const dq_ctx_t *c = (const dq_ctx_t *)vctx;
    const size_t vpw = c->bits == 4 ? 8 : 4;
    const uint32_t mask = c->bits == 4 ? 0xFu : 0xFFu;
    const size_t words_per_row = c->K / vpw;
    const size_t groups = c->K / c->group;
    double *wrow = (double *)malloc(c->K * sizeof(double));
    if (!wrow) return;
    for (size_t n = n0; n < n1; ++n) {
        const uint8_t *prow = c->packed + n * words_per_row * 4;
        for (size_t k = 0; k < c->K; ++k) {
            const size_t g = k / c->group;
            const double s = (double)gaf_scale_bias_to_f32(c->sdtype, load_u16(c->scales + (n * groups + g) * 2));
            const double b = (double)gaf_scale_bias_to_f32(c->sdtype, load_u16(c->biases + (n * groups + g) * 2));
            const uint32_t word = load_u32(prow + (k / vpw) * 4);
            const double q = (double)((word >> ((k % vpw) * (size_t)c->bits)) & mask);
            wrow[k] = q * s + b;
        }
        for (size_t m = 0; m < c->M; ++m) {
            const float *arow = c->a + m * c->K;
            double acc = 0.0;
            for (size_t k = 0; k < c->K; ++k) acc += (double)arow[k] * wrow[k];
            c->out_f64[m * c->N + n] = acc;
        }
    }
    free(wrow);
}

int gaf_matmul_f64(const float *a, size_t M, size_t K, const void *packed,
                   const void *scales, const void *biases, int sdtype,
                   size_t N, size_t group, int bits, double *out, int nthreads) {
    int rc = gaf_validate_shape(N, K, group, bits, sdtype);
    if (rc != GAF_OK) return rc;
    if (M == 0) return GAF_ERR_INVALID_ARGUMENT;
    dq_ctx_t c;
    memset(&c, 0, sizeof c);
    c.packed = (const uint8_t *)packed;
    c.scales = (const uint8_t *)scales;
    c.biases = (const uint8_t *)biases;
    c.sdtype = sdtype;
    c.K = K;
    c.group = group;
    c.bits = bits;
    c.out_f64 = out;
    c.a = a;
    c.M = M;
    c.N = N;
    gaf_parallel_for(N, truth_rows, &c, nthreads);
    return GAF_OK;
}

/* ------------------------------------------------------------------ */
/* reference CUDA kernel arithmetic, scalar                            */
/* core/src/compute/cuda/kernels/ops/quant_ops.cu:46-93                */
/* ------------------------------------------------------------------ */

int gaf_matvec_cuda_semantics_f32(const float *input, const uint32_t *packed,
                                  const uint16_t *scales, const uint16_t *biases,
                                  float *out, uint32_t in_dim, uint32_t out_dim,
                                  uint32_t group_size, uint32_t sdtype,
                                  uint32_t batch_rows) {
    /* host-side validateArgs, core/src/compute/cuda/gaffine_u4_matvec.zig:99-113 */
    if (in_dim == 0 || out_dim == 0 || group_size == 0 || batch_rows == 0) return GAF_ERR_INVALID_ARGUMENT;
    if (in_dim % 8 != 0 || group_size % 8 != 0) return GAF_ERR_INVALID_ARGUMENT;
    if (in_dim % group_size != 0) return GAF_ERR_INVALID_ARGUMENT;
    if (sdtype != GAF_SCALES_F16 && sdtype != GAF_SCALES_BF16) return GAF_ERR_INVALID_ARGUMENT;
    const uint32_t groups = in_dim / group_size;
    const uint32_t words_per_row = in_dim / 8;
    for (uint32_t b = 0; b < batch_rows; ++b) {
        for (uint32_t n = 0; n < out_dim; ++n) {
            /* one warp per output: lane l walks i = l, l+32, ...; lanes are then
             * summed by a shuffle tree (16,8,4,2,1). */
            float lane_acc[32];
            for (int l = 0; l < 32; ++l) lane_acc[l] = 0.0f;
            for (uint32_t i = 0; i < in_dim; ++i) {
                const uint32_t g = i / group_size;
                const uint32_t word = packed[(size_t)n * words_per_row + i / 8];
                const uint32_t q = (word >> ((i & 7) * 4)) & 0xF;
                const float s = gaf_scale_bias_to_f32((int)sdtype, scales[(size_t)n * groups + g]);
                const float bi = gaf_scale_bias_to_f32((int)sdtype, biases[(size_t)n * groups + g]);
                const float dq = (float)q * s + bi;
                lane_acc[i & 31] = fmaf(input[(size_t)b * in_dim + i], dq, lane_acc[i & 31]);
            }
            for (int off = 16; off >= 1; off >>= 1)
                for (int l = 0; l < off; ++l) lane_acc[l] += lane_acc[l + off];
            out[(size_t)b * out_dim + n] = lane_acc[0];
        }
    }
    return GAF_OK;
}

/* ------------------------------------------------------------------ */
/* thread policy: core/src/system/parallel.zig:20-52,278-306           */
/* ------------------------------------------------------------------ */

int gaf_logical_cpu_count(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

int gaf_reference_thread_count(void) {
    const char *env = getenv("THREADS");
    if (env && *env) {
        char *end = NULL;
        long v = strtol(env, &end, 10);
        if (end && *end == '\0' && v > 0) return (int)v;
    }
    int logical = gaf_logical_cpu_count();
    int physical = logical;
#if defined(__x86_64__) || defined(__i386__)
    physical = logical / 2;
    if (physical < 1) physical = 1;
#endif
    int optimal = 8 + physical / 4;
    if (optimal > physical) optimal = physical;
    if (optimal < 1) optimal = 1;
    return optimal;
}
