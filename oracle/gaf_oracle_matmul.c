/*
 * CPU oracle, matmul part: f32 grouped-affine matmul with the reference's
 * deferred-scale structure.  TEST INFRASTRUCTURE ONLY - see gaf_oracle.h.
 *
 * Follows core/src/compute/cpu/matmul_prefill.zig:
 *   u4: entry :28-109, 4x2 micro-kernel :121-358, 1x2 :364-444, 1x1 :450-480
 *   u8: entry :488-569, 4x2 :572-759, 1x2 :762-825, 1x1 :828-858
 * and core/src/compute/cpu/matmul_primitives.zig:784-895 / :977-1033 for the
 * single-row dot products used on an odd last column.
 *
 *   out[m,n] = sum_g ( s[n,g] * sum_{k in g} q[n,k]*x[m,k]
 *                    + b[n,g] * sum_{k in g} x[m,k] )
 *
 * 8-lane f32 vectors (256-bit, the reference's x86 cap), per-group partial
 * sums kept in lanes, horizontal reduction once at the end (4x2) or once per
 * group (1x2).  The reference compiles these loops with reassociation allowed,
 * so agreement with it is to a tolerance, not to the bit; this file fixes one
 * evaluation order so that its own results are reproducible.
 */
#define _GNU_SOURCE
#include "gaf_oracle.h"
#include "gaf_pool.h"

#include <stdlib.h>
#include <string.h>

typedef float v8f __attribute__((vector_size(32)));
typedef float v4f __attribute__((vector_size(16)));
typedef int32_t v8i __attribute__((vector_size(32)));
typedef int32_t v4i __attribute__((vector_size(16)));
typedef uint32_t v8u __attribute__((vector_size(32)));
typedef uint8_t v8u8 __attribute__((vector_size(8)));

#define MAX_GROUPS 1024 /* matmul_primitives.zig:97 */

static inline v8f splat8(float v) { return (v8f){v, v, v, v, v, v, v, v}; }
static inline v4f splat4(float v) { return (v4f){v, v, v, v}; }
static inline v8f load8(const float *p) {
    v8f v;
    memcpy(&v, p, 32);
    return v;
}
static inline v4f load4(const float *p) {
    v4f v;
    memcpy(&v, p, 16);
    return v;
}
static inline float hsum8(v8f v) {
    /* pairwise tree, the shape LLVM emits for @reduce(.Add, ...) */
    float a0 = v[0] + v[4], a1 = v[1] + v[5], a2 = v[2] + v[6], a3 = v[3] + v[7];
    float b0 = a0 + a2, b1 = a1 + a3;
    return b0 + b1;
}
static inline float hsum4(v4f v) { return (v[0] + v[2]) + (v[1] + v[3]); }
static inline v8f fma8(v8f a, v8f b, v8f c) { return a * b + c; } /* contracted to vfmadd */
static inline v4f fma4(v4f a, v4f b, v4f c) { return a * b + c; }

static inline uint32_t ld32(const uint8_t *p) {
    uint32_t v;
    memcpy(&v, p, 4);
    return v;
}
static inline uint16_t ld16(const uint8_t *p) {
    uint16_t v;
    memcpy(&v, p, 2);
    return v;
}

/* 8 nibbles of one word, K order (grouped_affine_quant.zig:24-34) */
static inline v8f nibbles8(uint32_t w) {
    const v8u ww = {w, w, w, w, w, w, w, w};
    const v8u sh = {0, 4, 8, 12, 16, 20, 24, 28};
    const v8u q = (ww >> sh) & 15u;
    return __builtin_convertvector(q, v8f);
}
/* 8 bytes of two words (matmul_prefill.zig:861-864) */
static inline v8f bytes8(const uint8_t *p) {
    v8u8 b;
    memcpy(&b, p, 8);
    return __builtin_convertvector(b, v8f);
}
/* 4 bytes of one word (grouped_affine_quant.zig:60-68) */
static inline v4f bytes4(uint32_t w) {
    v4i q = {(int32_t)(w & 255u), (int32_t)((w >> 8) & 255u), (int32_t)((w >> 16) & 255u),
             (int32_t)(w >> 24)};
    return __builtin_convertvector(q, v4f);
}

typedef struct {
    const float *a;
    const uint8_t *packed;
    const uint8_t *scales;
    const uint8_t *biases;
    int sdtype;
    float *out;
    size_t M, N, K, group;
    size_t words_per_row, groups, group_words;
} mm_ctx_t;

#define SB(ptr, idx) gaf_scale_bias_to_f32(c->sdtype, ld16((ptr) + (size_t)(idx) * 2))

/* ---------------------------------------------------------------- */
/* u4                                                                */
/* ---------------------------------------------------------------- */

static void u4_kernel4x2(const mm_ctx_t *c, size_t row, size_t col) {
    const uint8_t *w0 = c->packed + col * c->words_per_row * 4;
    const uint8_t *w1 = c->packed + (col + 1) * c->words_per_row * 4;
    const float *a0 = c->a + row * c->K;
    const float *a1 = a0 + c->K, *a2 = a1 + c->K, *a3 = a2 + c->K;
    const uint8_t *s0p = c->scales + col * c->groups * 2, *s1p = c->scales + (col + 1) * c->groups * 2;
    const uint8_t *b0p = c->biases + col * c->groups * 2, *b1p = c->biases + (col + 1) * c->groups * 2;

    v8f acc[4][2], bias_acc[4];
    for (int r = 0; r < 4; ++r) {
        acc[r][0] = acc[r][1] = splat8(0);
        bias_acc[r] = splat8(0);
    }
    for (size_t g = 0; g < c->groups; ++g) {
        const float s0 = SB(s0p, g), s1 = SB(s1p, g), b0 = SB(b0p, g), b1 = SB(b1p, g);
        const uint8_t *wg0 = w0 + g * c->group_words * 4, *wg1 = w1 + g * c->group_words * 4;
        const float *x[4] = {a0 + g * c->group, a1 + g * c->group, a2 + g * c->group, a3 + g * c->group};
        v8f wx[4][2], xs[4];
        for (int r = 0; r < 4; ++r) {
            wx[r][0] = wx[r][1] = splat8(0);
            xs[r] = splat8(0);
        }
        size_t p = 0;
        for (; p + 3 < c->group_words; p += 4) { /* 32 weights per column per step */
            v8f n0[4], n1[4];
            for (int j = 0; j < 4; ++j) {
                n0[j] = nibbles8(ld32(wg0 + (p + j) * 4));
                n1[j] = nibbles8(ld32(wg1 + (p + j) * 4));
            }
            for (int r = 0; r < 4; ++r) {
                v8f x0 = load8(x[r] + p * 8), x1 = load8(x[r] + (p + 1) * 8);
                v8f x2 = load8(x[r] + (p + 2) * 8), x3 = load8(x[r] + (p + 3) * 8);
                wx[r][0] = fma8(n0[0], x0, wx[r][0]);
                wx[r][0] = fma8(n0[1], x1, wx[r][0]);
                wx[r][0] = fma8(n0[2], x2, wx[r][0]);
                wx[r][0] = fma8(n0[3], x3, wx[r][0]);
                wx[r][1] = fma8(n1[0], x0, wx[r][1]);
                wx[r][1] = fma8(n1[1], x1, wx[r][1]);
                wx[r][1] = fma8(n1[2], x2, wx[r][1]);
                wx[r][1] = fma8(n1[3], x3, wx[r][1]);
                xs[r] += x0 + x1 + x2 + x3;
            }
        }
        for (; p < c->group_words; ++p) { /* groups that are not a multiple of 32 */
            v8f n0 = nibbles8(ld32(wg0 + p * 4)), n1 = nibbles8(ld32(wg1 + p * 4));
            for (int r = 0; r < 4; ++r) {
                v8f xv = load8(x[r] + p * 8);
                wx[r][0] = fma8(n0, xv, wx[r][0]);
                wx[r][1] = fma8(n1, xv, wx[r][1]);
                xs[r] += xv;
            }
        }
        const v8f s0v = splat8(s0), s1v = splat8(s1), b0v = splat8(b0), b1v = splat8(b1);
        for (int r = 0; r < 4; ++r) {
            acc[r][0] = fma8(wx[r][0], s0v, acc[r][0]);
            acc[r][1] = fma8(wx[r][1], s1v, acc[r][1]);
        }
        for (int r = 0; r < 4; ++r) bias_acc[r] = fma8(xs[r], b0v, bias_acc[r]);
        for (int r = 0; r < 4; ++r) acc[r][1] = fma8(xs[r], b1v, acc[r][1]);
    }
    for (int r = 0; r < 4; ++r) {
        c->out[(row + r) * c->N + col] = hsum8(acc[r][0]) + hsum8(bias_acc[r]);
        c->out[(row + r) * c->N + col + 1] = hsum8(acc[r][1]);
    }
}

static void u4_kernel1x2(const mm_ctx_t *c, size_t row, size_t col) {
    const uint8_t *w0 = c->packed + col * c->words_per_row * 4;
    const uint8_t *w1 = c->packed + (col + 1) * c->words_per_row * 4;
    const float *a = c->a + row * c->K;
    const uint8_t *s0p = c->scales + col * c->groups * 2, *s1p = c->scales + (col + 1) * c->groups * 2;
    const uint8_t *b0p = c->biases + col * c->groups * 2, *b1p = c->biases + (col + 1) * c->groups * 2;
    float out0 = 0, out1 = 0;
    for (size_t g = 0; g < c->groups; ++g) {
        const float s0 = SB(s0p, g), s1 = SB(s1p, g), b0 = SB(b0p, g), b1 = SB(b1p, g);
        const uint8_t *wg0 = w0 + g * c->group_words * 4, *wg1 = w1 + g * c->group_words * 4;
        const float *x = a + g * c->group;
        v8f wx0 = splat8(0), wx1 = splat8(0), xs = splat8(0);
        size_t p = 0;
        for (; p + 3 < c->group_words; p += 4) {
            v8f x0 = load8(x + p * 8), x1 = load8(x + (p + 1) * 8);
            v8f x2 = load8(x + (p + 2) * 8), x3 = load8(x + (p + 3) * 8);
            wx0 = fma8(nibbles8(ld32(wg0 + p * 4)), x0, wx0);
            wx0 = fma8(nibbles8(ld32(wg0 + (p + 1) * 4)), x1, wx0);
            wx0 = fma8(nibbles8(ld32(wg0 + (p + 2) * 4)), x2, wx0);
            wx0 = fma8(nibbles8(ld32(wg0 + (p + 3) * 4)), x3, wx0);
            wx1 = fma8(nibbles8(ld32(wg1 + p * 4)), x0, wx1);
            wx1 = fma8(nibbles8(ld32(wg1 + (p + 1) * 4)), x1, wx1);
            wx1 = fma8(nibbles8(ld32(wg1 + (p + 2) * 4)), x2, wx1);
            wx1 = fma8(nibbles8(ld32(wg1 + (p + 3) * 4)), x3, wx1);
            xs += x0 + x1 + x2 + x3;
        }
        for (; p < c->group_words; ++p) {
            v8f xv = load8(x + p * 8);
            wx0 = fma8(nibbles8(ld32(wg0 + p * 4)), xv, wx0);
            wx1 = fma8(nibbles8(ld32(wg1 + p * 4)), xv, wx1);
            xs += xv;
        }
        /* three horizontal reductions per group (matmul_prefill.zig:434-439) */
        const float swx0 = hsum8(wx0), swx1 = hsum8(wx1), sxs = hsum8(xs);
        out0 += swx0 * s0 + sxs * b0;
        out1 += swx1 * s1 + sxs * b1;
    }
    c->out[row * c->N + col] = out0;
    c->out[row * c->N + col + 1] = out1;
}

float gaf_dot_u4(const float *a, const void *w, const float *scales_f32,
                 const float *biases_f32, size_t group, size_t k_div_group) {
    const uint8_t *wb = (const uint8_t *)w;
    const size_t group_words = group / 8;
    v8f acc0 = splat8(0), acc1 = splat8(0);
    for (size_t g = 0; g < k_div_group; ++g) {
        const uint8_t *wg = wb + g * group_words * 4;
        const float *x = a + g * group;
        v8f l0 = splat8(0), l1 = splat8(0), t0 = splat8(0), t1 = splat8(0);
        size_t p = 0;
        for (; p + 3 < group_words; p += 4) {
            v8f x0 = load8(x + p * 8), x1 = load8(x + (p + 1) * 8);
            v8f x2 = load8(x + (p + 2) * 8), x3 = load8(x + (p + 3) * 8);
            l0 = fma8(nibbles8(ld32(wg + p * 4)), x0, l0);
            l1 = fma8(nibbles8(ld32(wg + (p + 1) * 4)), x1, l1);
            l0 = fma8(nibbles8(ld32(wg + (p + 2) * 4)), x2, l0);
            l1 = fma8(nibbles8(ld32(wg + (p + 3) * 4)), x3, l1);
            t0 += x0;
            t1 += x1;
            t0 += x2;
            t1 += x3;
        }
        for (; p < group_words; ++p) {
            v8f xv = load8(x + p * 8);
            l0 = fma8(nibbles8(ld32(wg + p * 4)), xv, l0);
            t0 += xv;
        }
        acc0 = fma8(l0 + l1, splat8(scales_f32[g]), acc0);
        acc1 = fma8(t0 + t1, splat8(biases_f32[g]), acc1);
    }
    return hsum8(acc0 + acc1);
}

static void u4_kernel1x1(const mm_ctx_t *c, size_t row, size_t col) {
    float sf[MAX_GROUPS], bf[MAX_GROUPS];
    const uint8_t *sp = c->scales + col * c->groups * 2, *bp = c->biases + col * c->groups * 2;
    for (size_t g = 0; g < c->groups; ++g) {
        sf[g] = SB(sp, g);
        bf[g] = SB(bp, g);
    }
    c->out[row * c->N + col] = gaf_dot_u4(c->a + row * c->K, c->packed + col * c->words_per_row * 4,
                                          sf, bf, c->group, c->groups);
}

static void u4_col_pairs(size_t p0, size_t p1, void *vctx) {
    const mm_ctx_t *c = (const mm_ctx_t *)vctx;
    for (size_t cp = p0; cp < p1; ++cp) {
        const size_t col = cp * 2;
        size_t row = 0;
        for (; row + 3 < c->M; row += 4) u4_kernel4x2(c, row, col);
        for (; row < c->M; ++row) u4_kernel1x2(c, row, col);
    }
}

/* ---------------------------------------------------------------- */
/* u8                                                                */
/* ---------------------------------------------------------------- */

static inline v8f pad4to8(v4f v) { return (v8f){v[0], v[1], v[2], v[3], 0, 0, 0, 0}; }

static void u8_kernel4x2(const mm_ctx_t *c, size_t row, size_t col) {
    const uint8_t *w0 = c->packed + col * c->words_per_row * 4;
    const uint8_t *w1 = c->packed + (col + 1) * c->words_per_row * 4;
    const float *a0 = c->a + row * c->K;
    const uint8_t *s0p = c->scales + col * c->groups * 2, *s1p = c->scales + (col + 1) * c->groups * 2;
    const uint8_t *b0p = c->biases + col * c->groups * 2, *b1p = c->biases + (col + 1) * c->groups * 2;
    v8f acc[4][2], bias_acc[4];
    for (int r = 0; r < 4; ++r) {
        acc[r][0] = acc[r][1] = splat8(0);
        bias_acc[r] = splat8(0);
    }
    for (size_t g = 0; g < c->groups; ++g) {
        const float s0 = SB(s0p, g), s1 = SB(s1p, g), b0 = SB(b0p, g), b1 = SB(b1p, g);
        const uint8_t *wg0 = w0 + g * c->group_words * 4, *wg1 = w1 + g * c->group_words * 4;
        v8f wx[4][2], xs[4];
        for (int r = 0; r < 4; ++r) {
            wx[r][0] = wx[r][1] = splat8(0);
            xs[r] = splat8(0);
        }
        size_t p = 0;
        for (; p + 1 < c->group_words; p += 2) { /* 8 bytes = 8 weights per step */
            v8f q0 = bytes8(wg0 + p * 4), q1 = bytes8(wg1 + p * 4);
            for (int r = 0; r < 4; ++r) {
                v8f xv = load8(a0 + r * c->K + g * c->group + p * 4);
                wx[r][0] = fma8(q0, xv, wx[r][0]);
                wx[r][1] = fma8(q1, xv, wx[r][1]);
                xs[r] += xv;
            }
        }
        for (; p < c->group_words; ++p) { /* odd word: 4 weights padded to 8 lanes */
            v8f q0 = pad4to8(bytes4(ld32(wg0 + p * 4))), q1 = pad4to8(bytes4(ld32(wg1 + p * 4)));
            for (int r = 0; r < 4; ++r) {
                v8f xv = pad4to8(load4(a0 + r * c->K + g * c->group + p * 4));
                wx[r][0] = fma8(q0, xv, wx[r][0]);
                wx[r][1] = fma8(q1, xv, wx[r][1]);
                xs[r] += xv;
            }
        }
        const v8f s0v = splat8(s0), s1v = splat8(s1), b0v = splat8(b0), b1v = splat8(b1);
        for (int r = 0; r < 4; ++r) {
            acc[r][0] = fma8(wx[r][0], s0v, acc[r][0]);
            acc[r][1] = fma8(wx[r][1], s1v, acc[r][1]);
        }
        for (int r = 0; r < 4; ++r) bias_acc[r] = fma8(xs[r], b0v, bias_acc[r]);
        for (int r = 0; r < 4; ++r) acc[r][1] = fma8(xs[r], b1v, acc[r][1]);
    }
    for (int r = 0; r < 4; ++r) {
        c->out[(row + r) * c->N + col] = hsum8(acc[r][0]) + hsum8(bias_acc[r]);
        c->out[(row + r) * c->N + col + 1] = hsum8(acc[r][1]);
    }
}

static void u8_kernel1x2(const mm_ctx_t *c, size_t row, size_t col) {
    const uint8_t *w0 = c->packed + col * c->words_per_row * 4;
    const uint8_t *w1 = c->packed + (col + 1) * c->words_per_row * 4;
    const float *a = c->a + row * c->K;
    const uint8_t *s0p = c->scales + col * c->groups * 2, *s1p = c->scales + (col + 1) * c->groups * 2;
    const uint8_t *b0p = c->biases + col * c->groups * 2, *b1p = c->biases + (col + 1) * c->groups * 2;
    float out0 = 0, out1 = 0;
    for (size_t g = 0; g < c->groups; ++g) {
        const float s0 = SB(s0p, g), s1 = SB(s1p, g), b0 = SB(b0p, g), b1 = SB(b1p, g);
        const uint8_t *wg0 = w0 + g * c->group_words * 4, *wg1 = w1 + g * c->group_words * 4;
        const float *x = a + g * c->group;
        v8f wx0 = splat8(0), wx1 = splat8(0), xs = splat8(0);
        size_t p = 0;
        for (; p + 1 < c->group_words; p += 2) {
            v8f xv = load8(x + p * 4);
            wx0 = fma8(bytes8(wg0 + p * 4), xv, wx0);
            wx1 = fma8(bytes8(wg1 + p * 4), xv, wx1);
            xs += xv;
        }
        for (; p < c->group_words; ++p) {
            v4f q0 = bytes4(ld32(wg0 + p * 4)), q1 = bytes4(ld32(wg1 + p * 4));
            v4f xv = load4(x + p * 4);
            out0 += hsum4(q0 * xv) * s0 + hsum4(xv) * b0;
            out1 += hsum4(q1 * xv) * s1 + hsum4(xv) * b1;
        }
        const float sxs = hsum8(xs);
        out0 += hsum8(wx0) * s0 + sxs * b0;
        out1 += hsum8(wx1) * s1 + sxs * b1;
    }
    c->out[row * c->N + col] = out0;
    c->out[row * c->N + col + 1] = out1;
}

float gaf_dot_u8(const float *a, const void *w, const float *scales_f32,
                 const float *biases_f32, size_t group, size_t k_div_group) {
    const uint8_t *wb = (const uint8_t *)w;
    const size_t group_words = group / 4;
    v4f acc0 = splat4(0), acc1 = splat4(0);
    for (size_t g = 0; g < k_div_group; ++g) {
        const uint8_t *wg = wb + g * group_words * 4;
        const float *x = a + g * group;
        v4f l0 = splat4(0), l1 = splat4(0), t0 = splat4(0), t1 = splat4(0);
        size_t p = 0;
        for (; p + 1 < group_words; p += 2) {
            v4f x0 = load4(x + p * 4), x1 = load4(x + (p + 1) * 4);
            l0 = fma4(bytes4(ld32(wg + p * 4)), x0, l0);
            l1 = fma4(bytes4(ld32(wg + (p + 1) * 4)), x1, l1);
            t0 += x0;
            t1 += x1;
        }
        for (; p < group_words; ++p) {
            v4f xv = load4(x + p * 4);
            l0 = fma4(bytes4(ld32(wg + p * 4)), xv, l0);
            t0 += xv;
        }
        acc0 = fma4(l0 + l1, splat4(scales_f32[g]), acc0);
        acc1 = fma4(t0 + t1, splat4(biases_f32[g]), acc1);
    }
    return hsum4(acc0 + acc1);
}

static void u8_kernel1x1(const mm_ctx_t *c, size_t row, size_t col) {
    float sf[MAX_GROUPS], bf[MAX_GROUPS];
    const uint8_t *sp = c->scales + col * c->groups * 2, *bp = c->biases + col * c->groups * 2;
    for (size_t g = 0; g < c->groups; ++g) {
        sf[g] = SB(sp, g);
        bf[g] = SB(bp, g);
    }
    c->out[row * c->N + col] = gaf_dot_u8(c->a + row * c->K, c->packed + col * c->words_per_row * 4,
                                          sf, bf, c->group, c->groups);
}

static void u8_col_pairs(size_t p0, size_t p1, void *vctx) {
    const mm_ctx_t *c = (const mm_ctx_t *)vctx;
    for (size_t cp = p0; cp < p1; ++cp) {
        const size_t col = cp * 2;
        size_t row = 0;
        for (; row + 3 < c->M; row += 4) u8_kernel4x2(c, row, col);
        for (; row < c->M; ++row) u8_kernel1x2(c, row, col);
    }
}

/* ---------------------------------------------------------------- */
/* entry                                                             */
/* ---------------------------------------------------------------- */

int gaf_matmul_f32(const float *a, size_t M, size_t K, const void *packed,
                   const void *scales, const void *biases, int sdtype,
                   size_t N, size_t group, int bits, float *out, int nthreads) {
    int rc = gaf_validate_shape(N, K, group, bits, sdtype);
    if (rc != GAF_OK) return rc;
    if (M == 0 || !a || !out || !packed || !scales || !biases) return GAF_ERR_INVALID_ARGUMENT;
    if (nthreads == 0) nthreads = gaf_reference_thread_count();

    mm_ctx_t c;
    c.a = a;
    c.packed = (const uint8_t *)packed;
    c.scales = (const uint8_t *)scales;
    c.biases = (const uint8_t *)biases;
    c.sdtype = sdtype;
    c.out = out;
    c.M = M;
    c.N = N;
    c.K = K;
    c.group = group;
    c.words_per_row = K / (bits == 4 ? 8 : 4);
    c.groups = K / group;
    c.group_words = group / (bits == 4 ? 8 : 4);

    /* parallel over column pairs (matmul_prefill.zig:76-100, :538-560) */
    gaf_parallel_for(N / 2, bits == 4 ? u4_col_pairs : u8_col_pairs, &c, nthreads);
    if (N % 2 == 1) { /* odd last column on the calling thread (:102-108) */
        for (size_t m = 0; m < M; ++m) {
            if (bits == 4)
                u4_kernel1x1(&c, m, N - 1);
            else
                u8_kernel1x1(&c, m, N - 1);
        }
    }
    return GAF_OK;
}
