/*
 * CPU oracle for the GGUF block-quantized projection matmul (Q4_0 / Q8_0 / Q4_K / Q5_K / Q6_K / MXFP4).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls this
 * file; it exists so the tests, the smoke check and the bench's CPU-baseline leg have an
 * independent statement of the arithmetic to compare the CUDA path against.
 *
 * PARITY UNPINNED at the reference boundary.  The reference engine delegates every
 * projection to `context.decode(batch)` (inference/crates/icn-engine/src/lib.rs:2264), which
 * runs ggml's MUL_MAT inside ggml-org/llama.cpp @ 0b1bad14ff204627636aeb1de22ddcd5acb859d4
 * (pinned in inference/native-pin.toml:3-14).  That source tree is an un-vendored submodule
 * and is not available, and the reference holds no golden vector for a quantized matmul.
 * What this file restates is the published ggml block-format algorithm of that dependency:
 *   - block layouts block_q8_0 / block_q4_K / block_q5_K / block_q6_K / block_q8_K,
 *   - dequantize_row_{q8_0,q4_K,q5_K,q6_K},
 *   - the reference quantizers quantize_row_{q8_0,q4_K,q5_K,q6_K}_ref and their helpers
 *     make_qkx2_quants / make_qx_quants,
 *   - the CPU backend's MUL_MAT strategy: quantize the activation row to Q8_0 (for Q8_0
 *     weights) or Q8_K (for K-quants), integer block dots, fp32 scale-and-accumulate.
 * It is pinned instead against the independent `gguf` Python package (dequantize for all
 * four types, quantize for Q8_0) through the fixtures under tests/golden/.
 *
 * Floating-point contract for dequantization (bit-exact target of the CUDA path):
 *   fp16 -> fp32 exact; every product and difference is a separately rounded fp32
 *   operation, no fused multiply-add (build with -ffp-contract=off):
 *     Q8_0:  w = d * q
 *     Q4_0:  w = (q - 8) * d
 *     MXFP4: w = kvalue[q] * 2^(e - 128)
 *     Q4_K:  w = (d * sc) * q - (dmin * m)
 *     Q5_K:  w = (d * sc) * q - (dmin * m)   with q = nibble + 16 * high bit
 *     Q6_K:  w = (d * sc) * q         with q in [-32, 31]
 *
 * Build: see oracle/Makefile (gcc -O3 -ffp-contract=off -fopenmp).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QK8_0 32
#define QK_K 256
#define K_SCALE_SIZE 12
#define GROUP_MAX_EPS 1e-15f

enum { GGQ_TYPE_Q4_0 = 2, GGQ_TYPE_Q8_0 = 8, GGQ_TYPE_Q4_K = 12, GGQ_TYPE_Q5_K = 13, GGQ_TYPE_Q6_K = 14, GGQ_TYPE_MXFP4 = 39 };

#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[QK8_0]; } blk_q8_0;                 /* 34 B  */
typedef struct { uint16_t d; uint8_t qs[QK8_0 / 2]; } blk_q4_0;            /* 18 B  */
typedef struct { uint8_t e; uint8_t qs[QK8_0 / 2]; } blk_mxfp4;            /* 17 B  */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[K_SCALE_SIZE];
                 uint8_t qs[QK_K / 2]; } blk_q4_K;                          /* 144 B */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[K_SCALE_SIZE];
                 uint8_t qh[QK_K / 8]; uint8_t qs[QK_K / 2]; } blk_q5_K;           /* 176 B */
typedef struct { uint8_t ql[QK_K / 2]; uint8_t qh[QK_K / 4];
                 int8_t scales[QK_K / 16]; uint16_t d; } blk_q6_K;          /* 210 B */
typedef struct { float d; int8_t qs[QK_K]; int16_t bsums[QK_K / 16]; } blk_q8_K; /* activation */
#pragma pack(pop)

_Static_assert(sizeof(blk_q8_0) == 34, "q8_0 size");
_Static_assert(sizeof(blk_q4_0) == 18, "q4_0 size");
_Static_assert(sizeof(blk_mxfp4) == 17, "mxfp4 size");
_Static_assert(sizeof(blk_q4_K) == 144, "q4_K size");
_Static_assert(sizeof(blk_q5_K) == 176, "q5_K size");
_Static_assert(sizeof(blk_q6_K) == 210, "q6_K size");
_Static_assert(sizeof(blk_q8_K) == 4 + 256 + 32, "q8_K size");

/* ------------------------------------------------------------------ fp16 / bf16 */

static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even fp32 -> fp16, IEEE semantics (overflow -> inf) */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477FF000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x38800000u) { /* subnormal half or zero */
        if (absx < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        int e = (int)(absx >> 23);
        uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
        int shift = 126 - e; /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t e = (absx >> 23) - 112;
    uint32_t man = absx & 0x7FFFFFu;
    uint32_t half = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

static float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t f32_to_bf16(float f) { /* RNE, nan kept quiet */
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

void ggq_f32_to_bf16(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}
void ggq_bf16_to_f32(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}
void ggq_f32_to_f16(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_f16(src[i]);
}
void ggq_f16_to_f32(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f16_to_f32(src[i]);
}

/* ------------------------------------------------------------------ sizes */

int64_t ggq_block_elems(int type) {
    return (type == GGQ_TYPE_Q8_0 || type == GGQ_TYPE_Q4_0 || type == GGQ_TYPE_MXFP4) ? QK8_0 : (type == GGQ_TYPE_Q4_K || type == GGQ_TYPE_Q5_K || type == GGQ_TYPE_Q6_K) ? QK_K : 0;
}
int64_t ggq_block_bytes(int type) {
    switch (type) {
    case GGQ_TYPE_Q8_0: return sizeof(blk_q8_0);
    case GGQ_TYPE_Q4_0: return sizeof(blk_q4_0);
    case GGQ_TYPE_MXFP4: return sizeof(blk_mxfp4);
    case GGQ_TYPE_Q4_K: return sizeof(blk_q4_K);
    case GGQ_TYPE_Q5_K: return sizeof(blk_q5_K);
    case GGQ_TYPE_Q6_K: return sizeof(blk_q6_K);
    default: return 0;
    }
}
/* bytes = (elements / block) * block_bytes, the rule behind the reference's
 * llama_cpp_2::gguf::tensor_storage_bytes call (inference/crates/icn-models/src/gguf.rs:129) */
int64_t ggq_row_bytes(int type, int64_t k) {
    int64_t be = ggq_block_elems(type);
    if (be == 0 || k <= 0 || k % be) return -1;
    return k / be * ggq_block_bytes(type);
}

/* ------------------------------------------------------------------ helpers */

static inline int nearest_int(float fval) {
    /* the published ggml trick: add 1.5 * 2^23 and read the mantissa (round-half-even) */
    float val = fval + 12582912.f;
    int i;
    memcpy(&i, &val, sizeof(int));
    return (i & 0x007fffff) - 0x00400000;
}

static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j - 0] >> 6) << 4));
    }
}

/* ------------------------------------------------------------------ dequantize */

static void dequant_row_q8_0(const blk_q8_0 *x, float *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float d = f16_to_f32(x[i].d);
        for (int j = 0; j < QK8_0; ++j) y[i * QK8_0 + j] = d * (float)x[i].qs[j];
    }
}

/* ggml dequantize_row_q4_0: weights 0..15 are the low nibbles, 16..31 the high nibbles; w = (q - 8) * d */
static void dequant_row_q4_0(const blk_q4_0 *x, float *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float d = f16_to_f32(x[i].d);
        for (int j = 0; j < QK8_0 / 2; ++j) {
            int x0 = (x[i].qs[j] & 0x0F) - 8;
            int x1 = (x[i].qs[j] >> 4) - 8;
            y[i * QK8_0 + j] = (float)x0 * d;
            y[i * QK8_0 + j + QK8_0 / 2] = (float)x1 * d;
        }
    }
}

/* MXFP4 (OCP microscaling): 32 e2m1 values share one e8m0 scale.  ggml keeps the e2m1 values doubled
 * (kvalues_mxfp4) and halves the scale instead: d = 2^(e - 128) (GGML_E8M0_TO_FP32_HALF), w = kvalue[q] * d. */
static const int8_t kvalues_mxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
static float e8m0_to_f32_half(uint8_t e) {
    uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
static void dequant_row_mxfp4(const blk_mxfp4 *x, float *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float d = e8m0_to_f32_half(x[i].e);
        for (int j = 0; j < QK8_0 / 2; ++j) {
            y[i * QK8_0 + j] = (float)kvalues_mxfp4[x[i].qs[j] & 0x0F] * d;
            y[i * QK8_0 + j + QK8_0 / 2] = (float)kvalues_mxfp4[x[i].qs[j] >> 4] * d;
        }
    }
}

static void dequant_row_q4_K(const blk_q4_K *x, float *y, int64_t k) {
    int64_t nb = k / QK_K;
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *q = x[i].qs;
        float d = f16_to_f32(x[i].d);
        float dmin = f16_to_f32(x[i].dmin);
        int is = 0;
        uint8_t sc, m;
        for (int j = 0; j < QK_K; j += 64) {
            get_scale_min_k4(is + 0, x[i].scales, &sc, &m);
            float d1 = d * (float)sc;
            float m1 = dmin * (float)m;
            get_scale_min_k4(is + 1, x[i].scales, &sc, &m);
            float d2 = d * (float)sc;
            float m2 = dmin * (float)m;
            for (int l = 0; l < 32; ++l) *y++ = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; ++l) *y++ = d2 * (float)(q[l] >> 4) - m2;
            q += 32;
            is += 2;
        }
    }
}

/* ggml dequantize_row_q5_K: the fifth bit of sub-block j's weight l is bit j of qh[l] */
static void dequant_row_q5_K(const blk_q5_K *x, float *y, int64_t k) {
    int64_t nb = k / QK_K;
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *ql = x[i].qs;
        const uint8_t *qh = x[i].qh;
        float d = f16_to_f32(x[i].d);
        float dmin = f16_to_f32(x[i].dmin);
        int is = 0;
        uint8_t sc, m;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < QK_K; j += 64) {
            get_scale_min_k4(is + 0, x[i].scales, &sc, &m);
            float d1 = d * (float)sc;
            float m1 = dmin * (float)m;
            get_scale_min_k4(is + 1, x[i].scales, &sc, &m);
            float d2 = d * (float)sc;
            float m2 = dmin * (float)m;
            for (int l = 0; l < 32; ++l) *y++ = d1 * (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (int l = 0; l < 32; ++l) *y++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
            ql += 32;
            is += 2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
}

static void dequant_row_q6_K(const blk_q6_K *x, float *y, int64_t k) {
    int64_t nb = k / QK_K;
    for (int64_t i = 0; i < nb; ++i) {
        float d = f16_to_f32(x[i].d);
        const uint8_t *ql = x[i].ql;
        const uint8_t *qh = x[i].qh;
        const int8_t *sc = x[i].scales;
        for (int n = 0; n < QK_K; n += 128) {
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                int q1 = (int)((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                float s1 = d * (float)sc[is + 0];
                float s2 = d * (float)sc[is + 2];
                float s3 = d * (float)sc[is + 4];
                float s4 = d * (float)sc[is + 6];
                y[l + 0] = s1 * (float)q1;
                y[l + 32] = s2 * (float)q2;
                y[l + 64] = s3 * (float)q3;
                y[l + 96] = s4 * (float)q4;
            }
            y += 128;
            ql += 64;
            qh += 32;
            sc += 8;
        }
    }
}

/* dequantize n_rows rows of k weights each; returns 0 or -1 on a bad type / k */
int ggq_dequantize(int type, const void *packed, float *out, int64_t n_rows, int64_t k) {
    int64_t rb = ggq_row_bytes(type, k);
    if (rb < 0) return -1;
    const uint8_t *p = (const uint8_t *)packed;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        const void *row = p + r * rb;
        float *y = out + r * k;
        if (type == GGQ_TYPE_Q8_0) dequant_row_q8_0((const blk_q8_0 *)row, y, k);
        else if (type == GGQ_TYPE_Q4_0) dequant_row_q4_0((const blk_q4_0 *)row, y, k);
        else if (type == GGQ_TYPE_MXFP4) dequant_row_mxfp4((const blk_mxfp4 *)row, y, k);
        else if (type == GGQ_TYPE_Q4_K) dequant_row_q4_K((const blk_q4_K *)row, y, k);
        else if (type == GGQ_TYPE_Q5_K) dequant_row_q5_K((const blk_q5_K *)row, y, k);
        else dequant_row_q6_K((const blk_q6_K *)row, y, k);
    }
    return 0;
}

/* ------------------------------------------------------------------ quantizers */

static void quant_row_q8_0(const float *x, blk_q8_0 *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; ++j) {
            float v = fabsf(x[i * QK8_0 + j]);
            if (v > amax) amax = v;
        }
        float d = amax / 127.0f;
        float id = d ? 1.0f / d : 0.0f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < QK8_0; ++j) y[i].qs[j] = (int8_t)roundf(x[i * QK8_0 + j] * id);
    }
}

/* ggml quantize_row_q4_0_ref: d = (the value of largest magnitude) / -8, q = min(15, trunc(x / d + 8.5)) */
static void quant_row_q4_0(const float *x, blk_q4_0 *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < QK8_0; ++j) {
            float v = x[i * QK8_0 + j];
            if (amax < fabsf(v)) {
                amax = fabsf(v);
                max = v;
            }
        }
        float d = max / -8;
        float id = d ? 1.0f / d : 0.0f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < QK8_0 / 2; ++j) {
            float x0 = x[i * QK8_0 + 0 + j] * id;
            float x1 = x[i * QK8_0 + QK8_0 / 2 + j] * id;
            uint8_t xi0 = (uint8_t)((int8_t)(x0 + 8.5f));
            uint8_t xi1 = (uint8_t)((int8_t)(x1 + 8.5f));
            xi0 = xi0 > 15 ? 15 : xi0;
            xi1 = xi1 > 15 ? 15 : xi1;
            y[i].qs[j] = (uint8_t)(xi0 | (xi1 << 4));
        }
    }
}

/* ggml quantize_row_mxfp4_ref: e = floor(log2(max|x|)) - 2 + 127, each value to the nearest d * kvalue
 * (the first of equally near ones).  floor(log2) is taken from the float's exponent here. */
static void quant_row_mxfp4(const float *x, blk_mxfp4 *y, int64_t k) {
    int64_t nb = k / QK8_0;
    for (int64_t i = 0; i < nb; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; ++j) {
            float v = fabsf(x[i * QK8_0 + j]);
            if (amax < v) amax = v;
        }
        int ex = 0;
        uint8_t e = 0;
        if (amax > 0.0f) {
            frexpf(amax, &ex);                 /* amax = m * 2^ex, m in [0.5, 1): floor(log2 amax) = ex - 1 */
            int ev = ex - 1 - 2 + 127;
            e = (uint8_t)(ev < 0 ? 0 : ev > 255 ? 255 : ev);
        }
        float d = e8m0_to_f32_half(e);
        y[i].e = e;
        for (int j = 0; j < QK8_0 / 2; ++j) {
            uint8_t q[2];
            for (int h = 0; h < 2; ++h) {
                float v = x[i * QK8_0 + h * (QK8_0 / 2) + j];
                int best = 0;
                float best_err = fabsf((float)kvalues_mxfp4[0] * d - v);
                for (int c = 1; c < 16; ++c) {
                    float err = fabsf((float)kvalues_mxfp4[c] * d - v);
                    if (err < best_err) {
                        best = c;
                        best_err = err;
                    }
                }
                q[h] = (uint8_t)best;
            }
            y[i].qs[j] = (uint8_t)(q[0] | (q[1] << 4));
        }
    }
}

static float make_qkx2_quants(int n, int nmax, const float *x, const float *weights, uint8_t *L,
                              float *the_min, uint8_t *Laux, float rmin, float rdelta, int nstep,
                              int use_mad) {
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        float w = weights[i];
        sum_w += w;
        sum_x += w * x[i];
    }
    if (min > 0) min = 0;
    if (max == min) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        *the_min = -min;
        return 0.f;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1 / iscale;
    float best_mad = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * (x[i] - min));
        L[i] = (uint8_t)(l < 0 ? 0 : l > nmax ? nmax : l);
        float diff = scale * L[i] + min - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        best_mad += weights[i] * diff;
    }
    if (nstep < 1) {
        *the_min = -min;
        return scale;
    }
    for (int is = 0; is <= nstep; ++is) {
        iscale = (rmin + rdelta * is + nmax) / (max - min);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * (x[i] - min));
            l = l < 0 ? 0 : l > nmax ? nmax : l;
            Laux[i] = (uint8_t)l;
            float w = weights[i];
            sum_l += w * l;
            sum_l2 += w * l * l;
            sum_xl += w * l * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0) {
                this_min = 0;
                this_scale = sum_xl / sum_l2;
            }
            float mad = 0;
            for (int i = 0; i < n; ++i) {
                float diff = this_scale * Laux[i] + this_min - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                mad += weights[i] * diff;
            }
            if (mad < best_mad) {
                for (int i = 0; i < n; ++i) L[i] = Laux[i];
                best_mad = mad;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

static void quant_row_q4_K(const float *x, blk_q4_K *y, int64_t k) {
    int64_t nb = k / QK_K;
    uint8_t L[QK_K];
    uint8_t Laux[32];
    float weights[32];
    float mins[QK_K / 32];
    float scales[QK_K / 32];
    for (int64_t i = 0; i < nb; ++i) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < QK_K / 32; ++j) {
            float sum_x2 = 0;
            for (int l = 0; l < 32; ++l) sum_x2 += x[32 * j + l] * x[32 * j + l];
            float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; ++l) weights[l] = av_x + fabsf(x[32 * j + l]);
            scales[j] = make_qkx2_quants(32, 15, x + 32 * j, weights, L + 32 * j, &mins[j], Laux,
                                         -1.f, 0.1f, 20, 0);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        memset(y[i].scales, 0, K_SCALE_SIZE);
        for (int j = 0; j < QK_K / 32; ++j) {
            int ls = nearest_int(inv_scale * scales[j]);
            int lm = nearest_int(inv_min * mins[j]);
            ls = ls > 63 ? 63 : ls;
            lm = lm > 63 ? 63 : lm;
            if (j < 4) {
                y[i].scales[j] = (uint8_t)ls;
                y[i].scales[j + 4] = (uint8_t)lm;
            } else {
                y[i].scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                y[i].scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                y[i].scales[j - 0] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        y[i].d = f32_to_f16(max_scale / 63.f);
        y[i].dmin = f32_to_f16(max_min / 63.f);
        uint8_t sc, m;
        for (int j = 0; j < QK_K / 32; ++j) {
            get_scale_min_k4(j, y[i].scales, &sc, &m);
            float d = f16_to_f32(y[i].d) * sc;
            if (!d) continue; /* keeps the levels of the per-sub-block search */
            float dm = f16_to_f32(y[i].dmin) * m;
            for (int ii = 0; ii < 32; ++ii) {
                int l = nearest_int((x[32 * j + ii] + dm) / d);
                l = l < 0 ? 0 : l > 15 ? 15 : l;
                L[32 * j + ii] = (uint8_t)l;
            }
        }
        uint8_t *q = y[i].qs;
        for (int j = 0; j < QK_K; j += 64) {
            for (int l = 0; l < 32; ++l) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
            q += 32;
        }
        x += QK_K;
    }
}

/* ggml quantize_row_q5_K_ref: the Q4_K scheme with 32 levels (search make_qkx2_quants(32, 31, ..., -0.5, 0.1, 15)) */
static void quant_row_q5_K(const float *x, blk_q5_K *y, int64_t k) {
    int64_t nb = k / QK_K;
    uint8_t L[QK_K];
    uint8_t Laux[32];
    float weights[32];
    float mins[QK_K / 32];
    float scales[QK_K / 32];
    for (int64_t i = 0; i < nb; ++i) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < QK_K / 32; ++j) {
            float sum_x2 = 0;
            for (int l = 0; l < 32; ++l) sum_x2 += x[32 * j + l] * x[32 * j + l];
            float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; ++l) weights[l] = av_x + fabsf(x[32 * j + l]);
            scales[j] = make_qkx2_quants(32, 31, x + 32 * j, weights, L + 32 * j, &mins[j], Laux,
                                         -0.5f, 0.1f, 15, 0);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        memset(y[i].scales, 0, K_SCALE_SIZE);
        for (int j = 0; j < QK_K / 32; ++j) {
            int ls = nearest_int(inv_scale * scales[j]);
            int lm = nearest_int(inv_min * mins[j]);
            ls = ls > 63 ? 63 : ls;
            lm = lm > 63 ? 63 : lm;
            if (j < 4) {
                y[i].scales[j] = (uint8_t)ls;
                y[i].scales[j + 4] = (uint8_t)lm;
            } else {
                y[i].scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                y[i].scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
                y[i].scales[j - 0] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        y[i].d = f32_to_f16(max_scale / 63.f);
        y[i].dmin = f32_to_f16(max_min / 63.f);
        uint8_t sc, m;
        for (int j = 0; j < QK_K / 32; ++j) {
            get_scale_min_k4(j, y[i].scales, &sc, &m);
            float d = f16_to_f32(y[i].d) * sc;
            if (!d) continue;
            float dm = f16_to_f32(y[i].dmin) * m;
            for (int ii = 0; ii < 32; ++ii) {
                int l = nearest_int((x[32 * j + ii] + dm) / d);
                l = l < 0 ? 0 : l > 31 ? 31 : l;
                L[32 * j + ii] = (uint8_t)l;
            }
        }
        uint8_t *qh = y[i].qh;
        uint8_t *ql = y[i].qs;
        memset(qh, 0, QK_K / 8);
        uint8_t m1 = 1, m2 = 2;
        for (int n = 0; n < QK_K; n += 64) {
            for (int j = 0; j < 32; ++j) {
                int l1 = L[n + j];
                if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
                int l2 = L[n + j + 32];
                if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
                ql[j] = (uint8_t)(l1 | (l2 << 4));
            }
            m1 <<= 2;
            m2 <<= 2;
            ql += 32;
        }
        x += QK_K;
    }
}

static float make_qx_quants(int n, int nmax, const float *x, int8_t *L, int rmse_type) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) {
        float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.f;
    }
    float iscale = -(float)nmax / max;
    float sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        int l = nearest_int(iscale * x[i]);
        l = l < -nmax ? -nmax : l > nmax - 1 ? nmax - 1 : l;
        L[i] = (int8_t)(l + nmax);
        float w = rmse_type == 1 ? x[i] * x[i] : rmse_type == 2 ? 1 : rmse_type == 3 ? fabsf(x[i])
                                                                                    : sqrtf(fabsf(x[i]));
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            int l = nearest_int(iscale * x[i]);
            l = l < -nmax ? -nmax : l > nmax - 1 ? nmax - 1 : l;
            float w = rmse_type == 1 ? x[i] * x[i] : rmse_type == 2 ? 1 : rmse_type == 3 ? fabsf(x[i])
                                                                                        : sqrtf(fabsf(x[i]));
            sumlx += w * x[i] * l;
            suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) {
                int l = nearest_int(iscale * x[i]);
                l = l < -nmax ? -nmax : l > nmax - 1 ? nmax - 1 : l;
                L[i] = (int8_t)(nmax + l);
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

static void quant_row_q6_K(const float *x, blk_q6_K *y, int64_t k) {
    int64_t nb = k / QK_K;
    int8_t L[QK_K];
    float scales[QK_K / 16];
    for (int64_t i = 0; i < nb; ++i) {
        float max_scale = 0, max_abs_scale = 0;
        for (int ib = 0; ib < QK_K / 16; ++ib) {
            float scale = make_qx_quants(16, 32, x + 16 * ib, L + 16 * ib, 1);
            scales[ib] = scale;
            float abs_scale = fabsf(scale);
            if (abs_scale > max_abs_scale) { max_abs_scale = abs_scale; max_scale = scale; }
        }
        if (max_abs_scale < GROUP_MAX_EPS) {
            memset(&y[i], 0, sizeof(blk_q6_K));
            y[i].d = f32_to_f16(0.f);
            x += QK_K;
            continue;
        }
        float iscale = -128.f / max_scale;
        y[i].d = f32_to_f16(1 / iscale);
        for (int ib = 0; ib < QK_K / 16; ++ib) {
            int v = nearest_int(iscale * scales[ib]);
            y[i].scales[ib] = (int8_t)(v > 127 ? 127 : v);
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            float d = f16_to_f32(y[i].d) * y[i].scales[j];
            if (!d) continue; /* keeps the levels of the per-sub-block search */
            for (int ii = 0; ii < 16; ++ii) {
                int l = nearest_int(x[16 * j + ii] / d);
                l = l < -32 ? -32 : l > 31 ? 31 : l;
                L[16 * j + ii] = (int8_t)(l + 32);
            }
        }
        uint8_t *ql = y[i].ql;
        uint8_t *qh = y[i].qh;
        for (int j = 0; j < QK_K; j += 128) {
            for (int l = 0; l < 32; ++l) {
                uint8_t q1 = L[j + l + 0] & 0xF;
                uint8_t q2 = L[j + l + 32] & 0xF;
                uint8_t q3 = L[j + l + 64] & 0xF;
                uint8_t q4 = L[j + l + 96] & 0xF;
                ql[l + 0] = (uint8_t)(q1 | (q3 << 4));
                ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) |
                                  ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
            ql += 64;
            qh += 32;
        }
        x += QK_K;
    }
}

/* quantize n_rows rows of k fp32 weights each */
int ggq_quantize(int type, const float *src, void *packed, int64_t n_rows, int64_t k) {
    int64_t rb = ggq_row_bytes(type, k);
    if (rb < 0) return -1;
    uint8_t *p = (uint8_t *)packed;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        void *row = p + r * rb;
        const float *x = src + r * k;
        if (type == GGQ_TYPE_Q8_0) quant_row_q8_0(x, (blk_q8_0 *)row, k);
        else if (type == GGQ_TYPE_Q4_0) quant_row_q4_0(x, (blk_q4_0 *)row, k);
        else if (type == GGQ_TYPE_MXFP4) quant_row_mxfp4(x, (blk_mxfp4 *)row, k);
        else if (type == GGQ_TYPE_Q4_K) quant_row_q4_K(x, (blk_q4_K *)row, k);
        else if (type == GGQ_TYPE_Q5_K) quant_row_q5_K(x, (blk_q5_K *)row, k);
        else quant_row_q6_K(x, (blk_q6_K *)row, k);
    }
    return 0;
}

/* ------------------------------------------------------------------ exact matmul (the oracle) */

/* y[m][n] = sum_k (double)dequant(W)[n][k] * (double)x[m][k], rounded once to fp32.
 * x is fp32 with leading dimension ldx, y is fp32 with leading dimension ldy. */
int ggq_matmul_exact(int type, const void *packed, int64_t n, int64_t k, const float *x, int64_t m,
                     int64_t ldx, float *y, int64_t ldy) {
    int64_t rb = ggq_row_bytes(type, k);
    if (rb < 0) return -1;
    const uint8_t *p = (const uint8_t *)packed;
#pragma omp parallel
    {
        float *wf = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < n; ++r) {
            const void *row = p + r * rb;
            if (type == GGQ_TYPE_Q8_0) dequant_row_q8_0((const blk_q8_0 *)row, wf, k);
            else if (type == GGQ_TYPE_Q4_0) dequant_row_q4_0((const blk_q4_0 *)row, wf, k);
            else if (type == GGQ_TYPE_MXFP4) dequant_row_mxfp4((const blk_mxfp4 *)row, wf, k);
            else if (type == GGQ_TYPE_Q4_K) dequant_row_q4_K((const blk_q4_K *)row, wf, k);
            else if (type == GGQ_TYPE_Q5_K) dequant_row_q5_K((const blk_q5_K *)row, wf, k);
            else dequant_row_q6_K((const blk_q6_K *)row, wf, k);
            for (int64_t t = 0; t < m; ++t) {
                const float *xr = x + t * ldx;
                double acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
                int64_t c = 0;
                for (; c + 4 <= k; c += 4) {
                    acc0 += (double)wf[c] * (double)xr[c];
                    acc1 += (double)wf[c + 1] * (double)xr[c + 1];
                    acc2 += (double)wf[c + 2] * (double)xr[c + 2];
                    acc3 += (double)wf[c + 3] * (double)xr[c + 3];
                }
                for (; c < k; ++c) acc0 += (double)wf[c] * (double)xr[c];
                y[t * ldy + r] = (float)((acc0 + acc1) + (acc2 + acc3));
            }
        }
        free(wf);
    }
    return 0;
}

/* ------------------------------------------------------------------ reference-style CPU path
 * The CPU backend of the pinned dependency does not dequantize: it re-quantizes each
 * activation row to 8-bit blocks and takes integer block dot products.  Restated here as
 * the timed CPU baseline ("port"). */

static void quant_act_q8_0(const float *x, blk_q8_0 *y, int64_t k) { quant_row_q8_0(x, y, k); }

static void quant_act_q8_K(const float *x, blk_q8_K *y, int64_t k) {
    int64_t nb = k / QK_K;
    for (int64_t i = 0; i < nb; ++i) {
        float max = 0, amax = 0;
        for (int j = 0; j < QK_K; ++j) {
            float ax = fabsf(x[j]);
            if (ax > amax) { amax = ax; max = x[j]; }
        }
        if (!amax) {
            y[i].d = 0;
            memset(y[i].qs, 0, QK_K);
            memset(y[i].bsums, 0, sizeof(y[i].bsums));
            x += QK_K;
            continue;
        }
        float iscale = -127.f / max;
        for (int j = 0; j < QK_K; ++j) {
            int v = nearest_int(iscale * x[j]);
            y[i].qs[j] = (int8_t)(v > 127 ? 127 : v);
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            int sum = 0;
            for (int ii = 0; ii < 16; ++ii) sum += y[i].qs[j * 16 + ii];
            y[i].bsums[j] = (int16_t)sum;
        }
        y[i].d = 1 / iscale;
        x += QK_K;
    }
}

static float vec_dot_q8_0_q8_0(int64_t k, const blk_q8_0 *x, const blk_q8_0 *y) {
    int64_t nb = k / QK8_0;
    float sumf = 0;
    for (int64_t ib = 0; ib < nb; ++ib) {
        int sumi = 0;
        for (int j = 0; j < QK8_0; ++j) sumi += x[ib].qs[j] * y[ib].qs[j];
        sumf += sumi * (f16_to_f32(x[ib].d) * f16_to_f32(y[ib].d));
    }
    return sumf;
}

/* ggml_vec_dot_q4_0_q8_0 (generic path) */
static float vec_dot_q4_0_q8_0(int64_t k, const blk_q4_0 *x, const blk_q8_0 *y) {
    int64_t nb = k / QK8_0;
    float sumf = 0;
    for (int64_t i = 0; i < nb; ++i) {
        int sumi0 = 0, sumi1 = 0;
        for (int j = 0; j < QK8_0 / 2; ++j) {
            int v0 = (x[i].qs[j] & 0x0F) - 8;
            int v1 = (x[i].qs[j] >> 4) - 8;
            sumi0 += v0 * y[i].qs[j];
            sumi1 += v1 * y[i].qs[j + QK8_0 / 2];
        }
        sumf += (float)(sumi0 + sumi1) * f16_to_f32(x[i].d) * f16_to_f32(y[i].d);
    }
    return sumf;
}

/* ggml_vec_dot_mxfp4_q8_0 (generic path) */
static float vec_dot_mxfp4_q8_0(int64_t k, const blk_mxfp4 *x, const blk_q8_0 *y) {
    int64_t nb = k / QK8_0;
    float sumf = 0;
    for (int64_t i = 0; i < nb; ++i) {
        int sumi1 = 0, sumi2 = 0;
        for (int j = 0; j < QK8_0 / 2; ++j) {
            sumi1 += y[i].qs[j] * kvalues_mxfp4[x[i].qs[j] & 0xF];
            sumi2 += y[i].qs[j + QK8_0 / 2] * kvalues_mxfp4[x[i].qs[j] >> 4];
        }
        sumf += f16_to_f32(y[i].d) * e8m0_to_f32_half(x[i].e) * (float)(sumi1 + sumi2);
    }
    return sumf;
}

static float vec_dot_q4_K_q8_K(int64_t k, const blk_q4_K *x, const blk_q8_K *y) {
    int64_t nb = k / QK_K;
    float sums[8] = {0};
    float sumf = 0;
    int8_t aux8[QK_K];
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *q4 = x[i].qs;
        const int8_t *q8 = y[i].qs;
        int8_t *a = aux8;
        for (int j = 0; j < QK_K / 64; ++j) {
            for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] & 0xF);
            a += 32;
            for (int l = 0; l < 32; ++l) a[l] = (int8_t)(q4[l] >> 4);
            a += 32;
            q4 += 32;
        }
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) get_scale_min_k4(j, x[i].scales, &sc[j], &mn[j]);
        int sumi = 0;
        for (int j = 0; j < QK_K / 16; ++j) sumi += y[i].bsums[j] * mn[j / 2];
        int32_t aux32[8] = {0};
        a = aux8;
        for (int j = 0; j < QK_K / 32; ++j) {
            int32_t scale = sc[j];
            for (int c = 0; c < 4; ++c) {
                for (int l = 0; l < 8; ++l) aux32[l] += scale * ((int)q8[l] * (int)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * aux32[l];
        float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * sumi;
    }
    for (int l = 0; l < 8; ++l) sumf += sums[l];
    return sumf;
}

/* ggml_vec_dot_q5_K_q8_K (generic path): as Q4_K with the fifth bit added to the unpacked levels */
static float vec_dot_q5_K_q8_K(int64_t k, const blk_q5_K *x, const blk_q8_K *y) {
    int64_t nb = k / QK_K;
    float sums[8] = {0};
    float sumf = 0;
    int8_t aux8[QK_K];
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *q4 = x[i].qs;
        const uint8_t *hm = x[i].qh;
        const int8_t *q8 = y[i].qs;
        int8_t *a = aux8;
        uint8_t m = 1;
        for (int j = 0; j < QK_K / 64; ++j) {
            for (int l = 0; l < 32; ++l) a[l] = (int8_t)((q4[l] & 0xF) + ((hm[l] & m) ? 16 : 0));
            a += 32;
            m <<= 1;
            for (int l = 0; l < 32; ++l) a[l] = (int8_t)((q4[l] >> 4) + ((hm[l] & m) ? 16 : 0));
            a += 32;
            m <<= 1;
            q4 += 32;
        }
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) get_scale_min_k4(j, x[i].scales, &sc[j], &mn[j]);
        int sumi = 0;
        for (int j = 0; j < QK_K / 16; ++j) sumi += y[i].bsums[j] * mn[j / 2];
        int32_t aux32[8] = {0};
        a = aux8;
        for (int j = 0; j < QK_K / 32; ++j) {
            int32_t scale = sc[j];
            for (int c = 0; c < 4; ++c) {
                for (int l = 0; l < 8; ++l) aux32[l] += scale * ((int)q8[l] * (int)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * aux32[l];
        float dmin = f16_to_f32(x[i].dmin) * y[i].d;
        sumf -= dmin * sumi;
    }
    for (int l = 0; l < 8; ++l) sumf += sums[l];
    return sumf;
}

static float vec_dot_q6_K_q8_K(int64_t k, const blk_q6_K *x, const blk_q8_K *y) {
    int64_t nb = k / QK_K;
    float sums[8] = {0};
    int8_t aux8[QK_K];
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *q4 = x[i].ql;
        const uint8_t *qh = x[i].qh;
        const int8_t *q8 = y[i].qs;
        int8_t *a = aux8;
        for (int j = 0; j < QK_K; j += 128) {
            for (int l = 0; l < 32; ++l) {
                a[l + 0] = (int8_t)((q4[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                a[l + 32] = (int8_t)((q4[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                a[l + 64] = (int8_t)((q4[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                a[l + 96] = (int8_t)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            }
            a += 128;
            q4 += 64;
            qh += 32;
        }
        int32_t aux32[8] = {0};
        a = aux8;
        for (int j = 0; j < QK_K / 16; ++j) {
            int scale = x[i].scales[j];
            for (int c = 0; c < 2; ++c) {
                for (int l = 0; l < 8; ++l) aux32[l] += scale * ((int)q8[l] * (int)a[l]);
                q8 += 8;
                a += 8;
            }
        }
        float d = f16_to_f32(x[i].d) * y[i].d;
        for (int l = 0; l < 8; ++l) sums[l] += d * aux32[l];
    }
    float sumf = 0;
    for (int l = 0; l < 8; ++l) sumf += sums[l];
    return sumf;
}

int ggq_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* y[m][n] = W x, computed the reference-CPU way.  threads <= 0 means "all". */
int ggq_matmul_cpu(int type, const void *packed, int64_t n, int64_t k, const float *x, int64_t m,
                   int64_t ldx, float *y, int64_t ldy, int threads) {
    int64_t rb = ggq_row_bytes(type, k);
    if (rb < 0) return -1;
    const uint8_t *p = (const uint8_t *)packed;
    const int act8_0 = type == GGQ_TYPE_Q8_0 || type == GGQ_TYPE_Q4_0 || type == GGQ_TYPE_MXFP4;      /* these pair with Q8_0 activations */
    size_t act_row = act8_0 ? (size_t)(k / QK8_0) * sizeof(blk_q8_0)
                                              : (size_t)(k / QK_K) * sizeof(blk_q8_K);
    uint8_t *act = (uint8_t *)malloc(act_row * (size_t)m);
    if (!act) return -2;
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t t = 0; t < m; ++t) {
        if (act8_0) quant_act_q8_0(x + t * ldx, (blk_q8_0 *)(act + t * act_row), k);
        else quant_act_q8_K(x + t * ldx, (blk_q8_K *)(act + t * act_row), k);
    }
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t r = 0; r < n; ++r) {
        const void *row = p + r * rb;
        for (int64_t t = 0; t < m; ++t) {
            const void *a = act + t * act_row;
            float v;
            if (type == GGQ_TYPE_Q8_0) v = vec_dot_q8_0_q8_0(k, (const blk_q8_0 *)row, (const blk_q8_0 *)a);
            else if (type == GGQ_TYPE_Q4_0) v = vec_dot_q4_0_q8_0(k, (const blk_q4_0 *)row, (const blk_q8_0 *)a);
            else if (type == GGQ_TYPE_MXFP4) v = vec_dot_mxfp4_q8_0(k, (const blk_mxfp4 *)row, (const blk_q8_0 *)a);
            else if (type == GGQ_TYPE_Q4_K) v = vec_dot_q4_K_q8_K(k, (const blk_q4_K *)row, (const blk_q8_K *)a);
            else if (type == GGQ_TYPE_Q5_K) v = vec_dot_q5_K_q8_K(k, (const blk_q5_K *)row, (const blk_q8_K *)a);
            else v = vec_dot_q6_K_q8_K(k, (const blk_q6_K *)row, (const blk_q8_K *)a);
            y[t * ldy + r] = v;
        }
    }
    free(act);
    return 0;
}
