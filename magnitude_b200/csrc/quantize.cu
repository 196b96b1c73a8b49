// The format's reference quantizer, fp32 -> Q4_0 / Q8_0 / Q4_K / Q5_K / Q6_K / MXFP4 (host code, threads over rows):
// what a model converter runs once per tensor (reference row "quantizer fp32 -> blocks", upstream of
// LlamaModel::load_from_file, inference/crates/icn-engine/src/lib.rs:972).  Restated from the
// published algorithm of the GGUF reference implementation: Q8_0 takes d = max|w| / 127; Q4_K fits
// every 32-weight sub-block with a weighted least-squares search over 21 candidate scales
// (levels 0..15, minimum <= 0) and then codes the eight scales and minima in 6 bits against fp16 d and
// dmin; Q6_K searches 19 candidate scales per 16-weight sub-block (levels -32..31) and codes the
// sixteen scales as int8 against fp16 d.  Plain fp32 arithmetic in a fixed order, no fused
// multiply-add, so the same input gives the same bytes on every host.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/b200q.h"
#include "common.cuh"

namespace {

constexpr float kGroupMaxEps = 1e-15f;

inline int nearest_int(float v) {      // round to nearest even through the 1.5 * 2^23 trick (|v| < 2^22)
    float t = v + 12582912.f;
    int i;
    memcpy(&i, &t, sizeof(int));
    return (i & 0x007fffff) - 0x00400000;
}

float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t float_to_half(float f) {      // round to nearest even, overflow to infinity
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (a > 0x7F800000u ? 0x200u : 0));
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (a < 0x38800000u) {
        if (a < 0x33000000u) return (uint16_t)sign;
        const int shift = 126 - (int)(a >> 23);
        const uint32_t man = (a & 0x7FFFFFu) | 0x800000u;
        uint32_t half = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = (((a >> 23) - 112) << 10) | ((a & 0x7FFFFFu) >> 13);
    const uint32_t rem = a & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
    return (uint16_t)(sign | half);
}

void put_half(uint8_t *dst, float v) {
    const uint16_t h = float_to_half(v);
    memcpy(dst, &h, 2);
}

// ---- Q8_0: [fp16 d][32 x int8] ------------------------------------------------------------------
void row_q8_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 34) {
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[j]));
        const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
        put_half(y, d);
        for (int j = 0; j < 32; ++j) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * id);
    }
}

// ---- Q4_0: [fp16 d][16 bytes: weights 0..15 in the low nibbles, 16..31 in the high nibbles] -----------
// d = (the value of largest magnitude) / -8, level = min(15, trunc(x / d + 8.5))
void row_q4_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 18) {
        float amax = 0, max = 0;
        for (int j = 0; j < 32; ++j)
            if (amax < fabsf(x[j])) amax = fabsf(x[j]), max = x[j];
        const float d = max / -8, id = d ? 1.0f / d : 0.0f;
        put_half(y, d);
        for (int j = 0; j < 16; ++j) {
            const uint8_t a = (uint8_t)std::min(15, (int)(uint8_t)(int8_t)(x[j] * id + 8.5f));
            const uint8_t c = (uint8_t)std::min(15, (int)(uint8_t)(int8_t)(x[16 + j] * id + 8.5f));
            y[2 + j] = (uint8_t)(a | (c << 4));
        }
    }
}

// ---- MXFP4: [e8m0 scale byte][16 bytes of e2m1 codes, weights 0..15 low nibbles, 16..31 high] ----------
// e = floor(log2 max|x|) - 2 + 127 (from the float's exponent), each value to the nearest 2^(e - 128) * kvalue,
// the first of equally near ones
void row_mxfp4(const float *x, uint8_t *y, int64_t k) {
    static const int8_t kv[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 17) {
        float amax = 0;
        for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[j]));
        uint8_t e = 0;
        if (amax > 0) {
            int ex;
            frexpf(amax, &ex);
            e = (uint8_t)std::min(255, std::max(0, ex - 1 - 2 + 127));
        }
        const uint32_t bits = b200q::e8m0_half_bits(e);
        float d;
        memcpy(&d, &bits, 4);
        y[0] = e;
        for (int j = 0; j < 16; ++j) {
            int q[2];
            for (int h = 0; h < 2; ++h) {
                const float v = x[16 * h + j];
                int best = 0;
                float best_err = fabsf((float)kv[0] * d - v);
                for (int c = 1; c < 16; ++c) {
                    const float err = fabsf((float)kv[c] * d - v);
                    if (err < best_err) best = c, best_err = err;
                }
                q[h] = best;
            }
            y[1 + j] = (uint8_t)(q[0] | (q[1] << 4));
        }
    }
}

// ---- Q4_K: [fp16 d][fp16 dmin][12 bytes of 6-bit scales and minima][128 bytes of nibbles] ---------
// weighted fit of x ~ scale * L + min over levels L in 0..nmax with min <= 0; returns the scale,
// *neg_min = -min
float fit_affine(int n, int nmax, const float *x, const float *wt, uint8_t *L, float *neg_min, uint8_t *Ltry,
                 float rmin = -1.f, float rdelta = 0.1f, int nstep = 20) {
    float lo = x[0], hi = x[0], sw = wt[0], sx = wt[0] * x[0];
    for (int i = 1; i < n; ++i) {
        lo = std::min(lo, x[i]);
        hi = std::max(hi, x[i]);
        sw += wt[i];
        sx += wt[i] * x[i];
    }
    if (lo > 0) lo = 0;
    if (hi == lo) {
        memset(L, 0, (size_t)n);
        *neg_min = -lo;
        return 0.f;
    }
    float iscale = (float)nmax / (hi - lo), scale = 1 / iscale, best = 0;
    for (int i = 0; i < n; ++i) {
        const int l = std::min(nmax, std::max(0, nearest_int(iscale * (x[i] - lo))));
        L[i] = (uint8_t)l;
        const float diff = scale * L[i] + lo - x[i];
        best += wt[i] * (diff * diff);
    }
    for (int step = 0; step <= nstep; ++step) {
        iscale = (rmin + rdelta * step + nmax) / (hi - lo);
        float sl = 0, sl2 = 0, sxl = 0;
        for (int i = 0; i < n; ++i) {
            const int l = std::min(nmax, std::max(0, nearest_int(iscale * (x[i] - lo))));
            Ltry[i] = (uint8_t)l;
            sl += wt[i] * l;
            sl2 += wt[i] * l * l;
            sxl += wt[i] * l * x[i];
        }
        const float D = sw * sl2 - sl * sl;
        if (D > 0) {
            float s = (sw * sxl - sx * sl) / D, m = (sl2 * sx - sl * sxl) / D;
            if (m > 0) {
                m = 0;
                s = sxl / sl2;
            }
            float err = 0;
            for (int i = 0; i < n; ++i) {
                const float diff = s * Ltry[i] + m - x[i];
                err += wt[i] * (diff * diff);
            }
            if (err < best) {
                memcpy(L, Ltry, (size_t)n);
                best = err;
                scale = s;
                lo = m;
            }
        }
    }
    *neg_min = -lo;
    return scale;
}

void scale_min_6bit(int j, const uint8_t *q, int *sc, int *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Q5_K is the same scheme with 32 levels: [d][dmin][scales 12][32 bytes of fifth bits][128 bytes of nibbles];
// its sub-block search runs over iscale = (-0.5 + 0.1 step + 31) / range, step 0..15.
template <int NMAX>
void row_q45_k(const float *x, uint8_t *y, int64_t k) {
    constexpr int kBlock = NMAX == 15 ? 144 : 176;
    uint8_t L[256], Ltry[32];
    float wt[32], mins[8], scales[8];
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += kBlock) {
        float max_scale = 0, max_min = 0;
        for (int j = 0; j < 8; ++j) {
            float sum2 = 0;
            for (int l = 0; l < 32; ++l) sum2 += x[32 * j + l] * x[32 * j + l];
            const float av = sqrtf(sum2 / 32);
            for (int l = 0; l < 32; ++l) wt[l] = av + fabsf(x[32 * j + l]);
            scales[j] = NMAX == 15 ? fit_affine(32, 15, x + 32 * j, wt, L + 32 * j, &mins[j], Ltry)
                                   : fit_affine(32, 31, x + 32 * j, wt, L + 32 * j, &mins[j], Ltry, -0.5f, 0.1f, 15);
            max_scale = std::max(max_scale, scales[j]);
            max_min = std::max(max_min, mins[j]);
        }
        const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f, inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        uint8_t *sc12 = y + 4;
        memset(sc12, 0, 12);
        for (int j = 0; j < 8; ++j) {
            const int ls = std::min(63, nearest_int(inv_scale * scales[j])), lm = std::min(63, nearest_int(inv_min * mins[j]));
            if (j < 4) {
                sc12[j] = (uint8_t)ls;
                sc12[j + 4] = (uint8_t)lm;
            } else {
                sc12[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                sc12[j - 4] |= (uint8_t)((ls >> 4) << 6);
                sc12[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        put_half(y, max_scale / 63.f);
        put_half(y + 2, max_min / 63.f);
        uint16_t hd, hm;
        memcpy(&hd, y, 2);
        memcpy(&hm, y + 2, 2);
        const float fd = half_to_float(hd), fm = half_to_float(hm);
        for (int j = 0; j < 8; ++j) {
            int sc, mn;
            scale_min_6bit(j, sc12, &sc, &mn);
            const float d = fd * sc;
            if (!d) continue;      // keeps the levels of the per-sub-block search
            const float dm = fm * mn;
            for (int i = 0; i < 32; ++i) L[32 * j + i] = (uint8_t)std::min(NMAX, std::max(0, nearest_int((x[32 * j + i] + dm) / d)));
        }
        if (NMAX == 15) {
            uint8_t *q = y + 16;
            for (int j = 0; j < 256; j += 64, q += 32)
                for (int l = 0; l < 32; ++l) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
        } else {
            uint8_t *qh = y + 16, *q = y + 48;
            memset(qh, 0, 32);
            for (int j = 0, bit = 0; j < 256; j += 64, q += 32, bit += 2)
                for (int l = 0; l < 32; ++l) {
                    const int l1 = L[j + l], l2 = L[j + l + 32];
                    qh[l] |= (uint8_t)(((l1 >> 4) << bit) | ((l2 >> 4) << (bit + 1)));
                    q[l] = (uint8_t)((l1 & 15) | ((l2 & 15) << 4));
                }
        }
    }
}
void row_q4_k(const float *x, uint8_t *y, int64_t k) { row_q45_k<15>(x, y, k); }
void row_q5_k(const float *x, uint8_t *y, int64_t k) { row_q45_k<31>(x, y, k); }

// ---- Q6_K: [128 low nibbles][64 bytes of high bit pairs][16 int8 scales][fp16 d] ---------------------
// symmetric fit x ~ scale * l, l in -nmax..nmax-1, weights x^2; stores l + nmax
float fit_symmetric(int n, int nmax, const float *x, int8_t *L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) amax = ax, max = x[i];
    }
    if (amax < kGroupMaxEps) {
        memset(L, 0, (size_t)n);
        return 0.f;
    }
    float iscale = -(float)nmax / max, sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        const int l = std::min(nmax - 1, std::max(-nmax, nearest_int(iscale * x[i])));
        L[i] = (int8_t)(l + nmax);
        const float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.f, best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            const int l = std::min(nmax - 1, std::max(-nmax, nearest_int(iscale * x[i])));
            const float w = x[i] * x[i];
            sumlx += w * x[i] * l;
            suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) L[i] = (int8_t)(nmax + std::min(nmax - 1, std::max(-nmax, nearest_int(iscale * x[i]))));
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

void row_q6_k(const float *x, uint8_t *y, int64_t k) {
    int8_t L[256];
    float scales[16];
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += 210) {
        float max_scale = 0, max_abs = 0;
        for (int ib = 0; ib < 16; ++ib) {
            scales[ib] = fit_symmetric(16, 32, x + 16 * ib, L + 16 * ib);
            if (fabsf(scales[ib]) > max_abs) max_abs = fabsf(scales[ib]), max_scale = scales[ib];
        }
        if (max_abs < kGroupMaxEps) {
            memset(y, 0, 210);
            continue;
        }
        const float iscale = -128.f / max_scale;
        put_half(y + 208, 1 / iscale);
        uint16_t hd;
        memcpy(&hd, y + 208, 2);
        const float fd = half_to_float(hd);
        int8_t *sc = reinterpret_cast<int8_t *>(y + 192);
        for (int ib = 0; ib < 16; ++ib) sc[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
        for (int j = 0; j < 16; ++j) {
            const float d = fd * sc[j];
            if (!d) continue;      // keeps the levels of the per-sub-block search
            for (int i = 0; i < 16; ++i) L[16 * j + i] = (int8_t)(std::min(31, std::max(-32, nearest_int(x[16 * j + i] / d))) + 32);
        }
        uint8_t *ql = y, *qh = y + 128;
        for (int j = 0; j < 256; j += 128, ql += 64, qh += 32)
            for (int l = 0; l < 32; ++l) {
                const uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
                ql[l] = (uint8_t)(q1 | (q3 << 4));
                ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
    }
}

}  // namespace

extern "C" b200q_status b200q_quantize(int32_t type, const float *weights, int64_t N, int64_t K, void *packed_out, size_t out_bytes,
                                       int32_t threads) {
    const int64_t want = b200q_tensor_storage_bytes(type, N < 0 || K < 0 ? -1 : N * K);
    if ((type != B200Q_TYPE_MXFP4 && type != B200Q_TYPE_Q4_0 && type != B200Q_TYPE_Q8_0 && type != B200Q_TYPE_Q4_K && type != B200Q_TYPE_Q5_K && type != B200Q_TYPE_Q6_K) || N < 0 || K < 0) return B200Q_ERR_INVALID_CONFIG;
    const int64_t blk = (type == B200Q_TYPE_Q8_0 || type == B200Q_TYPE_Q4_0 || type == B200Q_TYPE_MXFP4) ? 32 : 256, bb = type == B200Q_TYPE_MXFP4 ? 17 : type == B200Q_TYPE_Q4_0 ? 18 : type == B200Q_TYPE_Q8_0 ? 34 : type == B200Q_TYPE_Q4_K ? 144 : type == B200Q_TYPE_Q5_K ? 176 : 210;
    if (K % blk || want < 0 || (int64_t)out_bytes != want) return B200Q_ERR_INVALID_CONFIG;
    if (N * K == 0) return B200Q_OK;
    if (!weights || !packed_out) return B200Q_ERR_INVALID_CONFIG;
    const int64_t rb = K / blk * bb;
    int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
    nt = (int)std::max<int64_t>(1, std::min<int64_t>(nt, N));
    auto work = [=](int64_t r0, int64_t r1) {
        for (int64_t r = r0; r < r1; ++r) {
            const float *x = weights + r * K;
            uint8_t *y = reinterpret_cast<uint8_t *>(packed_out) + r * rb;
            if (type == B200Q_TYPE_Q8_0) row_q8_0(x, y, K);
            else if (type == B200Q_TYPE_Q4_0) row_q4_0(x, y, K);
            else if (type == B200Q_TYPE_MXFP4) row_mxfp4(x, y, K);
            else if (type == B200Q_TYPE_Q4_K) row_q4_k(x, y, K);
            else if (type == B200Q_TYPE_Q5_K) row_q5_k(x, y, K);
            else row_q6_k(x, y, K);
        }
    };
    std::vector<std::thread> pool;
    try {
        for (int t = 1; t < nt; ++t) pool.emplace_back(work, N * t / nt, N * (t + 1) / nt);
    } catch (...) {
        for (auto &th : pool) th.join();
        work(0, N);      // no threads to be had: do it all here
        return B200Q_OK;
    }
    work(0, N / nt);
    for (auto &th : pool) th.join();
    return B200Q_OK;
}
