// Device building blocks of the streaming projection kernel: the fixed-point activation form,
// its prologue, and the per-type work on one 64-weight unit of one weight row.
#pragma once

#include "common.cuh"

namespace b200q {

// where an activation matrix lives (row m at x + m * ldx elements)
struct XSrc {
    const void *x;
    long long ldx;
    int x_is_bf16;
    int x_vec_ok;       // rows are 16-byte aligned: vector loads allowed
    int K, Kpad;
    const float *gamma; // RMSNorm weight [K] applied on the load (with `rs`), or null
    float rs;           // 1 / sqrt(mean(x^2) + eps) of the row being converted
};

// sum of squares of this thread's share of activation row m (threads tid of T take 8 elements in turn)
__device__ __forceinline__ void load_x8(const XSrc &p, int m, int k0, float (&v)[8]);
__device__ __forceinline__ float row_square_share(const XSrc &p, int m, int tid, int T) {
    float ss = 0.f;
    for (int k0 = tid * 8; k0 < p.K; k0 += T * 8) {
        float v[8];
        load_x8(p, m, k0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);       // elements beyond K load as zero
    }
    return ss;
}
// x * rs * gamma for 8 loaded elements starting at k0
__device__ __forceinline__ void norm_x8(const XSrc &p, int k0, float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (k0 + i < p.K) ? v[i] * p.rs * p.gamma[k0 + i] : 0.f;
}

// byte offset, inside one byte plane of the fixed-point activation, of the 16-byte group that
// holds element k.  Groups are stored [c][unit][16] so a lane's four 16-byte reads of one
// 64-weight unit are contiguous across lanes (no bank conflicts).
template <int QT> __device__ __forceinline__ int xplane_off(int k, int units16) {
    if (QT == QT_Q6_K) {
        // unit = (superblock, 128-half, 16-position half); c = 32-weight quadrant inside the half
        const int unit = ((k >> 8) << 2) | (((k >> 7) & 1) << 1) | ((k >> 4) & 1);
        const int c = (k >> 5) & 3;
        return c * units16 + unit * 16 + (k & 15);
    }
    return ((k >> 4) & 3) * units16 + (k >> 6) * 16 + (k & 15);
}

struct XView {            // shared-window addresses of one activation row in fixed-point form
    uint32_t xh;          // signed high bytes
    uint32_t xl;          // signed low bytes
    uint32_t sx;          // fp32 per 32 weights
    uint32_t isum;        // int32 sum of the 16-bit integers: per 32 weights (Q4_K) or per 16 (Q6_K)
};

// One 64-weight unit of one activation row: 4 groups of 16 weights as byte planes, plus the
// block scales and sums that go with the unit (loaded once per item, reused for its 4 rows).
template <int QT> struct XRegs {
    uint4 h[4];
    uint4 l[4];
    float sx[4];          // Q4_K / Q8_0 use [0], [1]; Q6_K one per 32-weight quadrant
    int is[4];            // Q4_K: [0], [1] 32-weight sums; Q6_K: the four 16-weight sums of this unit

    // gu = global 64-weight unit of the row, gsb = its superblock, j = unit inside the superblock
    __device__ __forceinline__ void load(const XView &xv, int gu, int gsb, int j, int units16) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            h[c] = lds128(xv.xh + c * units16 + gu * 16);
            l[c] = lds128(xv.xl + c * units16 + gu * 16);
        }
        if (QT == QT_Q6_K) {
            // 32-weight scale blocks 8*sb + 4h + c ; 16-weight sums 16*sb + 8h + 2c + ph
            const int hh = j >> 1, ph = j & 1;
            const uint4 s = lds128(xv.sx + (8 * gsb + 4 * hh) * 4);
            sx[0] = __uint_as_float(s.x); sx[1] = __uint_as_float(s.y);
            sx[2] = __uint_as_float(s.z); sx[3] = __uint_as_float(s.w);
            const uint4 i0 = lds128(xv.isum + (16 * gsb + 8 * hh) * 4);
            const uint4 i1 = lds128(xv.isum + (16 * gsb + 8 * hh + 4) * 4);
            is[0] = (int)(ph ? i0.y : i0.x); is[1] = (int)(ph ? i0.w : i0.z);
            is[2] = (int)(ph ? i1.y : i1.x); is[3] = (int)(ph ? i1.w : i1.z);
        } else {
            const uint2 s = lds64(xv.sx + gu * 8);
            sx[0] = __uint_as_float(s.x); sx[1] = __uint_as_float(s.y);
            if (QT == QT_Q4_K || QT == QT_Q5_K || QT == QT_Q4_0 || QT == QT_MXFP4) {
                const uint2 i = lds64(xv.isum + gu * 8);
                is[0] = (int)i.x; is[1] = (int)i.y;
            }
        }
    }
};

// Weights of one 64-weight unit of one row, unpacked once and reused for every activation row.
template <int QT> struct WRegs;

template <> struct WRegs<QT_Q4_K> {
    uint32_t lo[8], hi[8];   // low nibbles = weights 0..31 of the group; hi keeps 16 * nibble
    int scA, mnA, scB, mnB;
    float d, dmin;
    // `rec` = shared address of the 144-byte block, j = 64-weight group 0..3
    __device__ __forceinline__ void load(uint32_t rec, int j) {
        const uint4 hdr = lds128(rec);
        const uint4 qa = lds128(rec + 16 + 32 * j);
        const uint4 qb = lds128(rec + 32 + 32 * j);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t a = word_of(qa, i), b = word_of(qb, i);
            lo[i] = a & 0x0F0F0F0Fu;
            hi[i] = a & 0xF0F0F0F0u;
            lo[4 + i] = b & 0x0F0F0F0Fu;
            hi[4 + i] = b & 0xF0F0F0F0u;
        }
        // 6-bit scales / mins of sub-blocks 2j and 2j+1 (bytes 2(j&1), 2(j&1)+1 of each word)
        const int sh = 16 * (j & 1);
        const uint32_t y2 = (hdr.y >> sh) & 0xFFFFu, z2 = (hdr.z >> sh) & 0xFFFFu, w2 = (hdr.w >> sh) & 0xFFFFu;
        const uint32_t sc_lo = y2 & 0x3F3Fu, mn_lo = z2 & 0x3F3Fu;
        const uint32_t sc_hi = (w2 & 0x0F0Fu) | ((y2 >> 2) & 0x3030u);
        const uint32_t mn_hi = ((w2 >> 4) & 0x0F0Fu) | ((z2 >> 2) & 0x3030u);
        const uint32_t sc2 = (j >= 2) ? sc_hi : sc_lo, mn2 = (j >= 2) ? mn_hi : mn_lo;
        scA = sc2 & 0xFF;
        scB = sc2 >> 8;
        mnA = mn2 & 0xFF;
        mnB = mn2 >> 8;
        d = half_bits_to_float(hdr.x);
        dmin = half_bits_to_float(hdr.x >> 16);
    }
    __device__ __forceinline__ float dot(const XRegs<QT_Q4_K> &xr) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_us(lo[i], word_of(xr.h[0], i), hA);
            lA = dp4a_us(lo[i], word_of(xr.l[0], i), lA);
            hA = dp4a_us(lo[4 + i], word_of(xr.h[1], i), hA);
            lA = dp4a_us(lo[4 + i], word_of(xr.l[1], i), lA);
            hB = dp4a_us(hi[i], word_of(xr.h[2], i), hB);
            lB = dp4a_us(hi[i], word_of(xr.l[2], i), lB);
            hB = dp4a_us(hi[4 + i], word_of(xr.h[3], i), hB);
            lB = dp4a_us(hi[4 + i], word_of(xr.l[3], i), lB);
        }
        const float fa = (float)((hA * 256 + lA) * scA);
        const float fb = (float)(((hB * 256 + lB) >> 4) * scB);   // hi held 16 * nibble: exact shift
        const float ua = (float)(mnA * xr.is[0]);
        const float ub = (float)(mnB * xr.is[1]);
        return xr.sx[0] * (d * fa - dmin * ua) + xr.sx[1] * (d * fb - dmin * ub);
    }
};

// Q5_K record on the device: the Q4_K fields, then the 32 bytes of fifth bits (bit s of byte l belongs
// to weight l of sub-block s).  Levels 0..31 sit one per byte, so both sub-blocks use plain dp4a.
template <> struct WRegs<QT_Q5_K> {
    uint32_t lo[8], hi[8];
    int scA, mnA, scB, mnB;
    float d, dmin;
    __device__ __forceinline__ void load(uint32_t rec, int j) {
        const uint4 hdr = lds128(rec);
        const uint4 qa = lds128(rec + 16 + 32 * j);
        const uint4 qb = lds128(rec + 32 + 32 * j);
        const uint4 ha = lds128(rec + 144);
        const uint4 hb = lds128(rec + 160);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t a = word_of(qa, i), b = word_of(qb, i);
            const uint32_t fa = word_of(ha, i) >> (2 * j), fb = word_of(hb, i) >> (2 * j);
            lo[i] = (a & 0x0F0F0F0Fu) | ((fa & 0x01010101u) << 4);
            hi[i] = ((a >> 4) & 0x0F0F0F0Fu) | ((fa & 0x02020202u) << 3);
            lo[4 + i] = (b & 0x0F0F0F0Fu) | ((fb & 0x01010101u) << 4);
            hi[4 + i] = ((b >> 4) & 0x0F0F0F0Fu) | ((fb & 0x02020202u) << 3);
        }
        const int sh = 16 * (j & 1);
        const uint32_t y2 = (hdr.y >> sh) & 0xFFFFu, z2 = (hdr.z >> sh) & 0xFFFFu, w2 = (hdr.w >> sh) & 0xFFFFu;
        const uint32_t sc_lo = y2 & 0x3F3Fu, mn_lo = z2 & 0x3F3Fu;
        const uint32_t sc_hi = (w2 & 0x0F0Fu) | ((y2 >> 2) & 0x3030u);
        const uint32_t mn_hi = ((w2 >> 4) & 0x0F0Fu) | ((z2 >> 2) & 0x3030u);
        const uint32_t sc2 = (j >= 2) ? sc_hi : sc_lo, mn2 = (j >= 2) ? mn_hi : mn_lo;
        scA = sc2 & 0xFF;
        scB = sc2 >> 8;
        mnA = mn2 & 0xFF;
        mnB = mn2 >> 8;
        d = half_bits_to_float(hdr.x);
        dmin = half_bits_to_float(hdr.x >> 16);
    }
    __device__ __forceinline__ float dot(const XRegs<QT_Q5_K> &xr) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_us(lo[i], word_of(xr.h[0], i), hA);
            lA = dp4a_us(lo[i], word_of(xr.l[0], i), lA);
            hA = dp4a_us(lo[4 + i], word_of(xr.h[1], i), hA);
            lA = dp4a_us(lo[4 + i], word_of(xr.l[1], i), lA);
            hB = dp4a_us(hi[i], word_of(xr.h[2], i), hB);
            lB = dp4a_us(hi[i], word_of(xr.l[2], i), lB);
            hB = dp4a_us(hi[4 + i], word_of(xr.h[3], i), hB);
            lB = dp4a_us(hi[4 + i], word_of(xr.l[3], i), lB);
        }
        const float fa = (float)((hA * 256 + lA) * scA);
        const float fb = (float)((hB * 256 + lB) * scB);
        const float ua = (float)(mnA * xr.is[0]);
        const float ub = (float)(mnB * xr.is[1]);
        return xr.sx[0] * (d * fa - dmin * ua) + xr.sx[1] * (d * fb - dmin * ub);
    }
};

// Q4_0 record on the device: the eight fp16 d of its native blocks, then the nibbles in the Q4_K
// arrangement; w = d (q - 8), so a block's dot is d (sum q x - 8 sum x) with both sums integers.
template <> struct WRegs<QT_Q4_0> {
    uint32_t lo[8], hi[8];   // low nibbles = block 2j; hi keeps 16 * nibble of block 2j + 1
    float dA, dB;
    __device__ __forceinline__ void load(uint32_t rec, int j) {
        const uint4 qa = lds128(rec + 16 + 32 * j);
        const uint4 qb = lds128(rec + 32 + 32 * j);
        const uint32_t dd = lds32(rec + 4 * j);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t a = word_of(qa, i), b = word_of(qb, i);
            lo[i] = a & 0x0F0F0F0Fu;
            hi[i] = a & 0xF0F0F0F0u;
            lo[4 + i] = b & 0x0F0F0F0Fu;
            hi[4 + i] = b & 0xF0F0F0F0u;
        }
        dA = half_bits_to_float(dd);
        dB = half_bits_to_float(dd >> 16);
    }
    __device__ __forceinline__ float dot(const XRegs<QT_Q4_0> &xr) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_us(lo[i], word_of(xr.h[0], i), hA);
            lA = dp4a_us(lo[i], word_of(xr.l[0], i), lA);
            hA = dp4a_us(lo[4 + i], word_of(xr.h[1], i), hA);
            lA = dp4a_us(lo[4 + i], word_of(xr.l[1], i), lA);
            hB = dp4a_us(hi[i], word_of(xr.h[2], i), hB);
            lB = dp4a_us(hi[i], word_of(xr.l[2], i), lB);
            hB = dp4a_us(hi[4 + i], word_of(xr.h[3], i), hB);
            lB = dp4a_us(hi[4 + i], word_of(xr.l[3], i), lB);
        }
        const float fa = (float)((hA * 256 + lA) - 8 * xr.is[0]);
        const float fb = (float)(((hB * 256 + lB) >> 4) - 8 * xr.is[1]);     // hi held 16 * nibble: exact shift
        return xr.sx[0] * (dA * fa) + xr.sx[1] * (dB * fb);
    }
};

// MXFP4 record on the device: the eight scale bytes of its native blocks (16 bytes with padding), then per
// block four words of eight e2m1 codes in weight order.  A look-up turns four codes into the bytes
// 64 + value, so a block's dot is 2^(e - 128) (sum b x - 64 sum x) with both sums integers.
template <> struct WRegs<QT_MXFP4> {
    uint32_t a[8], b[8];     // bytes 64 + value of block 2j (a) and block 2j + 1 (b), four weights per word
    float dA, dB;
    __device__ __forceinline__ void load(uint32_t rec, int j) {
        const uint4 qa = lds128(rec + 16 + 32 * j);
        const uint4 qb = lds128(rec + 32 + 32 * j);
        const uint32_t ee = lds32(rec + 4 * (j >> 1)) >> (16 * (j & 1));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a[2 * i] = mxfp4_bytes(word_of(qa, i));
            a[2 * i + 1] = mxfp4_bytes(word_of(qa, i) >> 16);
            b[2 * i] = mxfp4_bytes(word_of(qb, i));
            b[2 * i + 1] = mxfp4_bytes(word_of(qb, i) >> 16);
        }
        dA = __uint_as_float(e8m0_half_bits(ee & 0xFF));
        dB = __uint_as_float(e8m0_half_bits((ee >> 8) & 0xFF));
    }
    __device__ __forceinline__ float dot(const XRegs<QT_MXFP4> &xr) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_us(a[i], word_of(xr.h[0], i), hA);
            lA = dp4a_us(a[i], word_of(xr.l[0], i), lA);
            hA = dp4a_us(a[4 + i], word_of(xr.h[1], i), hA);
            lA = dp4a_us(a[4 + i], word_of(xr.l[1], i), lA);
            hB = dp4a_us(b[i], word_of(xr.h[2], i), hB);
            lB = dp4a_us(b[i], word_of(xr.l[2], i), lB);
            hB = dp4a_us(b[4 + i], word_of(xr.h[3], i), hB);
            lB = dp4a_us(b[4 + i], word_of(xr.l[3], i), lB);
        }
        const float fa = (float)((hA * 256 + lA) - 64 * xr.is[0]);
        const float fb = (float)((hB * 256 + lB) - 64 * xr.is[1]);
        return xr.sx[0] * (dA * fa) + xr.sx[1] * (dB * fb);
    }
};

template <> struct WRegs<QT_Q8_0> {
    uint4 q[4];
    float dA, dB;
    // `rec` = shared address of the 272-byte record, j = 64-weight group 0..3 (native blocks 2j, 2j+1)
    __device__ __forceinline__ void load(uint32_t rec, int j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = lds128(rec + 64 * j + 16 * c);
        const uint32_t dd = lds32(rec + 256 + 4 * j);
        dA = half_bits_to_float(dd);
        dB = half_bits_to_float(dd >> 16);
    }
    __device__ __forceinline__ float dot(const XRegs<QT_Q8_0> &xr) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_ss(word_of(q[0], i), word_of(xr.h[0], i), hA);
            lA = dp4a_ss(word_of(q[0], i), word_of(xr.l[0], i), lA);
            hA = dp4a_ss(word_of(q[1], i), word_of(xr.h[1], i), hA);
            lA = dp4a_ss(word_of(q[1], i), word_of(xr.l[1], i), lA);
            hB = dp4a_ss(word_of(q[2], i), word_of(xr.h[2], i), hB);
            lB = dp4a_ss(word_of(q[2], i), word_of(xr.l[2], i), lB);
            hB = dp4a_ss(word_of(q[3], i), word_of(xr.h[3], i), hB);
            lB = dp4a_ss(word_of(q[3], i), word_of(xr.l[3], i), lB);
        }
        return (dA * xr.sx[0]) * (float)(hA * 256 + lA) + (dB * xr.sx[1]) * (float)(hB * 256 + lB);
    }
};

template <> struct WRegs<QT_Q6_K> {
    uint32_t q[4][4];        // quadrant c (32-weight stride), word i: 6-bit values 0..63 as bytes
    float f[4];              // d * sub-block scale of quadrant c
    // `rec` = shared address of the 208-byte record, j = 2*half + position-half, d = superblock scale
    __device__ __forceinline__ void load(uint32_t rec, int j, float d) {
        const int h = j >> 1, ph = j & 1;
        const uint4 A = lds128(rec + 64 * h + 16 * ph);         // quadrants 0 | 2
        const uint4 B = lds128(rec + 64 * h + 32 + 16 * ph);    // quadrants 1 | 3
        const uint4 H = lds128(rec + 128 + 32 * h + 16 * ph);   // 2 bits x 4 quadrants
        const uint2 s8 = lds64(rec + 192 + 8 * h);              // 8 int8 scales
        // scales of sub-blocks 8h + 2c + ph, c = 0..3
        const uint32_t sw0 = ph ? (s8.x >> 8) : s8.x, sw1 = ph ? (s8.y >> 8) : s8.y;
        f[0] = d * (float)(int)(int8_t)(sw0 & 0xFF);
        f[1] = d * (float)(int)(int8_t)((sw0 >> 16) & 0xFF);
        f[2] = d * (float)(int)(int8_t)(sw1 & 0xFF);
        f[3] = d * (float)(int)(int8_t)((sw1 >> 16) & 0xFF);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t a = word_of(A, i), b = word_of(B, i), hh = word_of(H, i);
            q[0][i] = (a & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u);
            q[1][i] = (b & 0x0F0F0F0Fu) | ((hh << 2) & 0x30303030u);
            q[2][i] = ((a >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u);
            q[3][i] = ((b >> 4) & 0x0F0F0F0Fu) | ((hh >> 2) & 0x30303030u);
        }
    }
    __device__ __forceinline__ float dot(const XRegs<QT_Q6_K> &xr) const {
        float r = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            int ah = 0, al = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ah = dp4a_us(q[c][i], word_of(xr.h[c], i), ah);
                al = dp4a_us(q[c][i], word_of(xr.l[c], i), al);
            }
            r += (f[c] * xr.sx[c]) * (float)(ah * 256 + al - 32 * xr.is[c]);
        }
        return r;
    }
};

// ---------------------------------------------------------------------------------------------
// prologue: activation row -> fixed-point planes in shared memory
// ---------------------------------------------------------------------------------------------

constexpr float kXMax = 32512.f;   // 127 * 256: hi = (q + 128) >> 8 stays within a signed byte

// loads 8 consecutive activation elements starting at k0 (zeros beyond K)
__device__ __forceinline__ void load_x8(const XSrc &p, int m, int k0, float (&v)[8]) {
    if (k0 >= p.K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        return;
    }
    if (p.x_is_bf16) {
        const __nv_bfloat16 *xr = reinterpret_cast<const __nv_bfloat16 *>(p.x) + (long long)m * p.ldx + k0;
        if (p.x_vec_ok) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(xr);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(xr[i]);
        }
    } else {
        const float *xr = reinterpret_cast<const float *>(p.x) + (long long)m * p.ldx + k0;
        if (p.x_vec_ok) {
            const float4 a = *reinterpret_cast<const float4 *>(xr);
            const float4 b = *reinterpret_cast<const float4 *>(xr + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = xr[i];
        }
    }
}

template <int QT>
__device__ __forceinline__ void prep_store8(const float (&v)[8], int k0, uint8_t *xh, uint8_t *xl, float *sx,
                                            int *isum, int units16) {
    float amax = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
        bad |= !(fabsf(v[i]) <= 3.0e38f);   // inf or nan
    }
    // four consecutive lanes cover one 32-weight block
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const unsigned badm = __ballot_sync(0xFFFFFFFFu, bad);
    const unsigned grp = 0xFu << ((threadIdx.x & 31) & ~3);
    const bool blk_bad = (badm & grp) != 0;
    const float inv = (amax > 0.f && !blk_bad) ? kXMax / amax : 0.f;
    int q[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = blk_bad ? 0 : __float2int_rn(v[i] * inv);
        q[i] = max(-32512, min(32512, q[i]));
        sum += q[i];
    }
    uint32_t h0 = 0, h1 = 0, l0 = 0, l1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int ha = (q[i] + 128) >> 8, hb = (q[4 + i] + 128) >> 8;   // balanced digits
        h0 |= (uint32_t)(ha & 0xFF) << (8 * i);
        l0 |= (uint32_t)((q[i] - 256 * ha) & 0xFF) << (8 * i);
        h1 |= (uint32_t)(hb & 0xFF) << (8 * i);
        l1 |= (uint32_t)((q[4 + i] - 256 * hb) & 0xFF) << (8 * i);
    }
    const int off = xplane_off<QT>(k0, units16);
    *reinterpret_cast<uint2 *>(xh + off) = make_uint2(h0, h1);
    *reinterpret_cast<uint2 *>(xl + off) = make_uint2(l0, l1);
    const int sum16 = sum + __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if (QT == QT_Q6_K) {
        if ((threadIdx.x & 1) == 0) isum[k0 >> 4] = sum16;
    } else {
        const int sum32 = sum16 + __shfl_xor_sync(0xFFFFFFFFu, sum16, 2);
        if ((threadIdx.x & 3) == 0) isum[k0 >> 5] = sum32;
    }
    if ((threadIdx.x & 3) == 0)
        sx[k0 >> 5] = blk_bad ? __int_as_float(0x7FC00000) : amax * (1.0f / kXMax);
}

// Threads tid = 0 .. T-1 (whole warps) convert activation row m.  Loads are issued four deep before any is used so a
// long row costs one trip to L2, not one per 8 * T elements.
template <int QT, bool NORM = false>
__device__ __forceinline__ void prep_row(const XSrc &p, int m, int tid, int T, uint8_t *xh, uint8_t *xl,
                                         float *sx, int *isum, int units16) {
    constexpr int PB = 4;
    const int stride = T * 8;
    for (int base = tid * 8; base < p.Kpad; base += stride * PB) {
        float v[PB][8];
#pragma unroll
        for (int b = 0; b < PB; ++b)
            if (base + b * stride < p.Kpad) load_x8(p, m, base + b * stride, v[b]);
#pragma unroll
        for (int b = 0; b < PB; ++b)
            if (base + b * stride < p.Kpad) {
                if (NORM && p.gamma) norm_x8(p, base + b * stride, v[b]);
                prep_store8<QT>(v[b], base + b * stride, xh, xl, sx, isum, units16);
            }
    }
}

// The same conversion split in two, for a bf16 row of at most 4 * 8 * T elements: the global loads
// are issued early (while the previous job is still being reduced and stored) and the values wait
// in registers until the planes may be overwritten.
constexpr int kPrepBatch = 4;
struct XRaw {
    uint4 r[kPrepBatch];
};

__device__ __forceinline__ bool prep_can_prefetch(const XSrc &p, int T) {
    return p.x_is_bf16 && p.x_vec_ok && p.Kpad <= kPrepBatch * T * 8;
}

__device__ __forceinline__ void prep_prefetch(const XSrc &p, int tid, int T, XRaw &raw) {
    const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(p.x);
#pragma unroll
    for (int b = 0; b < kPrepBatch; ++b) {
        const int k0 = tid * 8 + b * T * 8;
        raw.r[b] = (k0 < p.K) ? *reinterpret_cast<const uint4 *>(x + k0) : make_uint4(0, 0, 0, 0);
    }
}

template <int QT>
__device__ __forceinline__ void prep_from_raw(const XSrc &p, int tid, int T, const XRaw &raw, uint8_t *xh, uint8_t *xl,
                                              float *sx, int *isum, int units16) {
#pragma unroll
    for (int b = 0; b < kPrepBatch; ++b) {
        const int k0 = tid * 8 + b * T * 8;
        if (k0 < p.Kpad) {   // warp-uniform: a warp covers 256 consecutive elements
            const uint32_t w[4] = {raw.r[b].x, raw.r[b].y, raw.r[b].z, raw.r[b].w};
            float v[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
            prep_store8<QT>(v, k0, xh, xl, sx, isum, units16);
        }
    }
}

// Sum R per-lane values over the 32 lanes with a folding butterfly (6 shuffles for R = 4, 5 for
// R = 2 instead of 5 per value).  The total of value r ends up in lane r * (32 / R).
template <int R> __device__ __forceinline__ float fold_rows(const float (&a)[R], int lane) {
    static_assert(R == 2 || R == 4, "R");
    float y;
    if (R == 4) {
        const bool up = lane & 16;
        float k0 = up ? a[2] : a[0], k1 = up ? a[3] : a[1];
        const float s0 = up ? a[0] : a[2], s1 = up ? a[1] : a[3];
        k0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 16);
        k1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 16);
        const bool up8 = lane & 8;
        y = (up8 ? k1 : k0) + __shfl_xor_sync(0xFFFFFFFFu, up8 ? k0 : k1, 8);
    } else {
        const bool up = lane & 16;
        y = (up ? a[1] : a[0]) + __shfl_xor_sync(0xFFFFFFFFu, up ? a[0] : a[1], 16);
        y += __shfl_xor_sync(0xFFFFFFFFu, y, 8);
    }
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 4);
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
    y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
    return y;
}


}  // namespace b200q
