// Decode GEMV (M = 1) and M <= 4 product: the HBM-bound streaming kernel.
//
// Y[m][n] = sum_k X[m][k] * dequant(W)[n][k]   for the streaming layout of common.cuh.
//
// Design (one persistent CTA per SM, no CPU fallback, no cluster multicast):
//   * CW consumer warps and one producer warp.  Every consumer warp owns a private ring of
//     shared-memory slots; lane w of the producer warp keeps consumer w's ring full with 1-D
//     bulk copies (cp.async.bulk, completion counted on a "full" mbarrier) and learns that a slot
//     was consumed from an "empty" mbarrier.  A work item is R rows x one chunk of 8 superblock
//     records (2048 weights per row); the rings keep CW * D items in flight per SM, so HBM reads
//     stay outstanding without spending registers on them.
//   * the activation is converted once per CTA into a 16-bit fixed-point form in shared memory:
//     per 32 weights one fp32 scale sx and per weight two signed bytes (x ~= sx * (256*hi + lo),
//     lo in [-128, 127]; relative step 2^-15 of the block maximum).  The packed 4/6/8-bit weights
//     multiply the two byte planes with dp4a, four weights per instruction, and block results are
//     scaled and accumulated in fp32.
//   * sub-block scales and mins are unpacked in registers; the min term of Q4_K and the -32
//     offset of Q6_K use per-block integer sums of the activation computed in the prologue.
//   * one lane handles one 64-weight unit of each of the item's R rows, so the activation bytes
//     it loads are reused R times; a row's partial sums live in the lanes of one warp and are
//     combined by warp shuffles.
//   * every mbarrier wait is bounded; on expiry the waiter raises the status word and leaves.
#include "common.cuh"
#include "kernels.h"

namespace b200q {

namespace {

constexpr int kMaxSeg = 4;
constexpr int kMaxWarps = 15;    // consumer warps (+1 producer = 512 threads, 128 registers each)
constexpr int kMaxDepth = 8;
constexpr int KC = 8;            // superblock records per chunk: 32 units of 64 weights, one per lane

template <int QT> struct GemvCfg;
template <> struct GemvCfg<QT_Q4_K> { static constexpr int CHUNK = KC * 144; };
template <> struct GemvCfg<QT_Q8_0> { static constexpr int CHUNK = KC * 272; };
template <> struct GemvCfg<QT_Q6_K> { static constexpr int CHUNK = 1680; };

struct GemvSeg {
    const uint8_t *w;   // streaming-layout rows
    void *y;            // output base (row m at y + m*ldy elements)
    long long ldy;
    int n;              // rows
    int row_begin;      // first virtual row of this segment (segments are concatenated)
};

struct GemvParams {
    GemvSeg seg[kMaxSeg];
    int nseg;
    int total_rows;
    const void *x;
    long long ldx;
    int x_is_bf16;
    int x_vec_ok;       // rows are 16-byte aligned: vector loads allowed
    int y_is_bf16;
    int M;
    int K, Kpad, nsb;
    long long row_bytes;
    int nchunks;
    unsigned bytes_full, bytes_tail;   // bytes of one row's chunk: all but the last / the last
    int partial_bytes;  // shared-memory bytes of the per-(row, chunk) partial sums
    int depth;          // ring slots per warp
    int debug;          // experiments only: 1 = stream without computing, 2 = compute without streaming
    int *status;
};

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

struct XView {            // shared-memory views of one activation row in fixed-point form
    const uint8_t *xh;    // signed high bytes
    const uint8_t *xl;    // signed low bytes
    const float *sx;      // per 32 weights
    const int *isum;      // sum of the 16-bit integers: per 32 weights (Q4_K) or per 16 (Q6_K)
};

struct XRegs {            // one 64-weight unit of one activation row: 4 groups of 16 weights
    uint4 h[4];
    uint4 l[4];
};

__device__ __forceinline__ void load_x(XRegs &xr, const XView &xv, int unit, int units16) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        xr.h[c] = *reinterpret_cast<const uint4 *>(xv.xh + c * units16 + unit * 16);
        xr.l[c] = *reinterpret_cast<const uint4 *>(xv.xl + c * units16 + unit * 16);
    }
}

// Weights of one 64-weight unit of one row, unpacked once and reused for every activation row.
template <int QT> struct WRegs;

template <> struct WRegs<QT_Q4_K> {
    uint32_t lo[8], hi[8];   // low nibbles = weights 0..31 of the group; hi keeps 16 * nibble
    int scA, mnA, scB, mnB;
    float d, dmin;
    // `rec` points at the 144-byte block, j = 64-weight group 0..3
    __device__ __forceinline__ void load(const uint8_t *rec, int j) {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(rec);
        const uint4 qa = *reinterpret_cast<const uint4 *>(rec + 16 + 32 * j);
        const uint4 qb = *reinterpret_cast<const uint4 *>(rec + 32 + 32 * j);
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
    // gu = global 64-weight unit index of the row
    __device__ __forceinline__ float dot(const XRegs &xr, const XView &xv, int gu) const {
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
        const float2 sx = *reinterpret_cast<const float2 *>(xv.sx + 2 * gu);
        const int2 is = *reinterpret_cast<const int2 *>(xv.isum + 2 * gu);
        const float fa = (float)((hA * 256 + lA) * scA);
        const float fb = (float)(((hB * 256 + lB) >> 4) * scB);   // hi held 16 * nibble: exact shift
        const float ua = (float)(mnA * is.x);
        const float ub = (float)(mnB * is.y);
        return sx.x * (d * fa - dmin * ua) + sx.y * (d * fb - dmin * ub);
    }
};

template <> struct WRegs<QT_Q8_0> {
    uint4 q[4];
    float dA, dB;
    // `rec` points at the 272-byte record, j = 64-weight group 0..3 (native blocks 2j, 2j+1)
    __device__ __forceinline__ void load(const uint8_t *rec, int j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = *reinterpret_cast<const uint4 *>(rec + 64 * j + 16 * c);
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(rec + 256 + 4 * j);
        dA = half_bits_to_float(dd);
        dB = half_bits_to_float(dd >> 16);
    }
    __device__ __forceinline__ float dot(const XRegs &xr, const XView &xv, int gu) const {
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
        const float2 sx = *reinterpret_cast<const float2 *>(xv.sx + 2 * gu);
        return (dA * sx.x) * (float)(hA * 256 + lA) + (dB * sx.y) * (float)(hB * 256 + lB);
    }
};

template <> struct WRegs<QT_Q6_K> {
    uint32_t q[4][4];        // quadrant c (32-weight stride), word i: 6-bit values 0..63 as bytes
    float f[4];              // d * sub-block scale of quadrant c
    int h, ph;
    // `rec` points at the 208-byte record, j = 2*half + position-half, d = superblock scale
    __device__ __forceinline__ void load(const uint8_t *rec, int j, float d) {
        h = j >> 1;
        ph = j & 1;
        const uint4 A = *reinterpret_cast<const uint4 *>(rec + 64 * h + 16 * ph);        // quadrants 0 | 2
        const uint4 B = *reinterpret_cast<const uint4 *>(rec + 64 * h + 32 + 16 * ph);   // quadrants 1 | 3
        const uint4 H = *reinterpret_cast<const uint4 *>(rec + 128 + 32 * h + 16 * ph);  // 2 bits x 4 quadrants
        const uint2 s8 = *reinterpret_cast<const uint2 *>(rec + 192 + 8 * h);            // 8 int8 scales
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
    // sb = global superblock index of the row
    __device__ __forceinline__ float dot(const XRegs &xr, const XView &xv, int sb) const {
        int ah[4] = {0, 0, 0, 0}, al[4] = {0, 0, 0, 0};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ah[c] = dp4a_us(q[c][i], word_of(xr.h[c], i), ah[c]);
                al[c] = dp4a_us(q[c][i], word_of(xr.l[c], i), al[c]);
            }
        }
        // 32-weight scale blocks 8*sb + 4h + c ; 16-weight sums 16*sb + 8h + 2c + ph
        const float4 sx = *reinterpret_cast<const float4 *>(xv.sx + 8 * sb + 4 * h);
        const int4 i0 = *reinterpret_cast<const int4 *>(xv.isum + 16 * sb + 8 * h);
        const int4 i1 = *reinterpret_cast<const int4 *>(xv.isum + 16 * sb + 8 * h + 4);
        const int s0 = ph ? i0.y : i0.x, s1 = ph ? i0.w : i0.z;
        const int s2 = ph ? i1.y : i1.x, s3 = ph ? i1.w : i1.z;
        const float v0 = (float)(ah[0] * 256 + al[0] - 32 * s0);
        const float v1 = (float)(ah[1] * 256 + al[1] - 32 * s1);
        const float v2 = (float)(ah[2] * 256 + al[2] - 32 * s2);
        const float v3 = (float)(ah[3] * 256 + al[3] - 32 * s3);
        return (f[0] * sx.x) * v0 + (f[1] * sx.y) * v1 + (f[2] * sx.z) * v2 + (f[3] * sx.w) * v3;
    }
};

// ---------------------------------------------------------------------------------------------
// prologue: activation row -> fixed-point planes in shared memory
// ---------------------------------------------------------------------------------------------

constexpr float kXMax = 32512.f;   // 127 * 256: hi = (q + 128) >> 8 stays within a signed byte

// loads 8 consecutive activation elements starting at k0 (zeros beyond K)
__device__ __forceinline__ void load_x8(const GemvParams &p, int m, int k0, float (&v)[8]) {
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

// Threads [0, T) convert activation row m.  Loads are issued four deep before any is used so a
// long row costs one trip to L2, not one per 8 * T elements.
template <int QT>
__device__ __forceinline__ void prep_row(const GemvParams &p, int m, int T, uint8_t *xh, uint8_t *xl,
                                         float *sx, int *isum, int units16) {
    constexpr int PB = 4;
    const int stride = T * 8;
    for (int base = threadIdx.x * 8; base < p.Kpad; base += stride * PB) {
        float v[PB][8];
#pragma unroll
        for (int b = 0; b < PB; ++b)
            if (base + b * stride < p.Kpad) load_x8(p, m, base + b * stride, v[b]);
#pragma unroll
        for (int b = 0; b < PB; ++b)
            if (base + b * stride < p.Kpad) prep_store8<QT>(v[b], base + b * stride, xh, xl, sx, isum, units16);
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

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------

// (segment, row inside it) of virtual row vr; segments are concatenated in launch order
__device__ __forceinline__ void locate_row(const GemvParams &p, int vr, int &s, int &row) {
    s = 0;
#pragma unroll
    for (int i = 1; i < kMaxSeg; ++i)
        if (i < p.nseg && vr >= p.seg[i].row_begin) s = i;
    row = vr - p.seg[s].row_begin;
}

// M = 1 runs with 8 consumer warps + 1 producer and at most half an SM's registers and shared
// memory, so two CTAs fit on an SM: under programmatic dependent launch the next projection's CTA
// moves in beside this one and streams its weights while this one still computes.
template <int MT> struct GemvShape {
    static constexpr int kWarps = MT == 1 ? 8 : kMaxWarps;       // default consumer warps
    static constexpr int kThreads = (kWarps + 1) * 32;
    static constexpr int kBlocksPerSm = MT == 1 ? 2 : 1;
};

template <int QT, int MT, int R>
__global__ void __launch_bounds__(GemvShape<MT>::kThreads, GemvShape<MT>::kBlocksPerSm) gemv_kernel(const GemvParams p) {
    using Cfg = GemvCfg<QT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CW = (blockDim.x >> 5) - 1;     // consumer warps; warp CW is the producer
    const int D = p.depth;

    // shared-memory carve-up: full[CW][D], empty[CW][D], activation planes, partial sums, rings
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + kMaxWarps * kMaxDepth * 8;
    uint8_t *xbase = smem + 2 * kMaxWarps * kMaxDepth * 8;
    const int units16 = (p.Kpad >> 6) * 16;
    const int plane = p.Kpad;
    const int n_isum = (QT == QT_Q6_K) ? (p.Kpad >> 4) : (p.Kpad >> 5);
    const int per_m = 2 * plane + (p.Kpad >> 5) * 4 + n_isum * 4;        // xh, xl, sx, isum
    float *partial = reinterpret_cast<float *>(xbase + ((MT * per_m + 127) & ~127));   // [row][chunk][MT]
    uint8_t *rings = reinterpret_cast<uint8_t *>(partial) + p.partial_bytes;
    const int ring_bytes = D * R * Cfg::CHUNK;

    // this CTA's contiguous range of virtual rows, cut into groups of R rows; a work item is one
    // group x one K-chunk, dealt round-robin to the consumer warps
    const int vb = (int)((long long)p.total_rows * blockIdx.x / gridDim.x);
    const int ve = (int)((long long)p.total_rows * (blockIdx.x + 1) / gridDim.x);
    const int n_groups = (ve - vb + R - 1) / R;
    const int n_items = n_groups * p.nchunks;

    if (threadIdx.x < CW) {
        for (int i = 0; i < D; ++i) {
            mbar_init(full0 + (threadIdx.x * kMaxDepth + i) * 8, 1);
            mbar_init(empty0 + (threadIdx.x * kMaxDepth + i) * 8, 1);
        }
        mbar_fence_init();
        fence_proxy_async();
    }
    // let the next kernel in the stream start: it only prefetches its own weights until this
    // grid has finished (see pdl_wait below)
    pdl_launch_dependents();
    __syncthreads();

    // =========================================================================================
    // producer warp: lane w feeds consumer warp w.  All lanes poll together (no lane blocks the
    // others): a lane issues its next item as soon as its consumer has released the slot.
    // =========================================================================================
    if (warp == CW) {
        const unsigned mask = __activemask();
        const bool feeder = lane < CW;
        const uint32_t ring_s = smem_u32(rings + lane * ring_bytes);
        const uint32_t fbar = full0 + lane * kMaxDepth * 8, ebar = empty0 + lane * kMaxDepth * 8;
        int item = (feeder && !(p.debug & 2)) ? lane : n_items;
        int g = 0, c = lane;           // item = g * nchunks + c, kept without dividing
        while (c >= p.nchunks) { c -= p.nchunks; ++g; }
        int slot = 0, k = 0;
        uint32_t phase = 0;            // parity of the release this slot's next reuse waits for
        uint64_t t_first = 0;
        bool timing = false;
        int idle = 0;
#pragma unroll 1
        while (true) {
            bool progressed = false;
            if (item < n_items) {
                const bool free_slot = (k < D) || mbar_try_wait(ebar + 8 * slot, phase ^ 1u);
                if (free_slot) {
                    const int vr0 = vb + g * R, nr = min(R, ve - vr0);
                    const int sb0 = c * KC;
                    const uint32_t bytes = (c == p.nchunks - 1) ? p.bytes_tail : p.bytes_full;
                    const uint32_t bar = fbar + 8 * slot;
                    const long long coff = rec_off(QT, sb0);
                    fence_proxy_async();   // the consumer's reads of this slot precede the engine's writes
                    mbar_expect_tx(bar, bytes * nr);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (r < nr) {
                            int s, row;
                            locate_row(p, vr0 + r, s, row);
                            bulk_g2s(ring_s + (slot * R + r) * Cfg::CHUNK,
                                     p.seg[s].w + (long long)row * p.row_bytes + coff, bytes, bar);
                        }
                    }
                    item += CW;
                    c += CW;
                    while (c >= p.nchunks) { c -= p.nchunks; ++g; }
                    ++k;
                    if (++slot == D) { slot = 0; phase ^= 1u; }
                    progressed = true;
                }
            }
            if (__all_sync(mask, item >= n_items)) break;
            if (__any_sync(mask, progressed)) {
                idle = 0;
                timing = false;
            } else if (++idle >= 1024) {   // nobody moved for a while: look at the clock
                idle = 0;
                const uint64_t now = globaltimer_ns();
                if (!timing) {
                    timing = true;
                    t_first = now;
                } else if (now - t_first > kWaitLimitNs) {
                    if (lane == 0) atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                    break;
                }
            }
        }
        return;
    }

    // =========================================================================================
    // consumer warps
    // =========================================================================================
    // everything below reads the activation or writes the output: the previous grid must be done
    pdl_wait();
    XView xv[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        uint8_t *b = xbase + m * per_m;
        xv[m].xh = b;
        xv[m].xl = b + plane;
        xv[m].sx = reinterpret_cast<const float *>(b + 2 * plane);
        xv[m].isum = reinterpret_cast<const int *>(b + 2 * plane + (p.Kpad >> 5) * 4);
        if (m < p.M && !(p.debug & 4))
            prep_row<QT>(p, m, CW * 32, b, b + plane, reinterpret_cast<float *>(b + 2 * plane),
                         reinterpret_cast<int *>(b + 2 * plane + (p.Kpad >> 5) * 4), units16);
    }
    // consumers only: the producer warp must not be held here, it is already feeding the rings
    asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");

    const uint8_t *ring = rings + warp * ring_bytes;
    const uint32_t fbar = full0 + warp * kMaxDepth * 8, ebar = empty0 + warp * kMaxDepth * 8;
    const int lsb = lane >> 2, j = lane & 3;   // this lane's record and 64-weight group in a chunk

    int slot = 0;
    uint32_t phase = 0;
    bool failed = false;
    int item = warp;
    int g = 0, c = warp;               // item = g * nchunks + c, kept without dividing
    while (c >= p.nchunks) { c -= p.nchunks; ++g; }

    // The cross-lane sum of an item's results is taken one iteration late, after the next item's
    // shared-memory loads have been issued, so its shuffle chain hides behind them.
    float pend[R][MT];
    int pend_cell = -1, pend_nr = 0;   // first partial-sum cell of the pending item
    auto flush_pending = [&]() {
        if (pend_cell < 0) return;
        if constexpr (MT == 1) {
            float a[R];
#pragma unroll
            for (int r = 0; r < R; ++r) a[r] = pend[r][0];
            const float v = fold_rows<R>(a, lane);
            const int r = lane / (32 / R);
            if ((lane & (32 / R - 1)) == 0 && r < pend_nr) partial[pend_cell + r * p.nchunks] = v;
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float v = pend[r][m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                    if (lane == 0 && r < pend_nr) partial[(pend_cell + r * p.nchunks) * MT + m] = v;
                }
            }
        }
        pend_cell = -1;
    };

#pragma unroll 1
    for (; item < n_items; item += CW) {
        bool ok = (p.debug & 2) ? true : mbar_wait_bounded(fbar + 8 * slot, phase);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) { failed = true; break; }

        const int nr = min(R, ve - vb - g * R);
        const int sb0 = c * KC;
        const int gsb = sb0 + lsb;
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

        // the pending sum uses full-warp shuffles, so it may sit inside the branch below only when
        // every lane takes that branch (a chunk of 8 whole records)
        const bool whole = (sb0 + KC <= p.nsb) && !(p.debug & 1);
        if (!whole) flush_pending();
        if (gsb < p.nsb && !(p.debug & 1)) {
            const int gu = gsb * 4 + j;
            const uint8_t *sl = ring + (slot * R) * Cfg::CHUNK;
            auto load_w = [&](WRegs<QT> &w, int r) {
                const uint8_t *row = sl + r * Cfg::CHUNK;
                if constexpr (QT == QT_Q4_K) {
                    w.load(row + lsb * 144, j);
                } else if constexpr (QT == QT_Q8_0) {
                    w.load(row + lsb * 272, j);
                } else {
                    const int doff = (int)(q6k_d_off(gsb, p.nsb) - rec_off(QT, sb0));
                    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + doff));
                    w.load(row + lsb * 208, j, d);
                }
            };
            if constexpr (MT == 1) {
                // one activation row: keep its bytes in registers, stream the R weight rows past them
                XRegs xr;
                load_x(xr, xv[0], gu, units16);
                if (whole) flush_pending();
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r < nr) {
                        WRegs<QT> w;
                        load_w(w, r);
                        acc[r][0] += w.dot(xr, xv[0], QT == QT_Q6_K ? gsb : gu);
                    }
                }
            } else {
                // several activation rows: unpack the weights once, stream the activations past them
                WRegs<QT> wr[R];
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r < nr) load_w(wr[r], r);
                if (whole) flush_pending();
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    XRegs xr;
                    load_x(xr, xv[m], gu, units16);
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        if (r < nr) acc[r][m] += wr[r].dot(xr, xv[m], QT == QT_Q6_K ? gsb : gu);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ebar + 8 * slot);   // slot may be refilled
        if (++slot == D) { slot = 0; phase ^= 1u; }

        // one shared-memory cell per (row, chunk, m): the final sum over chunks runs in a fixed
        // order whatever warp produced which cell
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) pend[r][m] = acc[r][m];
        pend_cell = (g * R) * p.nchunks + c;
        pend_nr = nr;
        c += CW;
        while (c >= p.nchunks) { c -= p.nchunks; ++g; }
    }
    flush_pending();

    if (failed) {
        if (lane == 0) atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
        // copies already issued for this warp must land before the CTA's shared memory is
        // released: wait for each slot that can still be in flight once more, again with a limit
        for (int i = 0; i < D && item < n_items; ++i, item += CW) {
            (void)mbar_wait_bounded(fbar + 8 * slot, phase);
            if (++slot == D) { slot = 0; phase ^= 1u; }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");

    // final pass: sum the chunks of every row of this CTA in order and store
    const int rows_here = (p.debug & 8) ? 0 : ve - vb;
    for (int t = threadIdx.x; t < rows_here * MT; t += CW * 32) {
        const int rl = t / MT, m = t - rl * MT;
        float v = 0.f;
        for (int c = 0; c < p.nchunks; ++c) v += partial[(rl * p.nchunks + c) * MT + m];
        if (m < p.M) {
            int s, row;
            locate_row(p, vb + rl, s, row);
            const long long idx = (long long)m * p.seg[s].ldy + row;
            if (p.y_is_bf16)
                reinterpret_cast<__nv_bfloat16 *>(p.seg[s].y)[idx] = __float2bfloat16_rn(v);
            else
                reinterpret_cast<float *>(p.seg[s].y)[idx] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

template <int QT, int MT, int R>
cudaError_t launch_t(const GemvLaunch &a, GemvParams &p, int grid, cudaStream_t st) {
    using Shape = GemvShape<MT>;
    constexpr int chunk = GemvCfg<QT>::CHUNK;
    int warps = a.warps > 0 ? a.warps : Shape::kWarps;
    if (warps > Shape::kWarps) warps = Shape::kWarps;
    const size_t n_isum = QT == QT_Q6_K ? p.Kpad / 16 : p.Kpad / 32;
    const size_t per_m = 2 * (size_t)p.Kpad + (p.Kpad / 32) * 4 + n_isum * 4;
    const int rows_cta = (p.total_rows + grid - 1) / grid;
    const int groups = (rows_cta + R - 1) / R;
    p.partial_bytes = (int)((((size_t)groups * R * p.nchunks * MT * 4) + 127) & ~size_t(127));
    const size_t fixed = 2 * kMaxWarps * kMaxDepth * 8 + ((MT * per_m + 127) & ~size_t(127)) + p.partial_bytes;
    // two CTAs per SM when the shape allows it (each may use half of the SM's shared memory
    // minus the per-block reservation), otherwise the whole SM
    size_t budget = a.smem_limit;
    const size_t half = (a.smem_sm - 2 * 1024) / 2;
    if (Shape::kBlocksPerSm == 2 && half < budget && fixed + (size_t)warps * 2 * R * chunk <= half) budget = half;
    if (fixed + (size_t)warps * 2 * R * chunk > budget) return cudaErrorInvalidValue;
    int depth = (int)((budget - fixed) / ((size_t)warps * R * chunk));
    if (depth > kMaxDepth) depth = kMaxDepth;
    if (a.depth > 0 && a.depth < depth) depth = a.depth;
    p.depth = depth;
    const size_t smem = fixed + (size_t)warps * depth * R * chunk;

    auto kern = gemv_kernel<QT, MT, R>;
    static size_t configured = 0;   // per instantiation; a context on another device re-sets it
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured || dev != configured_dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)((warps + 1) * 32));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int QT, int R>
cudaError_t launch_q(const GemvLaunch &a, GemvParams &p, int grid, cudaStream_t st) {
    switch (a.M) {
    case 1: return launch_t<QT, 1, R>(a, p, grid, st);
    case 2: return launch_t<QT, 2, 2>(a, p, grid, st);
    case 3: return launch_t<QT, 3, 2>(a, p, grid, st);
    default: return launch_t<QT, 4, 2>(a, p, grid, st);
    }
}

template <int R> cudaError_t launch_r(const GemvLaunch &a, GemvParams &p, int grid, cudaStream_t st) {
    switch (a.qt) {
    case QT_Q4_K: return launch_q<QT_Q4_K, R>(a, p, grid, st);
    case QT_Q8_0: return launch_q<QT_Q8_0, R>(a, p, grid, st);
    default: return launch_q<QT_Q6_K, R>(a, p, grid, st);
    }
}

}  // namespace

int gemv_max_m() { return 4; }

// Returns cudaSuccess, or cudaErrorInvalidValue when the shape cannot be staged in shared memory
// (caller then picks another route).
cudaError_t gemv_launch(const GemvLaunch &a, cudaStream_t st) {
    GemvParams p{};
    if (a.nseg < 1 || a.nseg > kMaxSeg || a.M < 1 || a.M > 4) return cudaErrorInvalidValue;
    if (a.qt != QT_Q4_K && a.qt != QT_Q8_0 && a.qt != QT_Q6_K) return cudaErrorInvalidValue;
    int rows = 0;
    for (int i = 0; i < a.nseg; ++i) {
        p.seg[i].w = a.w[i];
        p.seg[i].y = a.y[i];
        p.seg[i].ldy = a.ldy[i];
        p.seg[i].n = a.n[i];
        p.seg[i].row_begin = rows;
        rows += a.n[i];
    }
    p.nseg = a.nseg;
    p.total_rows = rows;
    p.x = a.x;
    p.ldx = a.ldx;
    p.x_is_bf16 = a.x_is_bf16;
    const size_t xelt = a.x_is_bf16 ? 2 : 4;
    p.x_vec_ok = ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) && ((a.ldx * xelt) % 16 == 0);
    p.y_is_bf16 = a.y_is_bf16;
    p.M = a.M;
    p.K = a.K;
    p.Kpad = a.Kpad;
    p.nsb = a.Kpad / SB;
    p.row_bytes = a.row_bytes;
    p.status = a.status;
    p.debug = a.debug;
    p.nchunks = (p.nsb + KC - 1) / KC;
    p.bytes_full = (unsigned)range_bytes(a.qt, 0, p.nsb < KC ? p.nsb : KC, p.nsb);
    p.bytes_tail = (unsigned)range_bytes(a.qt, (p.nchunks - 1) * KC, p.nsb, p.nsb);
    const int grid = a.grid > 0 ? a.grid : a.sm_count;
    // four rows per item when a CTA owns many rows (fewer, larger items) and M = 1; two otherwise
    const int rows_cta = (rows + grid - 1) / grid;
    const int rpi = a.rows_per_item > 0 ? a.rows_per_item : (rows_cta >= 64 ? 4 : 2);
    if (rpi == 4 && a.M == 1) return launch_r<4>(a, p, grid, st);
    return launch_r<2>(a, p, grid, st);
}

}  // namespace b200q
