// Decode GEMV (M = 1) and M <= 4 product: the HBM-bound streaming kernel.
//
// Y[m][n] = sum_k X[m][k] * dequant(W)[n][k]   for the streaming layout of common.cuh.
//
// Design (one persistent CTA per SM, no CPU fallback, no cluster multicast):
//   * every warp owns a private ring of shared-memory slots and streams its own rows into it
//     with 1-D bulk copies (cp.async.bulk, completion counted on an mbarrier).  A work item is
//     R rows x one K-chunk of KC superblock records; the ring keeps D items in flight per warp,
//     so an SM holds CW * D * R * ~2.3 KB of HBM reads in flight without spending registers.
//   * the activation is converted once per CTA into a 16-bit fixed-point form in shared memory:
//     per 32 weights one fp32 scale sx and per weight a signed high byte and an unsigned low
//     byte (x ~= sx * (256*hi + lo), relative step 2^-15 of the block maximum).  The packed
//     4/6/8-bit weights then multiply the two byte planes with dp4a, four weights per
//     instruction, and block results are scaled and accumulated in fp32.
//   * sub-block scales and mins are unpacked in registers; the min term of Q4_K and the -32
//     offset of Q6_K use per-16-weight integer sums of the activation computed in the prologue.
//   * a row's partial sums live in the lanes of one warp and are combined by warp shuffles.
//   * every mbarrier wait is bounded; on expiry the warp raises the status word and leaves.
#include "common.cuh"
#include "kernels.h"

namespace b200q {

namespace {

constexpr int kMaxSeg = 4;
constexpr int kMaxWarps = 16;
constexpr int kMaxDepth = 8;

template <int QT> struct GemvCfg;
template <> struct GemvCfg<QT_Q4_K> { static constexpr int KC = 16; static constexpr int CHUNK = 16 * 144; };
template <> struct GemvCfg<QT_Q8_0> { static constexpr int KC = 8;  static constexpr int CHUNK = 8 * 272; };
template <> struct GemvCfg<QT_Q6_K> { static constexpr int KC = 16; static constexpr int CHUNK = 2 * 1680; };

struct GemvSeg {
    const uint8_t *w;   // streaming-layout rows
    void *y;            // output base (row m at y + m*ldy elements)
    long long ldy;
    int n;              // rows
    int unit_begin;     // first unit (R rows each) of this segment in the global unit list
};

struct GemvParams {
    GemvSeg seg[kMaxSeg];
    int nseg;
    int total_units;
    const void *x;
    long long ldx;
    int x_is_bf16;
    int x_vec_ok;       // rows are 16-byte aligned: vector loads allowed
    int y_is_bf16;
    int M;
    int K, Kpad, nsb;
    long long row_bytes;
    int nchunks;
    int depth;          // ring slots per warp
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
    const uint8_t *xl;    // unsigned low bytes
    const float *sx;      // per 32 weights
    const int *isum;      // per 16 weights: sum of the 16-bit integers
};

// ---------------------------------------------------------------------------------------------
// per-type work on one 64-weight unit of one row, for MT activation rows
// ---------------------------------------------------------------------------------------------

struct XRegs {          // one 64-weight unit of one activation row: 4 groups of 16 weights
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

// Weights of one 64-weight unit of one row, unpacked to bytes once and reused for every
// activation row.
template <int QT> struct WRegs;

template <> struct WRegs<QT_Q4_K> {
    uint32_t lo[8], hi[8];   // low nibbles = weights 0..31 of the group, high nibbles = 32..63
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
            hi[i] = (a >> 4) & 0x0F0F0F0Fu;
            lo[4 + i] = b & 0x0F0F0F0Fu;
            hi[4 + i] = (b >> 4) & 0x0F0F0F0Fu;
        }
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, scA, mnA);
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, scB, mnB);
        d = half_bits_to_float(hdr.x);
        dmin = half_bits_to_float(hdr.x >> 16);
    }
    // gu = global 64-weight unit index of the row
    __device__ __forceinline__ float dot(const XRegs &xr, const XView &xv, int gu) const {
        int hA = 0, lA = 0, hB = 0, lB = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hA = dp4a_us(lo[i], word_of(xr.h[0], i), hA);
            lA = dp4a_uu(lo[i], word_of(xr.l[0], i), lA);
            hA = dp4a_us(lo[4 + i], word_of(xr.h[1], i), hA);
            lA = dp4a_uu(lo[4 + i], word_of(xr.l[1], i), lA);
            hB = dp4a_us(hi[i], word_of(xr.h[2], i), hB);
            lB = dp4a_uu(hi[i], word_of(xr.l[2], i), lB);
            hB = dp4a_us(hi[4 + i], word_of(xr.h[3], i), hB);
            lB = dp4a_uu(hi[4 + i], word_of(xr.l[3], i), lB);
        }
        const float2 sx = *reinterpret_cast<const float2 *>(xv.sx + 2 * gu);
        const int4 is = *reinterpret_cast<const int4 *>(xv.isum + 4 * gu);
        const float fa = (float)((hA * 256 + lA) * scA);
        const float fb = (float)((hB * 256 + lB) * scB);
        const float ua = (float)(mnA * (is.x + is.y));
        const float ub = (float)(mnB * (is.z + is.w));
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
            lA = dp4a_su(word_of(q[0], i), word_of(xr.l[0], i), lA);
            hA = dp4a_ss(word_of(q[1], i), word_of(xr.h[1], i), hA);
            lA = dp4a_su(word_of(q[1], i), word_of(xr.l[1], i), lA);
            hB = dp4a_ss(word_of(q[2], i), word_of(xr.h[2], i), hB);
            lB = dp4a_su(word_of(q[2], i), word_of(xr.l[2], i), lB);
            hB = dp4a_ss(word_of(q[3], i), word_of(xr.h[3], i), hB);
            lB = dp4a_su(word_of(q[3], i), word_of(xr.l[3], i), lB);
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
                al[c] = dp4a_uu(q[c][i], word_of(xr.l[c], i), al[c]);
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

template <int QT>
__device__ __forceinline__ void prep_row(const GemvParams &p, int m, uint8_t *xh, uint8_t *xl,
                                         float *sx, int *isum, int units16) {
    const int T = blockDim.x;
    for (int k0 = threadIdx.x * 8; k0 < p.Kpad; k0 += T * 8) {
        float v[8];
        if (k0 < p.K) {
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
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
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
        unsigned badm = __ballot_sync(0xFFFFFFFFu, bad);
        const unsigned grp = 0xFu << ((threadIdx.x & 31) & ~3);
        const bool blk_bad = (badm & grp) != 0;
        const float inv = (amax > 0.f && !blk_bad) ? 32767.f / amax : 0.f;
        int q[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            q[i] = blk_bad ? 0 : __float2int_rn(v[i] * inv);
            q[i] = max(-32767, min(32767, q[i]));
            sum += q[i];
        }
        uint32_t h0 = 0, h1 = 0, l0 = 0, l1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            h0 |= (uint32_t)((q[i] >> 8) & 0xFF) << (8 * i);
            l0 |= (uint32_t)(q[i] & 0xFF) << (8 * i);
            h1 |= (uint32_t)((q[4 + i] >> 8) & 0xFF) << (8 * i);
            l1 |= (uint32_t)(q[4 + i] & 0xFF) << (8 * i);
        }
        const int off = xplane_off<QT>(k0, units16);
        *reinterpret_cast<uint2 *>(xh + off) = make_uint2(h0, h1);
        *reinterpret_cast<uint2 *>(xl + off) = make_uint2(l0, l1);
        const int sum16 = sum + __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        if ((threadIdx.x & 1) == 0) isum[k0 >> 4] = sum16;
        if ((threadIdx.x & 3) == 0)
            sx[k0 >> 5] = blk_bad ? __int_as_float(0x7FC00000) : amax * (1.0f / 32767.f);
    }
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------

template <int QT, int MT, int R>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) gemv_kernel(const GemvParams p) {
    using Cfg = GemvCfg<QT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CW = blockDim.x >> 5;
    const int D = p.depth;

    // shared-memory carve-up
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);                 // [CW][kMaxDepth]
    uint8_t *xbase = smem + kMaxWarps * kMaxDepth * 8;
    const int units = p.Kpad >> 6, units16 = units * 16;
    const int plane = p.Kpad;                                            // bytes per byte plane
    const int per_m = 2 * plane + (p.Kpad >> 5) * 4 + (p.Kpad >> 4) * 4;  // xh, xl, sx, isum
    uint8_t *ring = xbase + ((MT * per_m + 127) & ~127) + warp * (D * R * Cfg::CHUNK);
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t bar_s = smem_u32(bars + warp * kMaxDepth);

    // this warp's contiguous range of units (R rows each); consecutive virtual warp ids sit on
    // different SMs so a small N still spreads over the whole GPU
    const int vw = warp * gridDim.x + blockIdx.x, TW = CW * gridDim.x;
    const int u_begin = (int)((long long)p.total_units * vw / TW);
    const int u_end = (int)((long long)p.total_units * (vw + 1) / TW);
    const int n_items = (u_end - u_begin) * p.nchunks;

    if (lane == 0) {
        for (int i = 0; i < D; ++i) mbar_init(bar_s + 8 * i, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncwarp();

    // locate (segment, first row, row count) of unit u
    auto unit_rows = [&](int u, int &s, int &r0, int &nr) {
        s = 0;
#pragma unroll
        for (int i = 1; i < kMaxSeg; ++i)
            if (i < p.nseg && u >= p.seg[i].unit_begin) s = i;
        r0 = (u - p.seg[s].unit_begin) * R;
        nr = min(R, p.seg[s].n - r0);
    };
    auto issue = [&](int it) {   // lane 0 only
        const int u = u_begin + it / p.nchunks, c = it % p.nchunks;
        int s, r0, nr;
        unit_rows(u, s, r0, nr);
        const int sb0 = c * Cfg::KC, sb1 = min(p.nsb, sb0 + Cfg::KC);
        const uint32_t bytes = (uint32_t)range_bytes(QT, sb0, sb1, p.nsb);
        const int slot = it % D;
        const uint32_t bar = bar_s + 8 * slot;
        mbar_expect_tx(bar, bytes * nr);
        const uint8_t *src = p.seg[s].w + (long long)r0 * p.row_bytes + rec_off(QT, sb0);
        for (int r = 0; r < nr; ++r)
            bulk_g2s(ring_s + (slot * R + r) * Cfg::CHUNK, src + (long long)r * p.row_bytes, bytes, bar);
    };

    // start streaming weights before touching the activation
    const int pre = min(D, n_items);
    if (lane == 0)
        for (int it = 0; it < pre; ++it) issue(it);

    // prologue: activation rows -> fixed point
    XView xv[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        uint8_t *b = xbase + m * per_m;
        xv[m].xh = b;
        xv[m].xl = b + plane;
        xv[m].sx = reinterpret_cast<const float *>(b + 2 * plane);
        xv[m].isum = reinterpret_cast<const int *>(b + 2 * plane + (p.Kpad >> 5) * 4);
        if (m < p.M)
            prep_row<QT>(p, m, b, b + plane, reinterpret_cast<float *>(b + 2 * plane),
                         reinterpret_cast<int *>(b + 2 * plane + (p.Kpad >> 5) * 4), units16);
    }
    __syncthreads();

    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

    bool failed = false;
    int it = 0;
#pragma unroll 1
    for (; it < n_items; ++it) {
        const int slot = it % D;
        const uint32_t parity = (uint32_t)(it / D) & 1u;
        bool ok = mbar_wait_bounded(bar_s + 8 * slot, parity);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) { failed = true; break; }

        const int u = u_begin + it / p.nchunks, c = it % p.nchunks;
        int s, r0, nr;
        unit_rows(u, s, r0, nr);
        const int sb0 = c * Cfg::KC;
        const int nsb_c = min(p.nsb, sb0 + Cfg::KC) - sb0;
        const uint8_t *sl = ring + (slot * R) * Cfg::CHUNK;

#pragma unroll 1
        for (int lu = lane; lu < nsb_c * 4; lu += 32) {
            const int lsb = lu >> 2, j = lu & 3;
            const int gsb = sb0 + lsb;
            const int gu = gsb * 4 + j;
            WRegs<QT> wr[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (r < nr) {
                    const uint8_t *row = sl + r * Cfg::CHUNK;
                    if constexpr (QT == QT_Q4_K) {
                        wr[r].load(row + lsb * 144, j);
                    } else if constexpr (QT == QT_Q8_0) {
                        wr[r].load(row + lsb * 272, j);
                    } else {
                        const int doff = (int)(q6k_d_off(gsb, p.nsb) - rec_off(QT, sb0));
                        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(row + doff));
                        wr[r].load(row + (int)(rec_off(QT, gsb) - rec_off(QT, sb0)), j, d);
                    }
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                XRegs xr;
                load_x(xr, xv[m], gu, units16);
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r < nr) acc[r][m] += wr[r].dot(xr, xv[m], QT == QT_Q6_K ? gsb : gu);
            }
        }
        __syncwarp();
        if (lane == 0 && it + D < n_items) {
            fence_proxy_async();   // order this warp's generic reads before the engine's writes
            issue(it + D);
        }

        if (c == p.nchunks - 1) {   // unit finished: reduce over lanes and store
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float v = acc[r][m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                    acc[r][m] = 0.f;
                    if (lane == 0 && r < nr && m < p.M) {
                        const long long idx = (long long)m * p.seg[s].ldy + r0 + r;
                        if (p.y_is_bf16)
                            reinterpret_cast<__nv_bfloat16 *>(p.seg[s].y)[idx] = __float2bfloat16_rn(v);
                        else
                            reinterpret_cast<float *>(p.seg[s].y)[idx] = v;
                    }
                }
            }
        }
    }

    if (failed) {
        if (lane == 0) atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
        // copies already issued must land before this CTA's shared memory is released:
        // wait for each outstanding slot once more, again with a limit
        const int last = min(n_items, it + D);
        for (int j2 = it; j2 < last; ++j2)
            (void)mbar_wait_bounded(bar_s + 8 * (j2 % D), (uint32_t)(j2 / D) & 1u);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

template <int QT, int MT, int R>
cudaError_t launch_t(const GemvParams &p, int grid, int warps, size_t smem, cudaStream_t st) {
    auto kern = gemv_kernel<QT, MT, R>;
    static size_t configured = 0;   // per instantiation; contexts on several devices re-set it
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured || dev != configured_dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
        configured_dev = dev;
    }
    kern<<<grid, warps * 32, smem, st>>>(p);
    return cudaGetLastError();
}

template <int QT>
cudaError_t launch_q(const GemvParams &p, int mt, int grid, int warps, size_t smem, cudaStream_t st) {
    switch (mt) {
    case 1: return launch_t<QT, 1, 2>(p, grid, warps, smem, st);
    case 2: return launch_t<QT, 2, 2>(p, grid, warps, smem, st);
    case 3: return launch_t<QT, 3, 2>(p, grid, warps, smem, st);
    default: return launch_t<QT, 4, 2>(p, grid, warps, smem, st);
    }
}

}  // namespace

int gemv_max_m() { return 4; }

// Returns cudaSuccess, or cudaErrorInvalidValue when the shape cannot be staged in shared memory
// (caller then picks another route).
cudaError_t gemv_launch(const GemvLaunch &a, cudaStream_t st) {
    constexpr int R = 2;
    GemvParams p{};
    if (a.nseg < 1 || a.nseg > kMaxSeg || a.M < 1 || a.M > 4) return cudaErrorInvalidValue;
    int units = 0;
    for (int i = 0; i < a.nseg; ++i) {
        p.seg[i].w = a.w[i];
        p.seg[i].y = a.y[i];
        p.seg[i].ldy = a.ldy[i];
        p.seg[i].n = a.n[i];
        p.seg[i].unit_begin = units;
        units += (a.n[i] + R - 1) / R;
    }
    p.nseg = a.nseg;
    p.total_units = units;
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

    int kc, chunk;
    switch (a.qt) {
    case QT_Q4_K: kc = GemvCfg<QT_Q4_K>::KC; chunk = GemvCfg<QT_Q4_K>::CHUNK; break;
    case QT_Q8_0: kc = GemvCfg<QT_Q8_0>::KC; chunk = GemvCfg<QT_Q8_0>::CHUNK; break;
    case QT_Q6_K: kc = GemvCfg<QT_Q6_K>::KC; chunk = GemvCfg<QT_Q6_K>::CHUNK; break;
    default: return cudaErrorInvalidValue;
    }
    p.nchunks = (p.nsb + kc - 1) / kc;

    const int warps = a.warps > 0 ? (a.warps > kMaxWarps ? kMaxWarps : a.warps) : 8;
    const size_t per_m = 2 * (size_t)p.Kpad + (p.Kpad / 32) * 4 + (p.Kpad / 16) * 4;
    const size_t fixed = kMaxWarps * kMaxDepth * 8 + ((a.M * per_m + 127) & ~size_t(127));
    const size_t budget = a.smem_limit;
    if (fixed + (size_t)warps * 2 * R * chunk > budget) return cudaErrorInvalidValue;
    int depth = (int)((budget - fixed) / ((size_t)warps * R * chunk));
    if (depth > kMaxDepth) depth = kMaxDepth;
    if (a.depth > 0 && a.depth < depth) depth = a.depth;
    p.depth = depth;
    const size_t smem = fixed + (size_t)warps * depth * R * chunk;
    const int grid = a.grid > 0 ? a.grid : a.sm_count;

    switch (a.qt) {
    case QT_Q4_K: return launch_q<QT_Q4_K>(p, a.M, grid, warps, smem, st);
    case QT_Q8_0: return launch_q<QT_Q8_0>(p, a.M, grid, warps, smem, st);
    default: return launch_q<QT_Q6_K>(p, a.M, grid, warps, smem, st);
    }
}

}  // namespace b200q
