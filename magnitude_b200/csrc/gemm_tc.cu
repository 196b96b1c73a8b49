// Prefill GEMM: Y[M][N] = X[M][K] . dequant(W)[N][K]^T on the 5th-generation tensor cores.
//
// One persistent CTA per SM walks output tiles of 128 weight rows x BN tokens (BN <= 256):
//   * warp 0 (one lane) loads the activation tile X[m0 : m0+BN][k : k+64] with TMA (2-D tiled
//     bulk tensor copy, 128-byte swizzle, no multicast) into a 4-stage shared-memory ring;
//   * warps 2..9 read the packed weight records of the tile's 128 rows straight from global
//     memory (L2 serves the repeats across token tiles), dequantize 64 weights per row and K-step
//     to bf16 in registers and write them into the same ring in the K-major 128-byte-swizzled
//     layout the tensor core reads (generic-proxy stores, then fence.proxy.async);
//   * warp 1 (one lane) issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32) with the dequantized
//     weights as the A operand (M = 128) and the activations as the B operand (N = BN), four
//     K = 16 instructions per stage, accumulating in tensor memory; tcgen05.commit releases the
//     stage to the producers and, after the last K-step, hands the accumulator to the epilogue;
//   * warps 10..13 read the accumulator (tcgen05.ld, one 32-lane quadrant per warp), convert to
//     the output type and store Y; two accumulator buffers (2 x 256 TMEM columns) let the next
//     tile's main loop run under the epilogue.
// Every mbarrier wait is bounded; a wait that runs out raises the status word and an abort flag,
// all roles leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

namespace {

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int BK = 64;           // weights per K-step (one 128-byte swizzle row of bf16)
constexpr int kStages = 4;
constexpr int kDequantWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = (2 + kDequantWarps + kEpiWarps) * 32;   // 448
constexpr int kTmemCols = 512;   // two accumulator buffers of 256 columns
constexpr int kStageABytes = BM * BK * 2;       // 16 KB
constexpr int kStageBBytes = 256 * BK * 2;      // 32 KB (BN <= 256)

struct GemmParams {
    const uint8_t *w;        // streaming-layout weights
    int qt;
    int N, K, Kpad, nsb;
    void *y;
    long long ldy;
    int y_is_bf16;
    int M;
    int bn;                  // tokens per tile (multiple of 16, <= 256)
    int m_tiles, n_tiles;
    int *status;
};

struct GemmSmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort;
};

// ---- tcgen05 wrappers -----------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 2-D tiled TMA load (no multicast): box lands at dst, bytes are counted on the mbarrier
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups
// 1024 bytes apart (see the tcgen05 matrix-descriptor format: start >> 4 in bits 0..13, leading
// offset in 16..29, stride offset in 32..45, version 1 in 46..47, layout type 2 in 61..63)
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                  // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
    d |= (uint64_t)1 << 46;                  // descriptor version
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}

// two fp32 -> one packed pair of 16-bit floats (lo in the low half).  The weights enter the tensor
// core as fp16 (11-bit significand: rounding error 2^-12, against 2^-9 for bf16) unless F16 is off.
template <bool F16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint4 ldg128(const uint8_t *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

// ---- dequantization to the swizzled A tile ---------------------------------------------------
//
// A dequant thread owns one weight row of the tile and one half (32 weights) of the 64-weight
// K-step.  Small integers become fp32 without a conversion instruction: a byte v placed in the
// mantissa of a float with a fixed exponent reads as (C + v), and one fused multiply-add
// (C + v) * s - (C * s + m) gives the weight.  Eight bf16 values form one 16-byte chunk; chunk cc
// of row r is stored at chunk position cc ^ (r & 7) of the row (128-byte swizzle).

__device__ __forceinline__ void st_chunk(uint32_t row_saddr, int r7, int cc, uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3) {
    const uint32_t a = row_saddr + ((cc ^ r7) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
}

// byte i of v -> float bits 0x43000000 | byte << 16   (value 128 + byte for byte < 128)
template <int I> __device__ __forceinline__ float f128_plus(uint32_t v) {
    return __uint_as_float(__byte_perm(v, 0x43000000u, 0x7044 | (I << 8)));
}
// byte i of v -> float bits 0x47000000 | byte << 8    (value 32768 + byte)
template <int I> __device__ __forceinline__ float f32768_plus(uint32_t v) {
    return __uint_as_float(__byte_perm(v, 0x47000000u, 0x7404 | (I << 4)));
}

template <int QT> struct Packed;

template <> struct Packed<QT_Q4_K> {
    uint4 hdr, qa, qb;
    // rec: the row's 144-byte record of this K-step's superblock; j: 64-weight unit inside it
    __device__ __forceinline__ void load(const uint8_t *rec, const uint8_t *, int j, int) {
        hdr = ldg128(rec);
        qa = ldg128(rec + 16 + 32 * j);
        qb = ldg128(rec + 32 + 32 * j);
    }
    template <bool F16> __device__ __forceinline__ void emit(int j, int h, uint32_t row_saddr, int r7) const {
        int sc, mn;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + h, sc, mn);
        const float ds = half_bits_to_float(hdr.x) * (float)sc;
        const float c0 = -(128.f * ds + half_bits_to_float(hdr.x >> 16) * (float)mn);
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const int sh = 4 * h;   // low nibbles = weights 0..31 of the unit, high nibbles = 32..63
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t a = (w[2 * c] >> sh) & 0x0F0F0F0Fu, b = (w[2 * c + 1] >> sh) & 0x0F0F0F0Fu;
            const uint32_t p0 = pack2<F16>(fmaf(f128_plus<0>(a), ds, c0), fmaf(f128_plus<1>(a), ds, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f128_plus<2>(a), ds, c0), fmaf(f128_plus<3>(a), ds, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f128_plus<0>(b), ds, c0), fmaf(f128_plus<1>(b), ds, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f128_plus<2>(b), ds, c0), fmaf(f128_plus<3>(b), ds, c0));
            st_chunk(row_saddr, r7, 4 * h + c, p0, p1, p2, p3);
        }
    }
};

template <> struct Packed<QT_Q8_0> {
    uint4 q0, q1;
    uint32_t d16;
    // rec: the 272-byte record; unit j holds native blocks 2j, 2j+1; this thread takes block 2j + h
    __device__ __forceinline__ void load(const uint8_t *rec, const uint8_t *, int j, int h) {
        q0 = ldg128(rec + 64 * j + 32 * h);
        q1 = ldg128(rec + 64 * j + 32 * h + 16);
        d16 = __ldg(reinterpret_cast<const unsigned short *>(rec + 256 + 2 * (2 * j + h)));
    }
    template <bool F16> __device__ __forceinline__ void emit(int, int h, uint32_t row_saddr, int r7) const {
        const float d = half_bits_to_float(d16);
        const float c0 = -32896.f * d;     // (32768 + 128): bytes are taken as unsigned after ^ 0x80
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t a = w[2 * c] ^ 0x80808080u, b = w[2 * c + 1] ^ 0x80808080u;
            const uint32_t p0 = pack2<F16>(fmaf(f32768_plus<0>(a), d, c0), fmaf(f32768_plus<1>(a), d, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f32768_plus<2>(a), d, c0), fmaf(f32768_plus<3>(a), d, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f32768_plus<0>(b), d, c0), fmaf(f32768_plus<1>(b), d, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f32768_plus<2>(b), d, c0), fmaf(f32768_plus<3>(b), d, c0));
            st_chunk(row_saddr, r7, 4 * h + c, p0, p1, p2, p3);
        }
    }
};

template <> struct Packed<QT_Q6_K> {
    uint4 l0, l1, h0, h1;
    uint32_t sc16, d16;
    // rec: the 208-byte record, dptr: its fp16 d.  The 64 weights of unit u are quadrants
    // 2(u&1), 2(u&1)+1 of half u>>1; this thread takes quadrant c = 2(u&1) + h (32 weights).
    __device__ __forceinline__ void load(const uint8_t *rec, const uint8_t *dptr, int u, int h) {
        const int hh = u >> 1, c = 2 * (u & 1) + h;
        const uint8_t *ql = rec + 64 * hh + 32 * (c & 1);
        const uint8_t *qh = rec + 128 + 32 * hh;
        l0 = ldg128(ql);
        l1 = ldg128(ql + 16);
        h0 = ldg128(qh);
        h1 = ldg128(qh + 16);
        sc16 = __ldg(reinterpret_cast<const unsigned short *>(rec + 192 + 8 * hh + 2 * c));
        d16 = __ldg(reinterpret_cast<const unsigned short *>(dptr));
    }
    template <bool F16> __device__ __forceinline__ void emit(int u, int h, uint32_t row_saddr, int r7) const {
        const int c = 2 * (u & 1) + h;
        const float d = half_bits_to_float(d16);
        const float s0 = d * (float)(int)(int8_t)(sc16 & 0xFF), s1 = d * (float)(int)(int8_t)(sc16 >> 8);
        const float c00 = -32800.f * s0, c01 = -32800.f * s1;   // 32768 + 32
        const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const int lsh = 4 * (c >> 1), hsh = 2 * c;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const float s = cc < 2 ? s0 : s1, c0 = cc < 2 ? c00 : c01;   // 16 weights per scale
            uint32_t v[2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                v[i] = ((lw[2 * cc + i] >> lsh) & 0x0F0F0F0Fu) | (((hw[2 * cc + i] >> hsh) & 0x03030303u) << 4);
            const uint32_t p0 = pack2<F16>(fmaf(f32768_plus<0>(v[0]), s, c0), fmaf(f32768_plus<1>(v[0]), s, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f32768_plus<2>(v[0]), s, c0), fmaf(f32768_plus<3>(v[0]), s, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f32768_plus<0>(v[1]), s, c0), fmaf(f32768_plus<1>(v[1]), s, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f32768_plus<2>(v[1]), s, c0), fmaf(f32768_plus<3>(v[1]), s, c0));
            st_chunk(row_saddr, r7, 4 * h + cc, p0, p1, p2, p3);
        }
    }
};

// ---- the kernel -------------------------------------------------------------------------------

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, GemmSmem *sm, int *status) {
    volatile int *ab = &sm->abort;
    if (*ab) return false;
    if (mbar_wait_bounded(bar, parity)) return true;
    *ab = 1;
    atomicMax(status, DEV_ERR_PIPE_TIMEOUT);
    return false;
}

template <int QT, bool F16>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // stage buffers first (1024-byte aligned for the 128-byte swizzle), bookkeeping after them
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_s = smem_u32(smem);
    const uint32_t b_s = a_s + kStages * kStageABytes;
    GemmSmem *sm = reinterpret_cast<GemmSmem *>(smem + kStages * (kStageABytes + kStageBBytes));
    const uint32_t full_s = smem_u32(sm->full), empty_s = smem_u32(sm->empty);
    const uint32_t tfull_s = smem_u32(sm->tmem_full), tempty_s = smem_u32(sm->tmem_empty);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles_total = p.m_tiles * p.n_tiles;
    const int ksteps = p.Kpad / BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(full_s + 8 * i, kDequantWarps + 1);
            mbar_init(empty_s + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull_s + 8 * i, 1);
            mbar_init(tempty_s + 8 * i, kEpiWarps);
        }
        sm->abort = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == 0) {   // one full warp allocates tensor memory and later frees it
        tmem_alloc(smem_u32(&sm->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&sm->tmem_base);

    if (warp == 0) {
        // ===== TMA producer: activation tiles ======================================================
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)p.bn * BK * 2;
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
                const int tm = tile % p.m_tiles;
                bool ok = true;
                for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                    const int stage = it % kStages;
                    ok = wait_or_abort(empty_s + 8 * stage, ((it / kStages) & 1) ^ 1, sm, p.status);
                    if (!ok) break;
                    mbar_expect_tx(full_s + 8 * stage, bytes);
                    tma_load_2d(b_s + stage * kStageBBytes, &xmap, ks * BK, tm * p.bn, full_s + 8 * stage);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer ==========================================================================
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((F16 ? 0u : 1u) << 7) | ((F16 ? 0u : 1u) << 10) |   // C fp32; A and B both fp16 or both bf16
                                    ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++tcount) {
                const int buf = tcount & 1;
                bool ok = wait_or_abort(tempty_s + 8 * buf, ((tcount >> 1) & 1) ^ 1, sm, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const int stage = it % kStages;
                    ok = wait_or_abort(full_s + 8 * stage, (it / kStages) & 1, sm, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t adesc = make_desc_sw128(a_s + stage * kStageABytes);
                    const uint64_t bdesc = make_desc_sw128(b_s + stage * kStageBBytes);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)   // 16 bf16 = 32 bytes = +2 in the address field
                        umma_bf16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | kk) != 0);
                    umma_commit(empty_s + 8 * stage);      // the stage may be refilled once these finish
                }
                if (!ok) break;
                umma_commit(tfull_s + 8 * buf);            // accumulator complete
            }
        }
    } else if (warp < 2 + kDequantWarps) {
        // ===== dequant producers: weight tiles =====================================================
        const int t = threadIdx.x - 64;
        const int r = t & (BM - 1), h = t >> 7;
        const int r7 = r & 7;
        const uint32_t row_off = (r >> 3) * 1024 + r7 * 128;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
            const int tn = tile / p.m_tiles;
            const int row = tn * BM + r;
            const bool live = row < p.N;
            const int rowc = live ? row : p.N - 1;   // clamp: out-of-range rows read a valid row, store zeros
            auto locate = [&](int ks, const uint8_t *&rec, const uint8_t *&dptr) {
                const int sb = ks >> 2;
                rec = p.w + record_off(QT, rowc, sb, p.N, p.nsb);
                dptr = (QT == QT_Q6_K) ? p.w + q6k_d_record_off(rowc, sb, p.N, p.nsb) : rec;
            };
            Packed<QT> cur, nxt;
            {
                const uint8_t *rec, *dptr;
                locate(0, rec, dptr);
                cur.load(rec, dptr, 0, h);
            }
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                if (ks + 1 < ksteps) {   // next K-step's packed bytes fly while this one is converted
                    const uint8_t *rec, *dptr;
                    locate(ks + 1, rec, dptr);
                    nxt.load(rec, dptr, (ks + 1) & 3, h);
                }
                const int stage = it % kStages;
                ok = wait_or_abort(empty_s + 8 * stage, ((it / kStages) & 1) ^ 1, sm, p.status);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                const uint32_t row_s = a_s + stage * kStageABytes + row_off;
                if (live) {
                    cur.template emit<F16>(ks & 3, h, row_s, r7);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) st_chunk(row_s, r7, 4 * h + c, 0u, 0u, 0u, 0u);
                }
                fence_proxy_async();       // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(full_s + 8 * stage);
                cur = nxt;
            }
        }
    } else {
        // ===== epilogue ============================================================================
        const int q = warp & 3;            // TMEM lane quadrant this warp may read
        int tcount = 0;
        for (int tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x, ++tcount) {
            const int tn = tile / p.m_tiles, tm = tile % p.m_tiles;
            const int buf = tcount & 1;
            bool ok = wait_or_abort(tfull_s + 8 * buf, (tcount >> 1) & 1, sm, p.status);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const int n = tn * BM + q * 32 + lane;
            const int m0 = tm * p.bn;
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + buf * 256 + ((uint32_t)(q * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (n < p.N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = m0 + c0 + i;
                        if (m < p.M && c0 + i < p.bn) {
                            const long long idx = (long long)m * p.ldy + n;
                            if (p.y_is_bf16)
                                reinterpret_cast<__nv_bfloat16 *>(p.y)[idx] = __float2bfloat16_rn(__uint_as_float(v[i]));
                            else
                                reinterpret_cast<float *>(p.y)[idx] = __uint_as_float(v[i]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_s + 8 * buf);
        }
    }

    // everyone meets here (also after an abort); then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Activations -> the 16-bit float type the weights are dequantized to (both tensor-core operands
// must share one format).  fp16 is the default: bf16 activations convert exactly unless they
// exceed fp16's range, where they saturate to +-65504; fp32 activations round to nearest even.
template <bool F16, bool SRC_BF16>
__global__ void convert_x_kernel(const void *__restrict__ src, long long lds, uint16_t *__restrict__ dst,
                                 long long ldd, int M, int K) {
    const long long total = (long long)M * K;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / K, k = i - m * K;
        float v;
        if (SRC_BF16) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(src)[m * lds + k]);
        else v = reinterpret_cast<const float *>(src)[m * lds + k];
        uint16_t o;
        if (F16) {
            v = fminf(fmaxf(v, -65504.f), 65504.f);   // NaN passes through both
            o = __half_as_ushort(__float2half_rn(v));
        } else {
            o = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        }
        dst[m * ldd + k] = o;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

template <int QT, bool F16>
cudaError_t launch_gemm(const GemmParams &p, const CUtensorMap &map, int grid, cudaStream_t st) {
    auto kern = gemm_tc_kernel<QT, F16>;
    const size_t smem = kStages * (kStageABytes + kStageBBytes) + sizeof(GemmSmem) + 1024;
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != configured_dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured_dev = dev;
    }
    kern<<<grid, kThreads, smem, st>>>(p, map);
    return cudaGetLastError();
}

}  // namespace

size_t gemm_x_scratch_bytes(int M, int K) { return ((size_t)M * ((K + 7) & ~7) * 2 + 255) & ~size_t(255); }

cudaError_t gemm_convert_x(const void *x, int x_is_bf16, long long ldx, void *scratch, int M, int K, int to_bf16,
                           cudaStream_t st) {
    const long long ldd = (K + 7) & ~7;
    const long long total = (long long)M * K;
    const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 16);
    uint16_t *dst = reinterpret_cast<uint16_t *>(scratch);
    if (to_bf16) {
        if (x_is_bf16) convert_x_kernel<false, true><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
        else convert_x_kernel<false, false><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
    } else {
        if (x_is_bf16) convert_x_kernel<true, true><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
        else convert_x_kernel<true, false><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
    }
    return cudaGetLastError();
}

// x: 16-bit float activations [M][K] (fp16, or bf16 when a.weights_bf16) with leading dimension ldx
// (elements); 16-byte aligned rows.
cudaError_t gemm_launch(const GemmLaunch &a, cudaStream_t st) {
    if (a.M < 1 || a.N < 1 || a.K < 1) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (a.ldx * 2) % 16) return cudaErrorInvalidValue;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;

    GemmParams p{};
    p.w = a.w;
    p.qt = a.qt;
    p.N = a.N;
    p.K = a.K;
    p.Kpad = a.Kpad;
    p.nsb = a.Kpad / SB;
    p.y = a.y;
    p.ldy = a.ldy;
    p.y_is_bf16 = a.y_is_bf16;
    p.M = a.M;
    p.bn = a.M >= 256 ? 256 : ((a.M + 15) / 16) * 16;
    if (a.bn_override >= 16 && a.bn_override <= 256 && a.bn_override % 16 == 0) p.bn = a.bn_override;
    p.m_tiles = (a.M + p.bn - 1) / p.bn;
    p.n_tiles = (a.N + BM - 1) / BM;
    p.status = a.status;

    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)p.bn};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = enc(&map, a.weights_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a.x), gdim, gstride, box, estride,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

    const int tiles = p.m_tiles * p.n_tiles;
    const int grid = std::min(tiles, a.sm_count);
    if (a.weights_bf16) {
        switch (a.qt) {
        case QT_Q4_K: return launch_gemm<QT_Q4_K, false>(p, map, grid, st);
        case QT_Q6_K: return launch_gemm<QT_Q6_K, false>(p, map, grid, st);
        case QT_Q8_0: return launch_gemm<QT_Q8_0, false>(p, map, grid, st);
        default: return cudaErrorInvalidValue;
        }
    }
    switch (a.qt) {
    case QT_Q4_K: return launch_gemm<QT_Q4_K, true>(p, map, grid, st);
    case QT_Q6_K: return launch_gemm<QT_Q6_K, true>(p, map, grid, st);
    case QT_Q8_0: return launch_gemm<QT_Q8_0, true>(p, map, grid, st);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200q
