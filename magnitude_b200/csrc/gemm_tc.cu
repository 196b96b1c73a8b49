// Prefill GEMM: Y[M][N] = X[M][K] . dequant(W)[N][K]^T on the 5th-generation tensor cores.
//
// One persistent CTA per SM walks output tiles of 128 weight rows x BN tokens (BN <= 256):
//   * warp 0 (one lane) loads the activation tile X[m0 : m0+BN][k : k+64] with TMA (2-D tiled
//     bulk tensor copy, 128-byte swizzle, no multicast) into a 3-stage shared-memory ring;
//     the same lane fetches the packed weight records of the tile's 128 rows, one superblock
//     record per row at a time (a 4-D tiled copy over the streaming layout), into a 2-deep ring;
//   * warps 2..17 dequantize 16 weights per thread and K-step from that ring to fp16 in registers
//     and write them into the stage ring in the K-major 128-byte-swizzled layout the tensor core
//     reads (generic-proxy stores, then fence.proxy.async);
//   * warp 1 (one lane) issues tcgen05.mma (kind::f16, fp16 x fp16 -> fp32) with the dequantized
//     weights as the A operand (M = 128) and the activations as the B operand (N = BN), four
//     K = 16 instructions per stage, accumulating in tensor memory; tcgen05.commit releases the
//     stage to the producers and, after the last K-step, hands the accumulator to the epilogue;
//   * warps 18..21 read the accumulator (tcgen05.ld, one 32-lane quadrant per warp), convert to
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
constexpr int kStages = 3;        // A/B stages
constexpr int kWBufs = 2;         // packed-weight buffers (one superblock record per row each)
constexpr int kWBufBytes = 35 * 1024;   // 128 rows x 272 bytes (largest record), rounded up to 1 KB
constexpr int kDBufBytes = 2048;        // Q6_K: 128 rows x the 16-byte group of fp16 d of a chunk
constexpr int kDequantWarps = 16;  // four threads per weight row, 16 weights each per K-step
constexpr int kEpiWarps = 4;
constexpr int kThreads = (2 + kDequantWarps + kEpiWarps) * 32;   // 704
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
    int nchunks_full;        // chunks of 8 whole records per row; a shorter tail chunk may follow
    int *status;
};

struct GemmSmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t wfull[kWBufs];
    uint64_t wempty[kWBufs];
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

// 4-D tiled TMA load (packed weight records: [bytes/4][row in group][chunk][row group])
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
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

// ---- dequantization to the swizzled A tile ---------------------------------------------------
//
// A dequant thread owns one weight row of the tile and one quarter (16 weights) of the 64-weight
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

// `qd` = which quarter (16 weights, two 16-byte chunks) of the 64-weight K-step the thread makes.
template <int QT> struct Packed;

template <> struct Packed<QT_Q4_K> {
    uint4 hdr, q;
    // rec: shared address of the row's 144-byte record of this K-step's superblock; j: 64-weight unit.
    // Quarters 0, 1 are the low nibbles of bytes 0..15 / 16..31 of the unit, quarters 2, 3 the high.
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j, int qd) {
        hdr = lds128(rec);
        q = lds128(rec + 16 + 32 * j + 16 * (qd & 1));
    }
    template <bool F16> __device__ __forceinline__ void emit(int j, int qd, uint32_t row_saddr, int r7) const {
        int sc, mn;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + (qd >> 1), sc, mn);
        const float ds = half_bits_to_float(hdr.x) * (float)sc;
        const float c0 = -(128.f * ds + half_bits_to_float(hdr.x >> 16) * (float)mn);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        const int sh = 4 * (qd >> 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint32_t a = (w[2 * c] >> sh) & 0x0F0F0F0Fu, b = (w[2 * c + 1] >> sh) & 0x0F0F0F0Fu;
            const uint32_t p0 = pack2<F16>(fmaf(f128_plus<0>(a), ds, c0), fmaf(f128_plus<1>(a), ds, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f128_plus<2>(a), ds, c0), fmaf(f128_plus<3>(a), ds, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f128_plus<0>(b), ds, c0), fmaf(f128_plus<1>(b), ds, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f128_plus<2>(b), ds, c0), fmaf(f128_plus<3>(b), ds, c0));
            st_chunk(row_saddr, r7, 2 * qd + c, p0, p1, p2, p3);
        }
    }
};

template <> struct Packed<QT_Q8_0> {
    uint4 q;
    uint32_t d16;
    // rec: shared address of the 272-byte record; unit j holds native blocks 2j, 2j+1; quarter qd is
    // half of block 2j + qd/2
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j, int qd) {
        q = lds128(rec + 64 * j + 16 * qd);
        d16 = lds16(rec + 256 + 2 * (2 * j + (qd >> 1)));
    }
    template <bool F16> __device__ __forceinline__ void emit(int, int qd, uint32_t row_saddr, int r7) const {
        const float d = half_bits_to_float(d16);
        const float c0 = -32896.f * d;     // (32768 + 128): bytes are taken as unsigned after ^ 0x80
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint32_t a = w[2 * c] ^ 0x80808080u, b = w[2 * c + 1] ^ 0x80808080u;
            const uint32_t p0 = pack2<F16>(fmaf(f32768_plus<0>(a), d, c0), fmaf(f32768_plus<1>(a), d, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f32768_plus<2>(a), d, c0), fmaf(f32768_plus<3>(a), d, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f32768_plus<0>(b), d, c0), fmaf(f32768_plus<1>(b), d, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f32768_plus<2>(b), d, c0), fmaf(f32768_plus<3>(b), d, c0));
            st_chunk(row_saddr, r7, 2 * qd + c, p0, p1, p2, p3);
        }
    }
};

template <> struct Packed<QT_Q6_K> {
    uint4 l, hq;
    uint32_t sc8, d16;
    // rec: shared address of the 208-byte record, dptr: of its fp16 d.  The 64 weights of unit u are quadrants
    // 2(u&1), 2(u&1)+1 of half u>>1; quarter qd is positions 16(qd&1)..+15 of quadrant
    // c = 2(u&1) + qd/2, which is exactly one 16-weight sub-block (one scale).
    __device__ __forceinline__ void load(uint32_t rec, uint32_t dptr, int u, int qd) {
        const int hh = u >> 1, c = 2 * (u & 1) + (qd >> 1), ph = qd & 1;
        l = lds128(rec + 64 * hh + 32 * (c & 1) + 16 * ph);
        hq = lds128(rec + 128 + 32 * hh + 16 * ph);
        const uint32_t a = rec + 192 + 8 * hh + 2 * c + ph;
        sc8 = (lds16(a & ~1u) >> (8 * (a & 1))) & 0xFF;
        d16 = lds16(dptr);
    }
    template <bool F16> __device__ __forceinline__ void emit(int u, int qd, uint32_t row_saddr, int r7) const {
        const int c = 2 * (u & 1) + (qd >> 1);
        const float s = half_bits_to_float(d16) * (float)(int)(int8_t)sc8;
        const float c0 = -32800.f * s;     // 32768 + 32
        const uint32_t lw[4] = {l.x, l.y, l.z, l.w};
        const uint32_t hw[4] = {hq.x, hq.y, hq.z, hq.w};
        const int lsh = 4 * (c >> 1), hsh = 2 * c;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            uint32_t v[2];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                v[i] = ((lw[2 * cc + i] >> lsh) & 0x0F0F0F0Fu) | (((hw[2 * cc + i] >> hsh) & 0x03030303u) << 4);
            const uint32_t p0 = pack2<F16>(fmaf(f32768_plus<0>(v[0]), s, c0), fmaf(f32768_plus<1>(v[0]), s, c0));
            const uint32_t p1 = pack2<F16>(fmaf(f32768_plus<2>(v[0]), s, c0), fmaf(f32768_plus<3>(v[0]), s, c0));
            const uint32_t p2 = pack2<F16>(fmaf(f32768_plus<0>(v[1]), s, c0), fmaf(f32768_plus<1>(v[1]), s, c0));
            const uint32_t p3 = pack2<F16>(fmaf(f32768_plus<2>(v[1]), s, c0), fmaf(f32768_plus<3>(v[1]), s, c0));
            st_chunk(row_saddr, r7, 2 * qd + cc, p0, p1, p2, p3);
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
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                               const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap wtail,
                                                               const __grid_constant__ CUtensorMap dmap, const __grid_constant__ CUtensorMap dtail) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // stage buffers first (1024-byte aligned for the 128-byte swizzle), bookkeeping after them
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_s = smem_u32(smem);
    const uint32_t b_s = a_s + kStages * kStageABytes;
    const uint32_t w_s = b_s + kStages * kStageBBytes;            // packed-weight buffers
    const uint32_t d_s = w_s + kWBufs * kWBufBytes;               // Q6_K d groups, one buffer per chunk parity
    GemmSmem *sm = reinterpret_cast<GemmSmem *>(smem + kStages * (kStageABytes + kStageBBytes) + kWBufs * kWBufBytes + 2 * kDBufBytes);
    const uint32_t wfull_s = smem_u32(sm->wfull), wempty_s = smem_u32(sm->wempty);
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
        for (int i = 0; i < kWBufs; ++i) {
            mbar_init(wfull_s + 8 * i, 1);
            mbar_init(wempty_s + 8 * i, kDequantWarps);
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
        // ===== TMA producer: activation tiles and packed weight records ============================
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)p.bn * BK * 2;
            constexpr int REC = rec_bytes(QT);
            int it = 0, rs = 0;     // K-steps and record-steps issued so far (rings run across tiles)
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
                const int tn = tile / p.m_tiles, tm = tile % p.m_tiles;
                for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                    if ((ks & 3) == 0) {
                        // one superblock record of each of the tile's 128 rows (four K-steps' worth)
                        const int sb = ks >> 2, c = sb >> 3, s_in = sb & 7;
                        const int wb = rs % kWBufs;
                        ok = wait_or_abort(wempty_s + 8 * wb, ((rs / kWBufs) & 1) ^ 1, sm, p.status);
                        if (!ok) break;
                        const bool tail = c >= p.nchunks_full;
                        uint32_t tx = BM * REC;
                        if (QT == QT_Q6_K && s_in == 0) tx += BM * 16;
                        mbar_expect_tx(wfull_s + 8 * wb, tx);
                        tma_load_4d(w_s + wb * kWBufBytes, tail ? &wtail : &wmap, s_in * (REC / 4), 0, tail ? 0 : c,
                                    tn * (BM / kRowGroup), wfull_s + 8 * wb);
                        if (QT == QT_Q6_K && s_in == 0) {
                            const int nrec = tail ? (p.nsb - c * kChunkRecs) : kChunkRecs;
                            tma_load_4d(d_s + (c & 1) * kDBufBytes, tail ? &dtail : &dmap, nrec * (REC / 4), 0, tail ? 0 : c,
                                        tn * (BM / kRowGroup), wfull_s + 8 * wb);
                        }
                        ++rs;
                    }
                    const int stage = it % kStages;
                    ok = wait_or_abort(empty_s + 8 * stage, ((it / kStages) & 1) ^ 1, sm, p.status);
                    if (!ok) break;
                    mbar_expect_tx(full_s + 8 * stage, bytes);
                    tma_load_2d(b_s + stage * kStageBBytes, &xmap, ks * BK, tm * p.bn, full_s + 8 * stage);
                }
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
        const int r = t & (BM - 1), qd = t >> 7;
        const int r7 = r & 7;
        const uint32_t row_off = (r >> 3) * 1024 + r7 * 128;
        constexpr int REC = rec_bytes(QT);
        int it = 0, rs = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
            int wb = 0;
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const int j = ks & 3;
                if (j == 0) {   // a new record: wait for its bytes
                    wb = rs % kWBufs;
                    if (lane == 0) ok = wait_or_abort(wfull_s + 8 * wb, (rs / kWBufs) & 1, sm, p.status);
                    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                    if (!ok) break;
                }
                const int sb = ks >> 2;
                Packed<QT> cur;
                cur.load(w_s + wb * kWBufBytes + r * REC, d_s + ((sb >> 3) & 1) * kDBufBytes + r * 16 + 2 * (sb & 7), j, qd);
                const int stage = it % kStages;
                if (lane == 0) ok = wait_or_abort(empty_s + 8 * stage, ((it / kStages) & 1) ^ 1, sm, p.status);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
                if (!ok) break;
                cur.template emit<F16>(j, qd, a_s + stage * kStageABytes + row_off, r7);
                fence_proxy_async();       // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_s + 8 * stage);
                    if (j == 3 || ks == ksteps - 1) mbar_arrive(wempty_s + 8 * wb);   // record consumed
                }
                if (j == 3 || ks == ksteps - 1) ++rs;
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

struct GemmMaps {
    CUtensorMap x, w, wtail, d, dtail;
};

template <int QT, bool F16>
cudaError_t launch_gemm(const GemmParams &p, const GemmMaps &m, int grid, cudaStream_t st) {
    auto kern = gemm_tc_kernel<QT, F16>;
    const size_t smem = kStages * (kStageABytes + kStageBBytes) + kWBufs * kWBufBytes + 2 * kDBufBytes + sizeof(GemmSmem) + 1024;
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != configured_dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured_dev = dev;
    }
    kern<<<grid, kThreads, smem, st>>>(p, m.x, m.w, m.wtail, m.d, m.dtail);
    return cudaGetLastError();
}

// tensor map over the packed records of the chunks [c0, c0 + nc) of every row:
// [bytes / 4 of a row-chunk][4 rows of a group][chunks][row groups], box = box0 x 4 x 1 x 32
bool encode_weight_map(EncodeTiledFn enc, CUtensorMap *map, const uint8_t *w, int qt, int nsb, int64_t groups,
                       int c0, int nc, int box0) {
    const int64_t rb = row_bytes_for(qt, nsb);
    const int64_t cb = chunk_row_bytes(qt, c0, nsb);
    const cuuint64_t gdim[4] = {(cuuint64_t)(cb / 4), (cuuint64_t)kRowGroup, (cuuint64_t)nc, (cuuint64_t)groups};
    const cuuint64_t gstride[3] = {(cuuint64_t)cb, (cuuint64_t)(kRowGroup * cb), (cuuint64_t)(kRowGroup * rb)};
    const cuuint32_t box[4] = {(cuuint32_t)box0, (cuuint32_t)kRowGroup, 1, (cuuint32_t)(BM / kRowGroup)};
    const cuuint32_t estride[4] = {1, 1, 1, 1};
    void *base = const_cast<uint8_t *>(w) + kRowGroup * rec_off(qt, (int64_t)c0 * kChunkRecs);
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, base, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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

    GemmMaps maps;
    CUtensorMap &map = maps.x;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)p.bn};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = enc(&map, a.weights_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a.x), gdim, gstride, box, estride,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

    // packed weights: whole chunks through one map, the shorter last chunk (if any) through another
    const int64_t groups = padded_rows(a.N) / kRowGroup;
    const int rec4 = rec_bytes(a.qt) / 4;
    p.nchunks_full = p.nsb / kChunkRecs;
    const int ntail = p.nsb % kChunkRecs;
    const int c_main = p.nchunks_full > 0 ? 0 : p.nchunks_full, n_main = p.nchunks_full > 0 ? p.nchunks_full : 1;
    const int c_tail = ntail > 0 ? p.nchunks_full : c_main;
    bool okm = encode_weight_map(enc, &maps.w, a.w, a.qt, p.nsb, groups, c_main, n_main, rec4) &&
               encode_weight_map(enc, &maps.wtail, a.w, a.qt, p.nsb, groups, c_tail, 1, rec4) &&
               encode_weight_map(enc, &maps.d, a.w, a.qt, p.nsb, groups, c_main, n_main, 4) &&
               encode_weight_map(enc, &maps.dtail, a.w, a.qt, p.nsb, groups, c_tail, 1, 4);
    if (!okm) return cudaErrorInvalidValue;

    const int tiles = p.m_tiles * p.n_tiles;
    const int grid = std::min(tiles, a.sm_count);
    if (a.weights_bf16) {
        switch (a.qt) {
        case QT_Q4_K: return launch_gemm<QT_Q4_K, false>(p, maps, grid, st);
        case QT_Q6_K: return launch_gemm<QT_Q6_K, false>(p, maps, grid, st);
        case QT_Q8_0: return launch_gemm<QT_Q8_0, false>(p, maps, grid, st);
        default: return cudaErrorInvalidValue;
        }
    }
    switch (a.qt) {
    case QT_Q4_K: return launch_gemm<QT_Q4_K, true>(p, maps, grid, st);
    case QT_Q6_K: return launch_gemm<QT_Q6_K, true>(p, maps, grid, st);
    case QT_Q8_0: return launch_gemm<QT_Q8_0, true>(p, maps, grid, st);
    default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------------------------------------
// Prefill without any allocation: the 16-bit copy of the activations lives in a fixed array that
// is part of the library image (every GPU that loads the library holds these 8 MiB until the
// process exits).  The array's name is only a host-side handle; the device address is asked for
// once per device, with that device current, and that address is what the kernels receive.
// Every call on a device shares the array and finds the previous call's contents in it; nothing
// in it has to start at zero, because the conversion kernel overwrites every element the GEMM
// then reads.  Calls that overlap on the GPU (two streams) race on it.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_x_scratch[kStaticScratchBytes];

size_t gemm_static_scratch_elems() { return kStaticScratchBytes / 2; }

// First use on a device resolves the array's device address (cudaGetSymbolAddress initialises the
// module on that device, so that first call should happen outside any stream capture).
cudaError_t gemm_launch_static(GemmLaunch a, int x_is_bf16, cudaStream_t st) {
    constexpr int kMaxDevices = 64;
    static void *dev_ptr[kMaxDevices] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!dev_ptr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_x_scratch);
        if (e != cudaSuccess) return e;
        dev_ptr[dev] = ptr;
    }
    const long long ldd = (a.K + 7) & ~7;
    if ((size_t)a.M * (size_t)ldd > gemm_static_scratch_elems()) return cudaErrorInvalidValue;
    e = gemm_convert_x(a.x, x_is_bf16, a.ldx, dev_ptr[dev], a.M, a.K, a.weights_bf16, st);
    if (e != cudaSuccess) return e;
    a.x = dev_ptr[dev];
    a.ldx = ldd;
    return gemm_launch(a, st);
}

}  // namespace b200q
