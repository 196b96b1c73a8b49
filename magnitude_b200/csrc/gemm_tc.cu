// Prefill GEMM: Y[M][N] = X[M][K] . dequant(W)[N][K]^T on the 5th-generation tensor cores.
//
// One persistent CTA per SM walks output tiles of 128 weight rows x BN tokens (BN <= 256):
//   * warp 0 (one lane) loads the activation tile X[m0 : m0+BN][k : k+64] (fp16) with TMA (2-D tiled
//     bulk tensor copy, 128-byte swizzle, no multicast) into its own shared-memory ring;
//   * warp 2 (one lane) fetches the packed weight records of the tile's 128 rows, one 256-weight
//     record per row at a time (a 4-D tiled copy over the streaming layout), into a 2-deep ring;
//   * warps 3..18 dequantize: thread (row r, unit j) turns the j-th 64 weights of every record of
//     row r into fp16 with packed half2 arithmetic and writes them into the weight-stage ring in the
//     K-major 128-byte-swizzled layout the tensor core reads (generic-proxy stores, then
//     fence.proxy.async).  The four units of a record are four consecutive K-steps, so the four
//     groups of four warps work on four stages at once;
//   * warp 1 (one lane) issues tcgen05.mma (kind::f16, fp16 x fp16 -> fp32) with the dequantized
//     weights as the A operand (M = 128) and the activations as the B operand (N = BN), four
//     K = 16 instructions per K-step, accumulating in tensor memory; tcgen05.commit releases the
//     two stages to their producers and, after the last K-step, hands the accumulator to the epilogue;
//   * warps 19..22 read the accumulator (tcgen05.ld, one 32-lane quadrant per warp), convert to
//     the output type and store Y; two accumulator buffers (2 x 256 TMEM columns) let the next
//     tile's main loop run under the epilogue.
// Every mbarrier wait is bounded; a wait that runs out raises the status word and an abort flag,
// all roles leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

#ifdef B200Q_GEMM_TRACE
// timing experiments only: the first CTA pair records its pipeline events (SM clock) into this array
__device__ long long g_gemm_trace[16384];
#define GEMM_TRACE(slot) do { if (blockIdx.x == 0 && (slot) < 16384) g_gemm_trace[(slot)] = clock64(); } while (0)
#define GEMM_TRACE_DECL(...) __VA_ARGS__
#else
#define GEMM_TRACE(slot) do { } while (0)
#define GEMM_TRACE_DECL(...)
#endif

namespace {

// timing experiments (parts of the pipeline switched off; results invalid) exist only in builds that ask for them
#ifdef B200Q_TIMING_EXPERIMENTS
#define PAIR_DBG(bit) (p.debug & (bit))
#else
#define PAIR_DBG(bit) (false)
#endif

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int BK = 64;           // weights per K-step (one 128-byte swizzle row of fp16)
constexpr int kAStages = 4;       // dequantized-weight stages: one per unit group, so each group meets every phase of its stage
constexpr int kWBufs = 2;         // packed-weight buffers (one 256-weight record per row each)
constexpr int kDBufBytes = 2048;        // Q6_K: 128 rows x the 16-byte group of fp16 d of a chunk
constexpr int kDequantWarps = 16;  // thread = (row, 64-weight unit of the record)
constexpr int kEpiWarps = 4;
constexpr int kFirstDequantWarp = 3, kFirstEpiWarp = kFirstDequantWarp + kDequantWarps;
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;   // 736
static_assert(kAStages * 4 == kDequantWarps, "one weight stage per group of four dequant warps");
constexpr int kTmemCols = 512;   // two accumulator buffers of 256 columns
constexpr int kStageABytes = BM * BK * 2;       // 16 KB
constexpr int kMaxBStages = 4;

// per-type shared-memory plan: the packed-record buffers differ in size, the activation ring takes
// what is left of the 227 KB
__host__ __device__ constexpr int wbuf_bytes(int qt) { return ((BM * rec_bytes(qt) + 1023) / 1024) * 1024; }
__host__ __device__ constexpr int b_stages(int qt) { return (qt == QT_Q4_K || qt == QT_Q4_0 || qt == QT_MXFP4) ? 4 : 3; }
__host__ __device__ constexpr int bn_max(int qt) { return qt == QT_Q6_K ? 256 : 240; }     // widest token tile
__host__ __device__ constexpr int b_stage_bytes(int qt) { return bn_max(qt) * BK * 2; }
__host__ __device__ constexpr int smem_data_bytes(int qt) {
    return kAStages * kStageABytes + b_stages(qt) * b_stage_bytes(qt) + kWBufs * wbuf_bytes(qt) + (qt == QT_Q6_K ? 2 * kDBufBytes : 0);
}

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
    int ksplit;              // one-CTA kernel: K ranges per tile (1 = none)
    float *part;             // ... their partial products [ksplit][M][N] when ksplit > 1
    int units_per_row;       // two-CTA kernel: 32-token units per 256-row stripe, ceil(M / 32)
    int tps, extra;          // ... tiles per stripe; the first `extra` stripes have one more
    int pair_tiles;          // ... tiles in all
    int debug;               // timing experiments only (results invalid): 1 no activation loads, 2 no dequant math,
                             // 4 no weight loads, 8 no MMA, 16 no epilogue body, 32 no proxy fence (one-CTA kernel);
                             // two-CTA kernel also: 1024 / 2048 no weight-stage / activation-stage hand-shakes
};

struct GemmSmem {
    uint64_t afull[kAStages];
    uint64_t aempty[kAStages];
    uint64_t bfull[kMaxBStages];
    uint64_t bempty[kMaxBStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t wfull[kWBufs];
    uint64_t wempty[kWBufs];
    uint32_t tmem_base;
    int abort;
    int wait_ns;
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

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
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

// ---- dequantization to the swizzled A tile ---------------------------------------------------
//
// A dequant thread owns one weight row of the tile and one 64-weight unit (one K-step) of every
// 256-weight record.  Small integers become fp16 without a conversion instruction: a byte v put
// under the high byte 0x64 reads as the half 1024 + v (under 0x54, a byte with only its high
// nibble set reads as 64 + v / 16).  One exact half2 subtraction removes the offset and one half2
// fused multiply-add applies the block's scale and minimum, two weights per instruction.  Eight fp16 values
// form one 16-byte chunk; chunk cc of row r is stored at chunk position cc ^ (r & 7) of the row
// (128-byte swizzle).

__device__ __forceinline__ void st_chunk(uint32_t row_saddr, int r7, int cc, uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3) {
    const uint32_t a = row_saddr + ((cc ^ r7) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
}

__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// bytes 0..3 of v -> ((b0, b1) - off) * s + c and ((b2, b3) - off) * s + c, MG the high byte given to each
template <uint32_t MG>
__device__ __forceinline__ void word_affine(uint32_t v, __half2 off, __half2 s, __half2 c, uint32_t &p0, uint32_t &p1) {
    p0 = as_u32(__hfma2(__hsub2(as_h2(__byte_perm(v, MG, 0x4140)), off), s, c));
    p1 = as_u32(__hfma2(__hsub2(as_h2(__byte_perm(v, MG, 0x4342)), off), s, c));
}
template <uint32_t MG>
__device__ __forceinline__ void word_scale(uint32_t v, __half2 off, __half2 s, uint32_t &p0, uint32_t &p1) {
    p0 = as_u32(__hmul2(__hsub2(as_h2(__byte_perm(v, MG, 0x4140)), off), s));
    p1 = as_u32(__hmul2(__hsub2(as_h2(__byte_perm(v, MG, 0x4342)), off), s));
}

// Scale s and minimum m of a Q4_K sub-block (weight = s q - m) as half2 constants around the
// integer q0 nearest m / s:  weight = s (q - q0) - (m - s q0).  Both terms are then of the weight's
// own size, so rounding s and the small remainder to fp16 costs about one extra rounding of the
// weight instead of a rounding of m, which is several times larger than the weights.
// `base` is the offset the byte trick adds (1024 or 64); base + q0 stays an exact fp16 integer.
__device__ __forceinline__ void centered(float s, float m, __half2 base, __half2 &off, __half2 &sh, __half2 &ch) {
    float q0 = rintf(__fdividef(m, s));
    q0 = (q0 >= 0.f && q0 <= 1023.f) ? q0 : (q0 > 1023.f ? 1023.f : 0.f);   // NaN (s == 0) -> 0
    off = __hadd2(base, __float2half2_rn(q0));
    sh = __float2half2_rn(s);
    ch = __float2half2_rn(fmaf(s, q0, -m));
}

template <int QT> struct Unit;

// the 64 converted weights of a thread (eight 16-byte chunks in K order) -> its row of the stage
__device__ __forceinline__ void store_row(const uint32_t (&o)[32], uint32_t row_saddr, int r7) {
#pragma unroll
    for (int c = 0; c < 8; ++c) st_chunk(row_saddr, r7, c, o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

template <> struct Unit<QT_Q4_K> {
    uint4 hdr, q0, q1;
    // rec: shared address of the row's 144-byte record; unit j = bytes 32j..32j+31 of the nibbles:
    // low nibbles are weights 0..31 of the K-step (sub-block 2j), high nibbles weights 32..63 (2j+1)
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j) {
        hdr = lds128(rec);
        q0 = lds128(rec + 16 + 32 * j);
        q1 = lds128(rec + 32 + 32 * j);
    }
    __device__ __forceinline__ void convert(int j, uint32_t (&o)[32]) const {
        int sa, ma, sb, mb;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, sa, ma);
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, sb, mb);
        const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
        __half2 o_lo, s_lo, c_lo, o_hi, s_hi, c_hi;
        centered(d * (float)sa, dmin * (float)ma, as_h2(0x64006400u), o_lo, s_lo, c_lo);
        centered(d * (float)sb, dmin * (float)mb, as_h2(0x54005400u), o_hi, s_hi, c_hi);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int n = 0; n < 4; ++n) {     // chunk n = low nibbles of words 2n, 2n+1; chunk 4 + n = their high nibbles
            word_affine<0x64>(w[2 * n] & 0x0F0F0F0Fu, o_lo, s_lo, c_lo, o[4 * n], o[4 * n + 1]);
            word_affine<0x64>(w[2 * n + 1] & 0x0F0F0F0Fu, o_lo, s_lo, c_lo, o[4 * n + 2], o[4 * n + 3]);
            word_affine<0x54>(w[2 * n] & 0xF0F0F0F0u, o_hi, s_hi, c_hi, o[16 + 4 * n], o[16 + 4 * n + 1]);
            word_affine<0x54>(w[2 * n + 1] & 0xF0F0F0F0u, o_hi, s_hi, c_hi, o[16 + 4 * n + 2], o[16 + 4 * n + 3]);
        }
    }
};

// Q5_K: the device record is the Q4_K record followed by the 32 bytes of fifth bits (bit s of byte l =
// weight l of sub-block s); a level 0..31 still fits the byte trick, so both halves of the unit go
// through the 0x64 form.
template <> struct Unit<QT_Q5_K> {
    uint4 hdr, q0, q1, h0, h1;
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j) {
        hdr = lds128(rec);
        q0 = lds128(rec + 16 + 32 * j);
        q1 = lds128(rec + 32 + 32 * j);
        h0 = lds128(rec + 144);
        h1 = lds128(rec + 160);
    }
    __device__ __forceinline__ void convert(int j, uint32_t (&o)[32]) const {
        int sa, ma, sb, mb;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, sa, ma);
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, sb, mb);
        const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
        __half2 o_lo, s_lo, c_lo, o_hi, s_hi, c_hi;
        centered(d * (float)sa, dmin * (float)ma, as_h2(0x64006400u), o_lo, s_lo, c_lo);
        centered(d * (float)sb, dmin * (float)mb, as_h2(0x64006400u), o_hi, s_hi, c_hi);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t f[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int n = 0; n < 4; ++n) {     // chunk n = weights 8n..8n+7 of sub-block 2j; chunk 4 + n = those of sub-block 2j + 1
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t fb = f[2 * n + i] >> (2 * j);
                const uint32_t lo = (w[2 * n + i] & 0x0F0F0F0Fu) | ((fb & 0x01010101u) << 4);
                const uint32_t hi = ((w[2 * n + i] >> 4) & 0x0F0F0F0Fu) | ((fb & 0x02020202u) << 3);
                word_affine<0x64>(lo, o_lo, s_lo, c_lo, o[4 * n + 2 * i], o[4 * n + 2 * i + 1]);
                word_affine<0x64>(hi, o_hi, s_hi, c_hi, o[16 + 4 * n + 2 * i], o[16 + 4 * n + 2 * i + 1]);
            }
        }
    }
};

// Q4_0: [8 x fp16 d][nibbles in the Q4_K arrangement]; weight = d q - 8 d, centred at q0 = 8 exactly
template <> struct Unit<QT_Q4_0> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j) {
        hdr = lds128(rec);
        q0 = lds128(rec + 16 + 32 * j);
        q1 = lds128(rec + 32 + 32 * j);
    }
    __device__ __forceinline__ void convert(int j, uint32_t (&o)[32]) const {
        const uint32_t dw[4] = {hdr.x, hdr.y, hdr.z, hdr.w};
        uint32_t dd = dw[0];
#pragma unroll
        for (int i = 1; i < 4; ++i)
            if (i == j) dd = dw[i];
        const float da = half_bits_to_float(dd), db = half_bits_to_float(dd >> 16);
        __half2 o_lo, s_lo, c_lo, o_hi, s_hi, c_hi;
        centered(da, 8.f * da, as_h2(0x64006400u), o_lo, s_lo, c_lo);
        centered(db, 8.f * db, as_h2(0x54005400u), o_hi, s_hi, c_hi);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            word_affine<0x64>(w[2 * n] & 0x0F0F0F0Fu, o_lo, s_lo, c_lo, o[4 * n], o[4 * n + 1]);
            word_affine<0x64>(w[2 * n + 1] & 0x0F0F0F0Fu, o_lo, s_lo, c_lo, o[4 * n + 2], o[4 * n + 3]);
            word_affine<0x54>(w[2 * n] & 0xF0F0F0F0u, o_hi, s_hi, c_hi, o[16 + 4 * n], o[16 + 4 * n + 1]);
            word_affine<0x54>(w[2 * n + 1] & 0xF0F0F0F0u, o_hi, s_hi, c_hi, o[16 + 4 * n + 2], o[16 + 4 * n + 3]);
        }
    }
};

// MXFP4: [8 scale bytes, 8 of padding][per block four words of eight e2m1 codes in weight order]; a look-up
// gives the bytes 64 + value, read as the halves 1024 + 64 + value; the scale 2^(e - 128) multiplies exactly
// as long as it is an fp16 number (2^-24 .. 2^15; products beyond fp16's range saturate to inf like any fp16 product)
template <> struct Unit<QT_MXFP4> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j) {
        hdr = lds128(rec);
        q0 = lds128(rec + 16 + 32 * j);
        q1 = lds128(rec + 32 + 32 * j);
    }
    __device__ __forceinline__ void convert(int j, uint32_t (&o)[32]) const {
        const uint32_t ew = (j >> 1) ? hdr.y : hdr.x;
        const uint32_t ee = ew >> (16 * (j & 1));
        const __half2 da = __float2half2_rn(__uint_as_float(e8m0_half_bits(ee & 0xFF)));
        const __half2 db = __float2half2_rn(__uint_as_float(e8m0_half_bits((ee >> 8) & 0xFF)));
        const __half2 o1088 = as_h2(0x64406440u);      // 1024 + 64
        const uint32_t wa[4] = {q0.x, q0.y, q0.z, q0.w}, wb[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int n = 0; n < 4; ++n) {     // chunk n = weights 8n .. 8n + 7 of block 2j; chunk 4 + n = those of block 2j + 1
            word_scale<0x64>(mxfp4_bytes(wa[n]), o1088, da, o[4 * n], o[4 * n + 1]);
            word_scale<0x64>(mxfp4_bytes(wa[n] >> 16), o1088, da, o[4 * n + 2], o[4 * n + 3]);
            word_scale<0x64>(mxfp4_bytes(wb[n]), o1088, db, o[16 + 4 * n], o[16 + 4 * n + 1]);
            word_scale<0x64>(mxfp4_bytes(wb[n] >> 16), o1088, db, o[16 + 4 * n + 2], o[16 + 4 * n + 3]);
        }
    }
};

template <> struct Unit<QT_Q8_0> {
    uint4 q[4];
    uint32_t dd;
    // rec: shared address of the 272-byte record [8 x 32 int8][8 x fp16 d]; unit j = native blocks 2j, 2j+1
    __device__ __forceinline__ void load(uint32_t rec, uint32_t, int j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = lds128(rec + 64 * j + 16 * i);
        dd = lds32(rec + 256 + 4 * j);
    }
    __device__ __forceinline__ void convert(int, uint32_t (&o)[32]) const {
        const __half2 d_lo = as_h2(__byte_perm(dd, 0, 0x1010)), d_hi = as_h2(__byte_perm(dd, 0, 0x3232));
        const __half2 o1152 = as_h2(0x64806480u);      // bytes are taken as unsigned after ^ 0x80: 1024 + 128 + q
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 d = i < 2 ? d_lo : d_hi;
            const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
            for (int c = 0; c < 2; ++c) {     // chunk 2i + c
                word_scale<0x64>(w[2 * c] ^ 0x80808080u, o1152, d, o[8 * i + 4 * c], o[8 * i + 4 * c + 1]);
                word_scale<0x64>(w[2 * c + 1] ^ 0x80808080u, o1152, d, o[8 * i + 4 * c + 2], o[8 * i + 4 * c + 3]);
            }
        }
    }
};

template <> struct Unit<QT_Q6_K> {
    uint4 l[4], hq[2];
    uint32_t sc4, d16;
    // rec: shared address of the 208-byte record [ql 128][qh 64][sc 16], dptr: of its fp16 d.  Unit u is
    // quadrants 2(u&1), 2(u&1)+1 of half u>>1: 64 bytes of ql (low nibbles for even u, high for odd),
    // 32 bytes of qh (bit pair 2(u&1) + quarter/2), four int8 scales (one per 16 weights).
    __device__ __forceinline__ void load(uint32_t rec, uint32_t dptr, int u) {
        const int hh = u >> 1;
#pragma unroll
        for (int i = 0; i < 4; ++i) l[i] = lds128(rec + 64 * hh + 16 * i);
        hq[0] = lds128(rec + 128 + 32 * hh);
        hq[1] = lds128(rec + 144 + 32 * hh);
        sc4 = lds32(rec + 192 + 8 * hh + 4 * (u & 1));
        d16 = lds16(dptr);
    }
    __device__ __forceinline__ void convert(int u, uint32_t (&o)[32]) const {
        const float d = half_bits_to_float(d16);
        const int lsh = 4 * (u & 1);
        const __half2 o1056 = as_h2(0x64206420u);      // 1024 + 32
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            const __half2 s = __float2half2_rn(d * (float)(int)(int8_t)(sc4 >> (8 * qd)));
            const int hsh = lsh + 2 * (qd >> 1);
            const uint32_t lw[4] = {l[qd].x, l[qd].y, l[qd].z, l[qd].w};
            const uint32_t hw[4] = {hq[qd & 1].x, hq[qd & 1].y, hq[qd & 1].z, hq[qd & 1].w};
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {     // chunk 2 qd + cc
                uint32_t v[2];
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    v[i] = ((lw[2 * cc + i] >> lsh) & 0x0F0F0F0Fu) | (((hw[2 * cc + i] >> hsh) & 0x03030303u) << 4);
                word_scale<0x64>(v[0], o1056, s, o[8 * qd + 4 * cc], o[8 * qd + 4 * cc + 1]);
                word_scale<0x64>(v[1], o1056, s, o[8 * qd + 4 * cc + 2], o[8 * qd + 4 * cc + 3]);
            }
        }
    }
};

// ---- the kernel -------------------------------------------------------------------------------

// Bounded wait.  FAST waits sit on the critical path (tensor-core issue, dequant hand-over, TMA
// issue) and re-check every few dozen nanoseconds; the others (the epilogue's, long by design)
// let the hardware suspend them for as long as it likes.  After the limit the waiter raises the
// status word and the abort flag, which every other waiter polls.
template <bool FAST>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, GemmSmem *sm, int *status) {
    if (FAST) {
#pragma unroll 1
        for (int i = 0; i < (1 << 14); ++i)
            if (mbar_try_wait_hint(bar, parity, (uint32_t)sm->wait_ns)) return true;
    } else if (mbar_try_wait(bar, parity)) {
        return true;
    }
    volatile int *ab = &sm->abort;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*ab) return false;
        if (globaltimer_ns() - t0 > kWaitLimitNs) {
            *ab = 1;
            atomicMax(status, DEV_ERR_PIPE_TIMEOUT);
            return false;
        }
    }
}

// After an abort the roles have left their loops, but TMA loads and MMAs they issued may still be
// in flight towards this CTA's shared memory: give them a fixed time (far above a load's latency)
// to land before the CTA exits and its shared memory goes to another CTA.
__device__ __forceinline__ void drain_after_abort(const int *abort_flag) {
    if (*reinterpret_cast<const volatile int *>(abort_flag)) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 100000) {
        }
        __syncthreads();
    }
}

// Split of the K range for small products: with few output tiles (a skinny batch against a
// weight of a few thousand rows) most SMs would idle, so each tile's records are cut into
// p.ksplit ranges that run as separate work units; their fp32 partial products go to a workspace
// [ksplit][M][N] and a second kernel adds them up in split order (deterministic).
struct TileK {
    int tn, tm, r0, r1;      // weight-row tile, token tile, record range [r0, r1) of the row
};
__device__ __forceinline__ TileK tile_k(const GemmParams &p, int tile) {
    TileK t;
    const int s = tile % p.ksplit, q = tile / p.ksplit;
    t.tn = q / p.m_tiles;
    t.tm = q - t.tn * p.m_tiles;
    t.r0 = (int)((long long)p.nsb * s / p.ksplit);
    t.r1 = (int)((long long)p.nsb * (s + 1) / p.ksplit);
    return t;
}

template <int QT>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                               const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap wtail,
                                                               const __grid_constant__ CUtensorMap dmap, const __grid_constant__ CUtensorMap dtail) {
    constexpr int SB_ = b_stages(QT);
    constexpr int WBUF = wbuf_bytes(QT);
    constexpr int REC = rec_bytes(QT);
    constexpr int kStageBBytes = b_stage_bytes(QT);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // stage buffers first (1024-byte aligned for the 128-byte swizzle), bookkeeping after them
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_s = smem_u32(smem);
    const uint32_t b_s = a_s + kAStages * kStageABytes;
    const uint32_t w_s = b_s + SB_ * kStageBBytes;                // packed-weight buffers
    const uint32_t d_s = w_s + kWBufs * WBUF;                     // Q6_K d groups, two buffers
    GemmSmem *sm = reinterpret_cast<GemmSmem *>(smem + smem_data_bytes(QT));
    const uint32_t wfull_s = smem_u32(sm->wfull), wempty_s = smem_u32(sm->wempty);
    const uint32_t afull_s = smem_u32(sm->afull), aempty_s = smem_u32(sm->aempty);
    const uint32_t bfull_s = smem_u32(sm->bfull), bempty_s = smem_u32(sm->bempty);
    const uint32_t tfull_s = smem_u32(sm->tmem_full), tempty_s = smem_u32(sm->tmem_empty);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_units = p.m_tiles * p.n_tiles * p.ksplit;      // work units: (tile, K range)

    if (threadIdx.x == 0) {
        for (int i = 0; i < kAStages; ++i) {
            mbar_init(afull_s + 8 * i, kDequantWarps / 4);     // the four warps of one unit group
            mbar_init(aempty_s + 8 * i, 1);
        }
        for (int i = 0; i < SB_; ++i) {
            mbar_init(bfull_s + 8 * i, 1);
            mbar_init(bempty_s + 8 * i, 1);
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
        sm->wait_ns = 40;
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
            int it = 0;             // K-steps issued so far (the ring runs across work units)
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const TileK t = tile_k(p, unit);
                for (int ks = 4 * t.r0; ks < 4 * t.r1; ++ks, ++it) {
                    const int stage = it % SB_;
                    ok = wait_or_abort<true>(bempty_s + 8 * stage, ((it / SB_) & 1) ^ 1, sm, p.status);
                    if (!ok) break;
                    if (PAIR_DBG(1)) {
                        mbar_arrive(bfull_s + 8 * stage);
                        continue;
                    }
                    mbar_expect_tx(bfull_s + 8 * stage, bytes);
                    tma_load_2d(b_s + stage * kStageBBytes, &xmap, ks * BK, t.tm * p.bn, bfull_s + 8 * stage);
                }
            }
        }
    } else if (warp == 2) {
        // ===== TMA producer: packed weight records =================================================
        if (lane == 0) {
            int rs = 0, dcount = 0;   // records issued so far; d groups loaded so far (Q6_K)
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const TileK t = tile_k(p, unit);
                for (int sb = t.r0; sb < t.r1; ++sb, ++rs) {
                    // one record of each of the tile's 128 rows (four K-steps' worth)
                    const int c = sb >> 3, s_in = sb & 7;
                    const int wb = rs % kWBufs;
                    ok = wait_or_abort<true>(wempty_s + 8 * wb, ((rs / kWBufs) & 1) ^ 1, sm, p.status);
                    if (!ok) break;
                    if (PAIR_DBG(4)) {
                        mbar_arrive(wfull_s + 8 * wb);
                        continue;
                    }
                    const bool tail = c >= p.nchunks_full;
                    const bool need_d = QT == QT_Q6_K && (s_in == 0 || sb == t.r0);   // first record of a chunk (or of the range)
                    uint32_t tx = BM * REC;
                    if (need_d) tx += BM * 16;
                    mbar_expect_tx(wfull_s + 8 * wb, tx);
                    tma_load_4d(w_s + wb * WBUF, tail ? &wtail : &wmap, s_in * (REC / 4), 0, tail ? 0 : c,
                                t.tn * (BM / kRowGroup), wfull_s + 8 * wb);
                    if (need_d) {
                        // the chunk's fp16 d values go to the d buffer used two loads ago: every record that
                        // read it is at least two records back, which the wait above has seen consumed
                        const int nrec = tail ? (p.nsb - c * kChunkRecs) : kChunkRecs;
                        tma_load_4d(d_s + (dcount & 1) * kDBufBytes, tail ? &dtail : &dmap, nrec * (REC / 4), 0, tail ? 0 : c,
                                    t.tn * (BM / kRowGroup), wfull_s + 8 * wb);
                        ++dcount;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer ==========================================================================
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) |                                   // C fp32; A and B fp16 (format 0)
                                    ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int it = 0, ucount = 0;
            bool rdy_a = false, rdy_b = false;
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++ucount) {
                const TileK t = tile_k(p, unit);
                const int buf = ucount & 1;
                bool ok = wait_or_abort<true>(tempty_s + 8 * buf, ((ucount >> 1) & 1) ^ 1, sm, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                const int ksteps = 4 * (t.r1 - t.r0);
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const int sa = it % kAStages, sb = it % SB_;
                    // the probes for this K-step were issued before the previous one's MMAs
                    ok = rdy_b || wait_or_abort<true>(bfull_s + 8 * sb, (it / SB_) & 1, sm, p.status);
                    ok = ok && (rdy_a || wait_or_abort<true>(afull_s + 8 * sa, (it / kAStages) & 1, sm, p.status));
                    if (!ok) break;
                    tc_fence_after();
                    {   // probe the next K-step's barriers now; the answers arrive while the MMAs issue
                        const int nx = it + 1;
                        rdy_b = mbar_test_wait(bfull_s + 8 * (nx % SB_), (nx / SB_) & 1);
                        rdy_a = mbar_test_wait(afull_s + 8 * (nx % kAStages), (nx / kAStages) & 1);
                    }
                    const uint64_t adesc = make_desc_sw128(a_s + sa * kStageABytes);
                    const uint64_t bdesc = make_desc_sw128(b_s + sb * kStageBBytes);
                    if (!PAIR_DBG(8))
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk)   // 16 fp16 = 32 bytes = +2 in the address field
                            umma_f16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks | kk) != 0);
                    umma_commit(aempty_s + 8 * sa);        // both stages may be refilled once these finish
                    umma_commit(bempty_s + 8 * sb);
                }
                if (!ok) break;
                umma_commit(tfull_s + 8 * buf);            // accumulator complete
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ===== dequant producers: weight tiles =====================================================
        const int t = threadIdx.x - kFirstDequantWarp * 32;
        const int r = t & (BM - 1), j = t >> 7;      // weight row of the tile; 64-weight unit of each record
        const int r7 = r & 7;
        const uint32_t row_off = (r >> 3) * 1024 + r7 * 128;
        // Records are taken one ahead: the bytes of the next record move into registers before the
        // current one is dequantized, so its buffer goes back to the TMA producer a whole record
        // (four K-steps) before the ring would otherwise allow.
        int f_unit = blockIdx.x, f_sb = 0, f_r1 = 0, f_r0 = 0;   // the record to fetch next
        bool f_valid = f_unit < n_units;
        if (f_valid) {
            const TileK tk = tile_k(p, f_unit);
            f_sb = f_r0 = tk.r0;
            f_r1 = tk.r1;
        }
        int fetched = 0, dcount = 0;
        bool ok = true;
        auto fetch = [&](Unit<QT> &u) {
            const int wb = fetched % kWBufs;
            if (lane == 0) ok = wait_or_abort<true>(wfull_s + 8 * wb, (fetched / kWBufs) & 1, sm, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) return;
            if (QT == QT_Q6_K && ((f_sb & 7) == 0 || f_sb == f_r0)) ++dcount;     // this record came with a new d group
            u.load(w_s + wb * WBUF + r * REC, d_s + ((dcount - 1) & 1) * kDBufBytes + r * 16 + 2 * (f_sb & 7), j);
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty_s + 8 * wb);     // the record is in registers
            ++fetched;
            if (++f_sb == f_r1) {                              // on to the next work unit of this CTA
                f_unit += gridDim.x;
                f_valid = f_unit < n_units;
                if (f_valid) {
                    const TileK tk = tile_k(p, f_unit);
                    f_sb = f_r0 = tk.r0;
                    f_r1 = tk.r1;
                }
            }
        };
        Unit<QT> cur, nxt;
        bool have_cur = f_valid;
        if (have_cur) fetch(cur);
        for (int rs = 0; have_cur && ok; ++rs) {
            const bool have_next = f_valid;
            if (have_next) {
                fetch(nxt);
                if (!ok) break;
            }
            // the arithmetic happens while the tensor core still reads the stage's previous contents:
            // once the stage is free only the eight stores remain before it can be handed over
            uint32_t o[32];
            if (!PAIR_DBG(2)) cur.convert(j, o);
            const int stage = j;       // K-step 4 rs + j: kAStages == 4, so the group owns this stage
            if (lane == 0) ok = wait_or_abort<true>(aempty_s + 8 * stage, (rs & 1) ^ 1, sm, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            if (!PAIR_DBG(2)) store_row(o, a_s + stage * kStageABytes + row_off, r7);
            if (!PAIR_DBG(32)) fence_proxy_async();       // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(afull_s + 8 * stage);
            cur = nxt;
            have_cur = have_next;
        }
    } else {
        // ===== epilogue ============================================================================
        const int q = warp & 3;            // TMEM lane quadrant this warp may read
        int ucount = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++ucount) {
            const TileK t = tile_k(p, unit);
            const int buf = ucount & 1;
            bool ok = wait_or_abort<false>(tfull_s + 8 * buf, (ucount >> 1) & 1, sm, p.status);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const int n = t.tn * BM + q * 32 + lane;
            const int m0 = t.tm * p.bn;
            float *part = p.ksplit > 1 ? p.part + (size_t)(unit % p.ksplit) * p.M * p.N : nullptr;
            for (int c0 = 0; c0 < (PAIR_DBG(16) ? 0 : p.bn); c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + buf * 256 + ((uint32_t)(q * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (n < p.N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = m0 + c0 + i;
                        if (m < p.M && c0 + i < p.bn) {
                            if (part) {
                                part[(size_t)m * p.N + n] = __uint_as_float(v[i]);
                                continue;
                            }
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
    drain_after_abort(&sm->abort);
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// sums the K-range partial products of a split launch in split order and stores the output
__global__ void gemm_ksplit_sum_kernel(const float *__restrict__ part, int ksplit, int M, int N, void *y, long long ldy, int y_is_bf16) {
    const long long total = (long long)M * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = part[i];
        for (int s = 1; s < ksplit; ++s) v += part[(long long)s * total + i];
        const long long m = i / N, n = i - m * N;
        if (y_is_bf16) reinterpret_cast<__nv_bfloat16 *>(y)[m * ldy + n] = __float2bfloat16_rn(v);
        else reinterpret_cast<float *>(y)[m * ldy + n] = v;
    }
}

// ---- the two-CTA kernel -----------------------------------------------------------------------
//
// Two CTAs on neighbouring SMs (a cluster of two) share one 256-row x BN-token tile: each CTA
// dequantizes 128 of the weight rows and stages half of the activation tile, and one thread of
// the leader CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads A from both CTAs' shared
// memory and each half of B once for both tensor cores.  Per SM and K-step that halves the
// activation bytes staged by TMA and read by the tensor core.  No multicast load anywhere: every
// CTA loads its own bytes; only the completion signals cross the pair:
//   * "stage full" barriers live in the leader: the peer's dequant warps arrive on them remotely
//     (mapa + mbarrier.arrive.release.cluster) and both CTAs' activation loads count their bytes
//     on the leader's barrier (cp.async.bulk.tensor ... .cta_group::2, no multicast);
//   * "stage empty" and "accumulator full" are tcgen05.commit.cta_group::2 ... multicast::cluster
//     arrivals on the same barrier offset in both CTAs;
//   * "accumulator empty" lives in the leader: the peer's epilogue warps arrive remotely.
// Tensor memory is allocated by each CTA for itself; a cluster barrier before the exit keeps either
// CTA's shared and tensor memory alive until the other has finished using it.

// Second form of the same kernel (TS = true): the dequantized weights never touch shared memory.
// A dequant thread holds one weight row's 64 values of a K-step in 32 registers, which is exactly
// one tcgen05.st.32x32b.x32 into the row's lane of tensor memory; the MMA then takes its A operand
// from tensor memory.  Per K-step that removes 16 KB of shared-memory stores and 16 KB of operand
// reads per SM, the two largest items on the shared-memory port after the activation operand, and
// the proxy fence that went with the stores.  Tensor memory (512 columns) then holds four A stages
// (32 columns each) and two accumulators of 192 columns, so token tiles are at most 192 wide and
// each CTA stages 96-token halves of the activation tile.
constexpr int kPairThreads = kThreads;
constexpr int kTsAccCols = 192;                     // accumulator buffer stride in TS form
constexpr int kTsACol0 = 2 * kTsAccCols;            // first A-stage column in TS form (4 stages x 32 columns)
// Stages of the pair kernel.  Dequantized-weight stages are used round robin by K-step (group j of
// the dequant warps fills K-steps j, j + 4, ...); with more than four, the hand-over after a stage is
// released (stores, proxy fence, arrival across the pair: more than a thousand cycles) is off the
// tensor cores' path.  Activation stages hide the latency of the TMA loads.  Q4_K's small records
// leave room for 11 stages of 16 KB; 6 + 4 (both in two-stage hand-over units, see the kernel)
// measured fastest: 1026 TFLOP/s on 2048 x 4096 x 14336 against 956 for 6 + 5 and 833 for 4 + 6; the
// same split serves Q5_K and Q6_K (Q6_K: 896 TFLOP/s against 792 with 4 + 6).  Q8_0's packed-record
// buffers (2 x 34 KB) and the TS form's tensor-memory budget leave four weight stages.
// B200Q_PAIR_SA / B200Q_PAIR_SB override the split at compile time.
constexpr int kMaxPairAStages = 8;
#ifndef B200Q_PAIR_SA
#define B200Q_PAIR_SA 6
#define B200Q_PAIR_SB 4
#endif
__host__ __device__ constexpr int pair_a_stages(int qt, bool ts) { return (!ts && qt != QT_Q8_0) ? B200Q_PAIR_SA : 4; }
__host__ __device__ constexpr int pair_b_rows(bool ts) { return ts ? 96 : 128; }       // tokens each CTA stages per K-step
__host__ __device__ constexpr int pair_b_stage_bytes(bool ts = false) { return ((pair_b_rows(ts) * BK * 2 + 1023) / 1024) * 1024; }
__host__ __device__ constexpr int pair_b_stages(int qt, bool ts = false) { return ts ? 8 : qt == QT_Q8_0 ? 5 : B200Q_PAIR_SB; }
// activation stages per hand-over unit: two when the stages pair up
__host__ __device__ constexpr int pair_b_group(int qt, bool ts = false) { return pair_b_stages(qt, ts) % 2 == 0 ? 2 : 1; }
constexpr int kMaxPairBStages = 8;
__host__ __device__ constexpr int pair_smem_data_bytes(int qt, bool ts = false) {
    return (ts ? 0 : pair_a_stages(qt, ts) * kStageABytes) + pair_b_stages(qt, ts) * pair_b_stage_bytes(ts) + kWBufs * wbuf_bytes(qt) + (qt == QT_Q6_K ? 2 * kDBufBytes : 0);
}

struct PairSmem {
    uint64_t afull[kMaxPairAStages];   // leader's copy is used: 4 local + 4 remote warp arrivals
    uint64_t aempty[kMaxPairAStages];
    uint64_t bfull[kMaxPairBStages];   // leader's copy is used: its own expect_tx arrival + both CTAs' bytes
    uint64_t bempty[kMaxPairBStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];            // leader's copy is used: 4 local + 4 remote warp arrivals
    uint64_t wfull[kWBufs];
    uint64_t wempty[kWBufs];
    uint32_t tmem_base;
    int abort;
    int wait_ns;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_rank(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled TMA load into this CTA's shared memory whose bytes are counted on a barrier given by
// its shared::cluster address (here: the leader's); no multicast
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at this offset in both CTAs once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
                 : "memory");
}

// the same MMA with the A operand in tensor memory (this CTA's 128 rows in its own lanes, the peer's in its)
__device__ __forceinline__ void umma_f16_pair_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 registers of one thread -> 32 consecutive columns of the thread's tensor-memory lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tensor-memory management of the pair: one warp of each CTA executes these (every tcgen05
// instruction of a kernel names the same CTA group)
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

template <bool FAST>
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, PairSmem *sm, int *status) {
    if (FAST) {
#pragma unroll 1
        for (int i = 0; i < (1 << 14); ++i)
            if (mbar_try_wait_hint(bar, parity, 40)) return true;
    } else if (mbar_try_wait(bar, parity)) {
        return true;
    }
    volatile int *ab = &sm->abort;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*ab) return false;
        if (globaltimer_ns() - t0 > kWaitLimitNs) {
            *ab = 1;
            atomicMax(status, DEV_ERR_PIPE_TIMEOUT);
            return false;
        }
    }
}

// Tiles of the pair kernel: a stripe (256 weight rows x all tokens) is cut into n tiles of nearly
// equal width, widths being multiples of 32 tokens (a "unit") up to 256: the first `p.extra`
// stripes get p.tps + 1 tiles, the others p.tps (see pick_pair_tiles).  Tile t goes to pair
// t mod pairs.
__device__ __forceinline__ void pair_tile(const GemmParams &p, int tile, int &stripe, int &t0, int &width) {
    int idx, n;
    const int big = p.extra * (p.tps + 1);
    if (tile < big) {
        n = p.tps + 1;
        stripe = tile / n;
        idx = tile - stripe * n;
    } else {
        n = p.tps;
        const int t = tile - big;
        const int q = t / n;
        stripe = p.extra + q;
        idx = t - q * n;
    }
    const int base = p.units_per_row / n, rem = p.units_per_row - base * n;   // `rem` tiles are one unit wider
    const int w = base + (idx < rem ? 1 : 0);
    t0 = 32 * (idx < rem ? idx * (base + 1) : rem * (base + 1) + (idx - rem) * base);
    width = 32 * w;
}

// p.n_tiles counts 256-row stripes here
template <int QT, bool TS>
__global__ void __launch_bounds__(kPairThreads, 1) gemm_tc_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                                      const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap wtail,
                                                                      const __grid_constant__ CUtensorMap dmap, const __grid_constant__ CUtensorMap dtail) {
    constexpr int SB_ = pair_b_stages(QT, TS);
    constexpr int WBUF = wbuf_bytes(QT);
    constexpr int REC = rec_bytes(QT);
    constexpr int kStageBBytes = pair_b_stage_bytes(TS);
    constexpr int kAccCols = TS ? kTsAccCols : 256;         // tensor-memory columns between the two accumulators
    constexpr int SA_ = pair_a_stages(QT, TS);              // dequantized-weight stages, used round robin by K-step
    // Hand-over granularity.  The tensor cores take two K-steps (eight MMAs) per turn of the issuing
    // thread's loop, so what that thread executes between MMAs is paid once per 128 weights: a weight
    // unit is two consecutive stages with one pair of barriers; an activation unit is two stages when
    // their number is even, one otherwise.
    constexpr int GA = 2, GB = pair_b_group(QT, TS);
    constexpr int UA = SA_ / GA, UB = SB_ / GB;
    static_assert(SA_ % GA == 0 && SB_ % GB == 0, "stages must fill whole hand-over units");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t a_s = smem_u32(smem);                    // TS: no weight stages in shared memory
    const uint32_t b_s = a_s + (TS ? 0 : SA_ * kStageABytes);
    const uint32_t w_s = b_s + SB_ * kStageBBytes;
    const uint32_t d_s = w_s + kWBufs * WBUF;
    PairSmem *sm = reinterpret_cast<PairSmem *>(smem + pair_smem_data_bytes(QT, TS));
    const uint32_t wfull_s = smem_u32(sm->wfull), wempty_s = smem_u32(sm->wempty);
    const uint32_t afull_s = smem_u32(sm->afull), aempty_s = smem_u32(sm->aempty);
    const uint32_t bfull_s = smem_u32(sm->bfull), bempty_s = smem_u32(sm->bempty);
    const uint32_t tfull_s = smem_u32(sm->tmem_full), tempty_s = smem_u32(sm->tmem_empty);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int ksteps = p.nsb * 4;
    const int chunks_per_tile = (p.nsb + kChunkRecs - 1) / kChunkRecs;

    if (threadIdx.x == 0) {
        for (int i = 0; i < UA; ++i) {
            mbar_init(afull_s + 8 * i, GA * 2 * (kDequantWarps / 4));   // GA groups of four warps in each CTA
            mbar_init(aempty_s + 8 * i, 1);
        }
        for (int i = 0; i < UB; ++i) {
            mbar_init(bfull_s + 8 * i, 1);
            mbar_init(bempty_s + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tfull_s + 8 * i, 1);
            mbar_init(tempty_s + 8 * i, 2 * kEpiWarps);
        }
        for (int i = 0; i < kWBufs; ++i) {
            mbar_init(wfull_s + 8 * i, 1);
            mbar_init(wempty_s + 8 * i, kDequantWarps);
        }
        sm->abort = 0;
        sm->wait_ns = 40;
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == 0) {
        tmem_alloc_pair(smem_u32(&sm->tmem_base), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // both CTAs' barriers exist before anything crosses the pair
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(&sm->tmem_base);

    if (warp == 0) {
        // ===== TMA producer: this CTA's half of the activation tile ================================
        if (lane == 0) {
            // every load is a full box of 128 (TS: 96) tokens (rows past the tile's half are never read), so
            // the byte count on the leader's barrier does not depend on the tile's width
            const uint32_t bytes_pair = 2u * pair_b_rows(TS) * BK * 2;
            const uint32_t bfull_leader = mapa_rank(bfull_s, 0);
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < p.pair_tiles && ok; tile += n_pairs) {
                int stripe, t0, width;
                pair_tile(p, tile, stripe, t0, width);
                for (int ks = 0; ks < ksteps; ++ks, ++it) {
                    const int stage = it % SB_, unit = stage / GB;
                    if (PAIR_DBG(2048)) continue;
                    if (stage % GB == 0) {      // first stage of a unit: the unit is free, and its barrier expects all its loads
                        ok = pair_wait<true>(bempty_s + 8 * unit, ((it / SB_) & 1) ^ 1, sm, p.status);
                        if (!ok) break;
                        if (PAIR_DBG(1)) {
                            if (rank == 0) mbar_arrive(bfull_s + 8 * unit);
                            continue;
                        }
                        if (rank == 0) mbar_expect_tx(bfull_s + 8 * unit, GB * bytes_pair);
                    } else if (PAIR_DBG(1)) {
                        continue;
                    }
                    tma_load_2d_pair(b_s + stage * kStageBBytes, &xmap, ks * BK, t0 + (int)rank * (width >> 1), bfull_leader + 8 * unit);
                }
            }
        }
    } else if (warp == 2) {
        // ===== TMA producer: packed weight records of this CTA's 128 rows ==========================
        if (lane == 0) {
            int rs = 0, tcount = 0;
            bool ok = true;
            for (int tile = pair; tile < p.pair_tiles && ok; tile += n_pairs, ++tcount) {
                int stripe, t0, width;
                pair_tile(p, tile, stripe, t0, width);
                const int group0 = (stripe * 2 * BM + (int)rank * BM) / kRowGroup;
                for (int sb = 0; sb < p.nsb; ++sb, ++rs) {
                    const int c = sb >> 3, s_in = sb & 7;
                    const int wb = rs % kWBufs;
                    ok = pair_wait<true>(wempty_s + 8 * wb, ((rs / kWBufs) & 1) ^ 1, sm, p.status);
                    if (!ok) break;
                    if (PAIR_DBG(4)) {
                        mbar_arrive(wfull_s + 8 * wb);
                        continue;
                    }
                    const bool tail = c >= p.nchunks_full;
                    uint32_t tx = BM * REC;
                    if (QT == QT_Q6_K && s_in == 0) tx += BM * 16;
                    mbar_expect_tx(wfull_s + 8 * wb, tx);
                    tma_load_4d(w_s + wb * WBUF, tail ? &wtail : &wmap, s_in * (REC / 4), 0, tail ? 0 : c, group0, wfull_s + 8 * wb);
                    if (QT == QT_Q6_K && s_in == 0) {
                        const int nrec = tail ? (p.nsb - c * kChunkRecs) : kChunkRecs;
                        const int cs = tcount * chunks_per_tile + c;
                        tma_load_4d(d_s + (cs & 1) * kDBufBytes, tail ? &dtail : &dmap, nrec * (REC / 4), 0, tail ? 0 : c, group0,
                                    wfull_s + 8 * wb);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer (leader CTA only) ========================================================
        // One thread, in order: whatever it executes between two turns leaves the tensor cores with
        // only the few MMAs still queued, so the loop is kept to a handful of instructions and takes
        // two K-steps (eight MMAs) per turn.  Units, parities and descriptors advance incrementally, and
        // the barriers of the NEXT turn are probed (without blocking) before this turn's MMAs are
        // issued: in the steady state the probe succeeds and the thread never executes a blocking wait.
        if (lane == 0 && rank == 0) {
            constexpr uint32_t kADescStep = kStageABytes >> 4, kBDescStep = kStageBBytes >> 4;
            constexpr int NB = GA / GB;                   // activation units taken per turn
            const uint64_t adesc0 = make_desc_sw128(a_s), bdesc0 = make_desc_sw128(b_s);
            auto advance = [](uint32_t &u, uint32_t &par, uint32_t units) {
                if (++u == units) u = 0, par ^= 1;
            };
            uint32_t ua = 0, pa = 0, ub = 0, pb = 0;      // unit and phase parity of the operands about to be used
            int tcount = 0;
            bool seen = false;                            // this turn's operands were found ready by the previous probe
            GEMM_TRACE_DECL(int it = 0;)
            for (int tile = pair; tile < p.pair_tiles; tile += n_pairs, ++tcount) {
                int stripe, t0, width;
                pair_tile(p, tile, stripe, t0, width);
                const uint32_t idesc = (1u << 4) | ((uint32_t)(width >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
                const int buf = tcount & 1;
                bool ok = pair_wait<true>(tempty_s + 8 * buf, ((tcount >> 1) & 1) ^ 1, sm, p.status);
                if (!ok) break;
                const uint32_t d_tmem = tmem_base + buf * kAccCols;
                for (int turn = 0; turn < ksteps / GA; ++turn) {
                    GEMM_TRACE(4 * it);
                    uint32_t ub1 = ub, pb1 = pb;          // second activation unit of the turn (NB == 2)
                    if (NB == 2) advance(ub1, pb1, UB);
                    if (!seen) {
                        ok = PAIR_DBG(2048) || (pair_wait<true>(bfull_s + 8 * ub, pb, sm, p.status) &&
                                                (NB == 1 || pair_wait<true>(bfull_s + 8 * ub1, pb1, sm, p.status)));
                        ok = ok && (PAIR_DBG(1024) || pair_wait<true>(afull_s + 8 * ua, pa, sm, p.status));
                        if (!ok) break;
                    }
                    GEMM_TRACE(4 * it + 1);
                    tc_fence_after();
                    uint32_t nua = ua, npa = pa, nub = ub1, npb = pb1;
                    advance(nua, npa, UA);
                    advance(nub, npb, UB);
                    if (NB == 2) {
                        uint32_t nub1 = nub, npb1 = npb;
                        advance(nub1, npb1, UB);
                        seen = mbar_test_wait_both(bfull_s + 8 * nub, npb, bfull_s + 8 * nub1, npb1) && mbar_test_wait(afull_s + 8 * nua, npa);
                    } else {
                        seen = mbar_test_wait_both(bfull_s + 8 * nub, npb, afull_s + 8 * nua, npa);
                    }
                    GEMM_TRACE(4 * it + 2);
#pragma unroll
                    for (int h = 0; h < GA; ++h) {
                        const uint32_t sa = GA * ua + h, sb = GB == 2 ? 2 * ub + h : (h == 0 ? ub : ub1);
                        const uint64_t adesc = adesc0 + sa * kADescStep, bdesc = bdesc0 + sb * kBDescStep;
#pragma unroll
                        for (int kk = 0; kk < BK / 16; ++kk) {     // 16 fp16 = 32 bytes = +2 in the address field
                            if (PAIR_DBG(8)) continue;
                            // TS: 16 fp16 of a row = 8 columns of its tensor-memory lane
                            if (TS) umma_f16_pair_ts(d_tmem, tmem_base + kTsACol0 + sa * 32 + 8 * kk, bdesc + 2 * kk, idesc, (turn | h | kk) != 0);
                            else umma_f16_pair(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (turn | h | kk) != 0);
                        }
                    }
                    if (!PAIR_DBG(1024)) umma_commit_pair(aempty_s + 8 * ua);
                    if (!PAIR_DBG(2048)) {
                        umma_commit_pair(bempty_s + 8 * ub);
                        if (NB == 2) umma_commit_pair(bempty_s + 8 * ub1);
                    }
                    GEMM_TRACE(4 * it + 3);
                    GEMM_TRACE_DECL(++it;)
                    ua = nua, pa = npa, ub = nub, pb = npb;
                }
                if (!ok) break;
                umma_commit_pair(tfull_s + 8 * buf);
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ===== dequant producers: this CTA's 128 weight rows =======================================
        const int t = threadIdx.x - kFirstDequantWarp * 32;
        // TS: a warp may only touch the tensor-memory lanes of its quadrant (warp index mod 4), so it takes those rows
        const int r = TS ? 32 * (warp & 3) + lane : t & (BM - 1), j = t >> 7;
        const int r7 = r & 7;
        const uint32_t row_off = (r >> 3) * 1024 + r7 * 128;
        const uint32_t afull_leader = mapa_rank(afull_s, 0);
        const int my_tiles = pair < p.pair_tiles ? (p.pair_tiles - pair + n_pairs - 1) / n_pairs : 0;
        const int total = my_tiles * p.nsb;
        bool ok = true;
        auto fetch = [&](int rs, Unit<QT> &u) {
            const int wb = rs % kWBufs;
            if (lane == 0) ok = pair_wait<true>(wfull_s + 8 * wb, (rs / kWBufs) & 1, sm, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) return;
            const int tcount = rs / p.nsb, sb = rs - tcount * p.nsb;
            const int cs = tcount * chunks_per_tile + (sb >> 3);
            u.load(w_s + wb * WBUF + r * REC, d_s + (cs & 1) * kDBufBytes + r * 16 + 2 * (sb & 7), j);
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty_s + 8 * wb);
        };
        Unit<QT> cur, nxt;
        if (total > 0) fetch(0, cur);
        const bool tracer = warp == kFirstDequantWarp && lane == 0;
        for (int rs = 0; rs < total && ok; ++rs) {
            if (tracer) GEMM_TRACE(8192 + 8 * rs);
            if (rs + 1 < total) {
                fetch(rs + 1, nxt);
                if (!ok) break;
            }
            if (tracer) GEMM_TRACE(8192 + 8 * rs + 1);
            uint32_t o[32];
            if (!PAIR_DBG(2)) cur.convert(j, o);
            // K-step 4 rs + j, and the stages are used round robin by K-step
            const int stage = (4 * rs + j) % SA_;
            const uint32_t use = (uint32_t)((4 * rs + j) / SA_);       // how often this stage has been filled before
            if (tracer) GEMM_TRACE(8192 + 8 * rs + 2);
            if (lane == 0 && !PAIR_DBG(1024)) ok = pair_wait<true>(aempty_s + 8 * (stage / GA), (use & 1) ^ 1, sm, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            if (tracer) GEMM_TRACE(8192 + 8 * rs + 3);
            if (TS) {
                tc_fence_after();      // the stage's previous reader (the tensor core) is done: ordered before these stores
                // the row's 64 values -> 32 columns of its lane; the MMA reads them once the stores have landed
                if (!PAIR_DBG(2)) tmem_st32(tmem_base + kTsACol0 + stage * 32 + ((uint32_t)(32 * (warp & 3)) << 16), o);
                if (tracer) GEMM_TRACE(8192 + 8 * rs + 4);
                tmem_st_wait();
                tc_fence_before();
            } else {
                if (!PAIR_DBG(2)) store_row(o, a_s + stage * kStageABytes + row_off, r7);
                if (tracer) GEMM_TRACE(8192 + 8 * rs + 4);
                fence_proxy_async();
            }
            if (tracer) GEMM_TRACE(8192 + 8 * rs + 5);
            __syncwarp();
            if (lane == 0 && !PAIR_DBG(1024)) {
                // the leader's own warps arrive locally; only the peer's arrival has to cross the pair
                if (rank == 0) mbar_arrive(afull_s + 8 * (stage / GA));
                else mbar_arrive_cluster(afull_leader + 8 * (stage / GA));
            }
            if (tracer) GEMM_TRACE(8192 + 8 * rs + 6);
            cur = nxt;
        }
    } else {
        // ===== epilogue: this CTA's 128 rows of the accumulator ====================================
        const int q = warp & 3;
        const uint32_t tempty_leader = mapa_rank(tempty_s, 0);
        int tcount = 0;
        for (int tile = pair; tile < p.pair_tiles; tile += n_pairs, ++tcount) {
            int stripe, t0, width;
            pair_tile(p, tile, stripe, t0, width);
            const int buf = tcount & 1;
            bool ok = pair_wait<false>(tfull_s + 8 * buf, (tcount >> 1) & 1, sm, p.status);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const int n = stripe * 2 * BM + (int)rank * BM + q * 32 + lane;
            const int m0 = t0;
            // lane = one output column n; its 32 accumulator columns per load are 32 consecutive tokens,
            // i.e. 32 stores one output row (ldy elements) apart: the pointer just steps by ldy
            const bool full_tile = m0 + width <= p.M;
            for (int c0 = 0; c0 < (PAIR_DBG(16) ? 0 : width); c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + buf * kAccCols + ((uint32_t)(q * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (n < p.N) {
                    if (p.y_is_bf16) {
                        __nv_bfloat16 *yp = reinterpret_cast<__nv_bfloat16 *>(p.y) + (long long)(m0 + c0) * p.ldy + n;
#pragma unroll
                        for (int i = 0; i < 32; ++i, yp += p.ldy)
                            if (full_tile || m0 + c0 + i < p.M) *yp = __float2bfloat16_rn(__uint_as_float(v[i]));
                    } else {
                        float *yp = reinterpret_cast<float *>(p.y) + (long long)(m0 + c0) * p.ldy + n;
#pragma unroll
                        for (int i = 0; i < 32; ++i, yp += p.ldy)
                            if (full_tile || m0 + c0 + i < p.M) *yp = __uint_as_float(v[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * buf);
        }
    }

    // both CTAs meet (also after an abort) before either releases shared or tensor memory
    tc_fence_before();
    __syncthreads();
    drain_after_abort(&sm->abort);
    cluster_sync_all();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// Activations -> fp16, the format the weights are dequantized to (both tensor-core operands must
// share one format), rounding to nearest even.  fp16 has three more mantissa bits than bf16 but a
// narrower exponent: bf16 values between 2^-14 and 65504 in magnitude convert exactly, larger ones
// saturate to +-65504, smaller ones lose bits as fp16 subnormals or flush to zero (below 2^-25).
__device__ __forceinline__ uint32_t to_h2_sat(float lo, float hi) {
    lo = fminf(fmaxf(lo, -65504.f), 65504.f);   // NaN passes through both
    hi = fminf(fmaxf(hi, -65504.f), 65504.f);
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <bool SRC_BF16>
__global__ void convert_x_kernel(const void *__restrict__ src, long long lds, uint16_t *__restrict__ dst,
                                 long long ldd, int M, int K) {
    const long long total = (long long)M * K;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / K, k = i - m * K;
        float v;
        if (SRC_BF16) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(src)[m * lds + k]);
        else v = reinterpret_cast<const float *>(src)[m * lds + k];
        dst[m * ldd + k] = (uint16_t)to_h2_sat(v, 0.f);
    }
}

// eight elements per thread with 16-byte accesses: K a multiple of 8, source rows 16-byte aligned
template <bool SRC_BF16>
__global__ void convert_x_vec8_kernel(const void *__restrict__ src, long long lds, uint16_t *__restrict__ dst,
                                      long long ldd, int M, int K8) {
    const unsigned total = (unsigned)M * (unsigned)K8;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned m = i / (unsigned)K8, c = i - m * (unsigned)K8;
        float f[8];
        if (SRC_BF16) {
            const uint4 v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(src) + (long long)m * lds + 8 * c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                f[2 * e] = __uint_as_float(w[e] << 16);
                f[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
            }
        } else {
            const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(src) + (long long)m * lds + 8 * c);
            const float4 b = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(src) + (long long)m * lds + 8 * c + 4);
            f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
        }
        uint4 o;
        o.x = to_h2_sat(f[0], f[1]);
        o.y = to_h2_sat(f[2], f[3]);
        o.z = to_h2_sat(f[4], f[5]);
        o.w = to_h2_sat(f[6], f[7]);
        *reinterpret_cast<uint4 *>(dst + (long long)m * ldd + 8 * c) = o;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn lookup_encode_fn() {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        return reinterpret_cast<EncodeTiledFn>(ptr);
    return nullptr;
}
EncodeTiledFn encode_fn() {
    static const EncodeTiledFn fn = lookup_encode_fn();     // initialised once, also under concurrent first calls
    return fn;
}

struct GemmMaps {
    CUtensorMap x, w, wtail, d, dtail;
};

template <int QT>
cudaError_t launch_gemm(const GemmParams &p, const GemmMaps &m, int grid, cudaStream_t st) {
    auto kern = gemm_tc_kernel<QT>;
    constexpr size_t smem = smem_data_bytes(QT) + sizeof(GemmSmem) + 1024;
    static_assert(smem <= 232448, "shared-memory plan exceeds the 227 KB a block may use");
    static std::atomic<int> configured_dev{-1};     // contexts on several threads may launch at once
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

template <int QT, bool TS>
cudaError_t launch_gemm_pair(const GemmParams &p, const GemmMaps &m, int grid, cudaStream_t st) {
    auto kern = gemm_tc_pair_kernel<QT, TS>;
    constexpr size_t smem = pair_smem_data_bytes(QT, TS) + sizeof(PairSmem) + 1024;
    static_assert(smem <= 232448, "shared-memory plan exceeds the 227 KB a block may use");
    static std::atomic<int> configured_dev{-1};     // contexts on several threads may launch at once
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != configured_dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, p, m.x, m.w, m.wtail, m.d, m.dtail);
}

// Number of tiles of the two-CTA kernel.  A K-step of this kernel costs about the same whatever
// the tile's width (the dequantization of the 128 x 64 weight block and its hand-over bound it,
// not the MMA), so the fewest, widest tiles win: every stripe is cut into ceil(units / 8) tiles of
// nearly equal width.
void pick_pair_tiles(GemmParams &p, int width_override, int max_units) {
    const int stripes = p.n_tiles, upr = p.units_per_row;
    int tps = (upr + max_units - 1) / max_units;
    if (width_override >= 32 && width_override <= 32 * max_units) tps = (upr + width_override / 32 - 1) / (width_override / 32);
    p.tps = tps;
    p.extra = 0;
    p.pair_tiles = stripes * tps;
}

// Token-tile width: with more tiles than SMs the last wave is partly idle, so a slightly narrower
// tile that fills the waves evenly can finish sooner.  Cost model: waves x (width + 90), the
// constant standing for the part of a K-step's time that does not shrink with the tile (measured:
// 0.46 us per K-step at 128 tokens, 0.69 us at 240); ties go to the wider tile.
int pick_bn(int M, int n_tiles, int sms, int widest) {
    if (M <= widest) return ((M + 15) / 16) * 16;
    int best = widest;
    long long best_cost = -1;
    for (int bn = widest; bn >= 128; bn -= 16) {
        const long long tiles = (long long)((M + bn - 1) / bn) * n_tiles;
        const long long waves = (tiles + sms - 1) / sms;
        const long long cost = waves * (bn + 90);
        if (best_cost < 0 || cost < best_cost) best_cost = cost, best = bn;
    }
    return best;
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

#ifdef B200Q_GEMM_TRACE
extern "C" int b200q_debug_gemm_trace(long long *out_16384) {
    return (int)cudaMemcpyFromSymbol(out_16384, g_gemm_trace, sizeof(long long) * 16384);
}
#endif

size_t gemm_x_scratch_bytes(int M, int K) { return ((size_t)M * ((K + 7) & ~7) * 2 + 255) & ~size_t(255); }

cudaError_t gemm_convert_x(const void *x, int x_is_bf16, long long ldx, void *scratch, int M, int K, cudaStream_t st) {
    const long long ldd = (K + 7) & ~7;
    uint16_t *dst = reinterpret_cast<uint16_t *>(scratch);
    const int esz = x_is_bf16 ? 2 : 4;
    const bool vec = K % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) && (ldx * esz) % 16 == 0 &&
                     (long long)M * (K / 8) < (1ll << 31);
    if (vec) {
        const long long total = (long long)M * (K / 8);
        const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 8);
        if (x_is_bf16) convert_x_vec8_kernel<true><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K / 8);
        else convert_x_vec8_kernel<false><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K / 8);
    } else {
        const long long total = (long long)M * K;
        const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 16);
        if (x_is_bf16) convert_x_kernel<true><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
        else convert_x_kernel<false><<<blocks, 256, 0, st>>>(x, ldx, dst, ldd, M, K);
    }
    return cudaGetLastError();
}

// x: fp16 activations [M][K] with leading dimension ldx
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
    p.n_tiles = (a.N + BM - 1) / BM;
    // large products run on CTA pairs (256-row tiles); small ones keep the one-CTA kernel
    const bool use_pair = a.pair && a.M >= 128 && a.N > BM && a.sm_count >= 2;
    const bool use_ts = use_pair && a.pair >= 2;          // A operand from tensor memory, token tiles up to 192
    if (use_pair) {
        p.n_tiles = (a.N + 2 * BM - 1) / (2 * BM);       // 256-row stripes
        p.units_per_row = (a.M + 31) / 32;
        p.bn = 256;
        pick_pair_tiles(p, a.bn_override, use_ts ? 6 : 8);
    } else {
        const int widest = bn_max(a.qt);
        p.bn = pick_bn(a.M, p.n_tiles, a.sm_count, widest);
        if (a.bn_override >= 16 && a.bn_override <= widest && a.bn_override % 16 == 0) p.bn = a.bn_override;
    }
    p.m_tiles = (a.M + p.bn - 1) / p.bn;
    p.status = a.status;
    p.debug = a.debug;

    GemmMaps maps;
    CUtensorMap &map = maps.x;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)(use_pair ? pair_b_rows(use_ts) : p.bn)};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(a.x), gdim, gstride, box, estride,
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
    p.ksplit = 1;
    p.part = nullptr;
    if (!use_pair && a.part && a.M < 128 && tiles * 2 <= a.sm_count) {
        // few tiles: cut K so that every SM gets a work unit (one round)
        int ks = std::min(p.nsb, a.sm_count / tiles);
        while (ks > 1 && (size_t)ks * a.M * a.N * sizeof(float) > a.part_bytes) --ks;
        if (ks > 1) {
            p.ksplit = ks;
            p.part = a.part;
        }
    }
    if (use_pair) {
        const int grid2 = 2 * std::min(p.pair_tiles, a.sm_count / 2);
        switch (a.qt) {
        case QT_Q4_K: return use_ts ? launch_gemm_pair<QT_Q4_K, true>(p, maps, grid2, st) : launch_gemm_pair<QT_Q4_K, false>(p, maps, grid2, st);
        case QT_Q5_K: return use_ts ? launch_gemm_pair<QT_Q5_K, true>(p, maps, grid2, st) : launch_gemm_pair<QT_Q5_K, false>(p, maps, grid2, st);
        case QT_Q4_0: return use_ts ? launch_gemm_pair<QT_Q4_0, true>(p, maps, grid2, st) : launch_gemm_pair<QT_Q4_0, false>(p, maps, grid2, st);
        case QT_MXFP4: return use_ts ? launch_gemm_pair<QT_MXFP4, true>(p, maps, grid2, st) : launch_gemm_pair<QT_MXFP4, false>(p, maps, grid2, st);
        case QT_Q6_K: return use_ts ? launch_gemm_pair<QT_Q6_K, true>(p, maps, grid2, st) : launch_gemm_pair<QT_Q6_K, false>(p, maps, grid2, st);
        case QT_Q8_0: return use_ts ? launch_gemm_pair<QT_Q8_0, true>(p, maps, grid2, st) : launch_gemm_pair<QT_Q8_0, false>(p, maps, grid2, st);
        default: return cudaErrorInvalidValue;
        }
    }
    const int grid = std::min(tiles * p.ksplit, a.sm_count);
    cudaError_t e;
    switch (a.qt) {
    case QT_Q4_K: e = launch_gemm<QT_Q4_K>(p, maps, grid, st); break;
    case QT_Q5_K: e = launch_gemm<QT_Q5_K>(p, maps, grid, st); break;
    case QT_Q4_0: e = launch_gemm<QT_Q4_0>(p, maps, grid, st); break;
    case QT_MXFP4: e = launch_gemm<QT_MXFP4>(p, maps, grid, st); break;
    case QT_Q6_K: e = launch_gemm<QT_Q6_K>(p, maps, grid, st); break;
    case QT_Q8_0: e = launch_gemm<QT_Q8_0>(p, maps, grid, st); break;
    default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || p.ksplit == 1) return e;
    const long long total = (long long)a.M * a.N;
    gemm_ksplit_sum_kernel<<<(int)std::min<long long>((total + 255) / 256, 148 * 4), 256, 0, st>>>(p.part, p.ksplit, a.M, a.N, a.y, a.ldy,
                                                                                             a.y_is_bf16);
    return cudaGetLastError();
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
    static std::atomic<void *> dev_ptr[kMaxDevices];     // zero-initialised; racing first calls store the same address
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!dev_ptr[dev].load()) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_x_scratch);
        if (e != cudaSuccess) return e;
        dev_ptr[dev] = ptr;
    }
    const long long ldd = (a.K + 7) & ~7;
    if ((size_t)a.M * (size_t)ldd > gemm_static_scratch_elems()) return cudaErrorInvalidValue;
    e = gemm_convert_x(a.x, x_is_bf16, a.ldx, dev_ptr[dev].load(), a.M, a.K, st);
    if (e != cudaSuccess) return e;
    a.x = dev_ptr[dev].load();
    a.ldx = ldd;
    return gemm_launch(a, st);
}

cudaError_t gemm_set_wait_limit_ns(unsigned long long ns) { return cudaMemcpyToSymbol(s_wait_limit_ns, &ns, sizeof(ns)); }

}  // namespace b200q
