// Skinny-batch product (2 <= M <= 16 activation rows; speculative-decode verify, small continuous
// batches): Y[m][n] = sum_k X[m][k] * dequant(W)[n][k], HBM-bound like the M = 1 kernel.
//
// The packed weights are read from HBM exactly once and never dequantized to a rounded format:
//   * work item = 16 weight rows x one chunk (8 superblock records = 2048 weights) of the streaming
//     layout.  A persistent CTA per SM owns a contiguous run of items (chunk-major, so most CTAs
//     stay inside one chunk); its producer warp streams them into a shared-memory ring, one bulk
//     copy per four-row group of the layout (four per item).  The groups are padded apart in shared
//     memory and MMA row f is row f >> 2 of group f & 3, so that the rows one fragment load touches
//     lie in four different groups and spread over the banks.
//   * 8 consumer warps; warp w owns record w of the chunk, i.e. a fixed 256-wide K range, for all
//     16 rows.  Its activations for that range (every token, exact bf16) stay in REGISTERS as
//     the B fragments of mma.sync.m16n8k16, loaded once per chunk straight from X (in the element
//     order the weight bytes dictate), so the hot loop reads nothing but the weights from shared
//     memory.  fp32 activations enter as two bf16 halves (two token slots per row).
//   * weights enter the tensor cores as exact small integers in bf16: the nibble / 6-bit value q
//     placed under the high byte 0x43 reads as the bf16 number 128 + q (one logic op per pair, no
//     conversion).  The MMA therefore returns sum (128 + q) x per sub-block in fp32; the epilogue
//     applies the sub-block's fp32 scale and folds the offset and the Q4_K minimum through the
//     per-sub-block sums of the activations:  acc += p * C - q * X,  (p, q) per (row, sub-block).
//     Q8_0 splits its byte into two nibble planes (128 + low, 2048 + 16 high) sharing the B fragment.
//     Nothing is rounded except in fp32, so results agree with the fp64 oracle to ~1e-6.
//   * the 8 warps' partial tiles (different K ranges of the same rows) go through a small ring in
//     shared memory to a "reducer" warp (two in the 16-token form, each taking half the token
//     pairs), which adds them in warp order and stores the item's sums; the consumers never meet
//     at a barrier.  When K spans several chunks the sums
//     of a chunk go to a workspace and a second, small launch adds the chunks in order (bit-
//     reproducible) and stores Y.
// Every mbarrier wait is bounded; a wait that runs out raises the status word and a flag that every
// role polls, copies in flight are awaited (again bounded) and the kernel returns.
#include <algorithm>
#include <atomic>
#include <new>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

#ifdef B200Q_SKINNY_TRACE
// timing experiments only: CTA 0 records its pipeline events into this array
__device__ unsigned long long g_sk_trace[4096];
#define SK_TRACE(slot) do { if (blockIdx.x == 0 && (slot) < 4096) g_sk_trace[(slot)] = (unsigned long long)clock64(); } while (0)
#else
#define SK_TRACE(slot) do { } while (0)
#endif

namespace {

constexpr int kSkWarps = 8;                       // consumer warps = records per chunk
// + the producer warp and one reducer warp per 8-token tile (a single reducer warp was the slowest
// role of the 16-token form)
__host__ __device__ constexpr int sk_threads(int nt) { return (kSkWarps + 1 + nt) * 32; }
constexpr int kSkRows = 16;                       // weight rows per item (MMA M)
constexpr int kSkMaxDepth = 12;
constexpr int kSkMaxCtas = 320;     // two CTAs per SM for the 8-token tile
#ifndef B200Q_SKINNY_CTAS_PER_SM
#define B200Q_SKINNY_CTAS_PER_SM 2
#endif
// CTAs per SM by token tile: the 16-token form's resident activation fragments leave registers for one
__host__ __device__ constexpr int sk_ctas_per_sm(int nt) { return nt == 1 ? B200Q_SKINNY_CTAS_PER_SM : 1; }
constexpr int kSkMaxJobs = 32;
constexpr int kSkInline = 4;                      // products whose descriptions travel in the kernel parameters
constexpr int kRedStride = 20;                    // floats between the tokens of a partial tile (bank spread)
constexpr int kRedDepth = 4;                      // partial-tile sets in flight between consumers and reducer

// bytes one row adds to a full chunk
__host__ __device__ constexpr int sk_chunk_row_bytes(int qt) { return qt == QT_Q6_K ? 1680 : rec_bytes(qt) * kChunkRecs; }
// shared-memory distance between the four-row groups of a stage: four rows of a full chunk, padded to
// 32 modulo 128.  The rows of a group lie as in device memory (one copy per group); the four rows a
// fragment-load phase touches come from the four groups at the same offset, i.e. 32 bytes apart
// modulo 128 (Q6_K reads 4-byte words: eight rows = four groups x two 16-byte steps).
__host__ __device__ constexpr int sk_group_stride(int qt) { return ((kRowGroup * sk_chunk_row_bytes(qt) - 32 + 127) / 128) * 128 + 32; }
__host__ __device__ constexpr int sk_subblocks(int qt) { return qt == QT_Q6_K ? 16 : 8; }   // scale blocks per record

struct SkJob {
    const uint8_t *w;          // streaming-layout weights
    const void *x;             // activations [M][K], bf16 or fp32
    void *y;
    float *part;               // [chunk][M][n_rb * 16] chunk sums (null when K is one chunk)
    long long ldx, ldy;
    int N, M, K, nsb, nchunks, n_rb, groups;
    int x_is_bf16, x_vec_ok;   // x_vec_ok: rows are 16-byte aligned (vector loads allowed)
    int crb_full, crb_tail;    // bytes one row adds to a full / the last chunk
    int y_is_bf16;
    int pairsum;               // tokens 8..15 hold the low halves of fp32 activations: y[m] = t[m] + t[m + 8]
    int item0;                 // first item of this job in the launch's item order
};

struct SkParams {
    const SkJob *jobs;         // device table, or null when the (at most kSkInline) jobs are in `inl`
    SkJob inl[kSkInline];
    int njobs;
    int depth;
    int *status;
    int begin[kSkMaxCtas + 1]; // items [begin[b], begin[b + 1]) belong to CTA b
};

struct SkHead {
    uint64_t full[kSkMaxDepth];
    uint64_t empty[kSkMaxDepth];
    uint64_t redfull[kRedDepth];
    uint64_t redempty[kRedDepth];
    int fail;                  // some wait ran out: every role leaves its loop
    SkJob jobs[kSkMaxJobs];
};
constexpr size_t kSkHeadBytes = (sizeof(SkHead) + 127) & ~size_t(127);

template <int QT, int NT> struct SkLayout {
    static constexpr int SBK = sk_subblocks(QT);
    static constexpr int GS = sk_group_stride(QT);
    static constexpr int kStageBytes = (kSkRows / kRowGroup) * GS;
    static_assert(GS >= kRowGroup * sk_chunk_row_bytes(QT) && GS % 128 == 32, "group stride");
    static constexpr int kRedFloats = 8 * NT * kRedStride;                    // one warp's partial tile
    static constexpr size_t kRedOff = kSkHeadBytes;
    static constexpr size_t kSctOff = kRedOff + size_t(kRedDepth) * kSkWarps * kRedFloats * 4;
    static constexpr size_t kXstOff = kSctOff + size_t(kSkWarps) * SBK * kSkRows * 8;
    static constexpr size_t kRingOff = (kXstOff + size_t(kSkWarps) * SBK * 8 * NT * 4 + 127) & ~size_t(127);
};

// Shared-memory reads of the hot loop are plain (non-volatile) asm so that the compiler may
// interleave them with the tensor-core instructions; their addresses are "laundered" through
// hold_after_wait() after the barrier wait that makes the data valid, and the results are pinned by
// keep_before() before the barrier arrival that gives the memory away.
__device__ __forceinline__ uint32_t ldsn32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 ldsn64(uint32_t a) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 ldsn128(uint32_t a) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 ldsn_f2(uint32_t a) {
    float2 v;
    asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t hold_after_wait(uint32_t a) {
    asm volatile("" : "+r"(a)::"memory");
    return a;
}
template <int NT> __device__ __forceinline__ void keep_before(float (&acc)[NT][4]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) asm volatile("" ::"f"(acc[nt][0]), "f"(acc[nt][1]), "f"(acc[nt][2]), "f"(acc[nt][3]) : "memory");
}
__device__ __forceinline__ void sts_f2(uint32_t a, float x, float y) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}

// D = A(16x16 bf16, row) * B(16x8 bf16, col) [+ D]
__device__ __forceinline__ void mma_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_more(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// bytes 0 and 2 of v (each a value below 128) as the bf16 pair (base + b0, base + b2); HI is the
// bf16 high byte twice (0x4300 = 128 with steps of 1, 0x4500 = 2048 with steps of 16)
template <uint32_t HI> __device__ __forceinline__ uint32_t pair02(uint32_t v) { return (v & 0x000F000Fu) | HI; }

// acc += p * c - q * X for the four accumulator elements of one token tile (q arrives negated)
__device__ __forceinline__ void fold(float (&acc)[4], const float (&c)[4], float2 pa, float2 pb, float2 X) {
    acc[0] = fmaf(pa.x, c[0], fmaf(pa.y, X.x, acc[0]));
    acc[1] = fmaf(pa.x, c[1], fmaf(pa.y, X.y, acc[1]));
    acc[2] = fmaf(pb.x, c[2], fmaf(pb.y, X.x, acc[2]));
    acc[3] = fmaf(pb.x, c[3], fmaf(pb.y, X.y, acc[3]));
}

// ---- per-type work on one record of 16 rows -----------------------------------------------------
// recA / recB: shared addresses of the record of rows g and g + 8; sct: this warp's (p, -q) table
// [sub-block][16 rows]; xst: this warp's activation sums [sub-block][token tile][8]; B: the fragments.
// Sub-blocks are taken QB at a time with QB * NT = 8 independent accumulator chains in flight, so
// the tensor-core latency of one chain hides behind the others.

// The (p, -q) table entries of a Q4_K / Q5_K header: lane L prepares row L >> 1, sub-blocks
// 4 (L & 1) .. + 3, with p = d sc and q = 128 p + dmin m.  The 6-bit fields are unpacked four at a
// time in the bytes of a word, the same way in every lane; a byte becomes a float through the 2^23
// form (one byte permute, one subtraction).
__device__ __forceinline__ void k_scale_table(uint32_t rec_row, int lane, uint32_t sct) {
    const int row = lane >> 1;
    const bool upper = lane & 1;
    const uint4 hdr = ldsn128(rec_row);       // d | dmin << 16, then the twelve scale bytes
    const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
    const uint32_t scw = upper ? ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u)) : (hdr.y & 0x3F3F3F3Fu);
    const uint32_t mnw = upper ? (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)) : (hdr.z & 0x3F3F3F3Fu);
    const uint32_t dst = sct + ((upper ? 4 : 0) * kSkRows + row) * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float sc = __uint_as_float(__byte_perm(scw, 0x4B000000u, 0x7440 + i)) - 8388608.f;
        const float mn = __uint_as_float(__byte_perm(mnw, 0x4B000000u, 0x7440 + i)) - 8388608.f;
        const float p = d * sc;
        sts_f2(dst + i * (kSkRows * 8), p, -fmaf(128.f, p, dmin * mn));
    }
}

template <int QT, int NT> struct SkRecord;

template <int NT> struct SkRecord<QT_Q4_K, NT> {
    static constexpr int QB = 8 / NT;
    // lane L prepares row L >> 1, sub-blocks 4 (L & 1) .. + 3: p = d sc, q = 128 p + dmin m
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t, int lane, uint32_t sct) {
        k_scale_table(rec_row, lane, sct);
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
        uint2 wa[4], wb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            wa[j] = ldsn64(recA + 16 + 32 * j + 8 * t);
            wb[j] = ldsn64(recB + 16 + 32 * j + 8 * t);
        }
#pragma unroll
        for (int b0 = 0; b0 < 8; b0 += QB) {
            float c[QB][NT][4];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
#pragma unroll
                for (int q = 0; q < QB; ++q) {
                    const int sb = b0 + q, j = sb >> 1, h = sb & 1;
                    uint32_t ra = s ? wa[j].y : wa[j].x, rb = s ? wb[j].y : wb[j].x;
                    if (h) ra >>= 4, rb >>= 4;
                    const uint32_t a0 = pair02<0x43004300u>(ra), a2 = pair02<0x43004300u>(ra >> 8);
                    const uint32_t a1 = pair02<0x43004300u>(rb), a3 = pair02<0x43004300u>(rb >> 8);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int bi = ((nt * 8 + sb) * 2 + s) * 2;
                        if (s == 0) mma_first(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                        else mma_more(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                const int sb = b0 + q;
                const float2 pa = ldsn_f2(sct + (sb * kSkRows + g) * 8), pb = ldsn_f2(sct + (sb * kSkRows + g + 8) * 8);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) fold(acc[nt], c[q][nt], pa, pb, ldsn_f2(xst + ((sb * NT + nt) * 8 + 2 * t) * 4));
            }
        }
    }
};

// Q5_K: the Q4_K record followed by 32 bytes of fifth bits; levels 0..31 still sit exactly in the bf16 form 128 + q
template <int NT> struct SkRecord<QT_Q5_K, NT> {
    static constexpr int QB = 8 / NT;
    // lane L prepares row L >> 1, sub-blocks 4 (L & 1) .. + 3: p = d sc, q = 128 p + dmin m
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t, int lane, uint32_t sct) {
        k_scale_table(rec_row, lane, sct);
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
        uint2 wa[4], wb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            wa[j] = ldsn64(recA + 16 + 32 * j + 8 * t);
            wb[j] = ldsn64(recB + 16 + 32 * j + 8 * t);
        }
        // fifth bits of this lane's eight positions: bit sb of a byte belongs to sub-block sb
        const uint2 fa = ldsn64(recA + 144 + 8 * t), fb = ldsn64(recB + 144 + 8 * t);
#pragma unroll
        for (int b0 = 0; b0 < 8; b0 += QB) {
            float c[QB][NT][4];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
#pragma unroll
                for (int q = 0; q < QB; ++q) {
                    const int sb = b0 + q, j = sb >> 1, h = sb & 1;
                    uint32_t ra = s ? wa[j].y : wa[j].x, rb = s ? wb[j].y : wb[j].x;
                    if (h) ra >>= 4, rb >>= 4;
                    const uint32_t ha = (s ? fa.y : fa.x) >> sb, hb = (s ? fb.y : fb.x) >> sb;
                    const uint32_t a0 = pair02<0x43004300u>(ra) | ((ha & 0x00010001u) << 4);
                    const uint32_t a2 = pair02<0x43004300u>(ra >> 8) | (((ha >> 8) & 0x00010001u) << 4);
                    const uint32_t a1 = pair02<0x43004300u>(rb) | ((hb & 0x00010001u) << 4);
                    const uint32_t a3 = pair02<0x43004300u>(rb >> 8) | (((hb >> 8) & 0x00010001u) << 4);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int bi = ((nt * 8 + sb) * 2 + s) * 2;
                        if (s == 0) mma_first(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                        else mma_more(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                const int sb = b0 + q;
                const float2 pa = ldsn_f2(sct + (sb * kSkRows + g) * 8), pb = ldsn_f2(sct + (sb * kSkRows + g + 8) * 8);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) fold(acc[nt], c[q][nt], pa, pb, ldsn_f2(xst + ((sb * NT + nt) * 8 + 2 * t) * 4));
            }
        }
    }
};

// Q4_0: [8 x fp16 d][nibbles in the Q4_K arrangement]; w = d (q - 8): p = d, the X term carries 128 + 8
template <int NT> struct SkRecord<QT_Q4_0, NT> {
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t, int lane, uint32_t sct) {
        const int row = lane >> 1, half = lane & 1;
        const uint2 dd = ldsn64(rec_row + 8 * half);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t wv = i < 2 ? dd.x : dd.y;
            const float d = half_bits_to_float(wv >> (16 * (i & 1)));
            sts_f2(sct + ((4 * half + i) * kSkRows + row) * 8, d, -136.f * d);
        }
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
        SkRecord<QT_Q4_K, NT>::run(recA, recB, g, t, B, sct, xst, acc);
    }
};

// MXFP4: [8 scale bytes, 8 of padding][per block four words of eight e2m1 codes in weight order].  A look-up
// gives the bytes 64 + value, which sit exactly in the bf16 form 128 + b: p = 2^(e - 128), the X term carries 192.
template <int NT> struct SkRecord<QT_MXFP4, NT> {
    static constexpr int QB = 8 / NT;
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t, int lane, uint32_t sct) {
        const int row = lane >> 1, half = lane & 1;
        const uint32_t ee = ldsn32(rec_row + 4 * half);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float d = __uint_as_float(e8m0_half_bits((ee >> (8 * i)) & 0xFF));
            sts_f2(sct + ((4 * half + i) * kSkRows + row) * 8, d, -192.f * d);
        }
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
#pragma unroll
        for (int b0 = 0; b0 < 8; b0 += QB) {
            uint32_t wa[QB], wb[QB];     // lane t: the codes of weights 8t .. 8t + 7 of each block
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                wa[q] = ldsn32(recA + 16 + 16 * (b0 + q) + 4 * t);
                wb[q] = ldsn32(recB + 16 + 16 * (b0 + q) + 4 * t);
            }
            float c[QB][NT][4];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
#pragma unroll
                for (int q = 0; q < QB; ++q) {
                    const int sb = b0 + q;
                    const uint32_t ba = mxfp4_bytes(wa[q] >> (16 * s)), bb = mxfp4_bytes(wb[q] >> (16 * s));
                    // (b0, b2) and (b1, b3) as bf16 pairs 128 + b
                    const uint32_t a0 = __byte_perm(ba, 0x43434343u, 0x4240), a2 = __byte_perm(ba, 0x43434343u, 0x4341);
                    const uint32_t a1 = __byte_perm(bb, 0x43434343u, 0x4240), a3 = __byte_perm(bb, 0x43434343u, 0x4341);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int bi = ((nt * 8 + sb) * 2 + s) * 2;
                        if (s == 0) mma_first(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                        else mma_more(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                const int sb = b0 + q;
                const float2 pa = ldsn_f2(sct + (sb * kSkRows + g) * 8), pb = ldsn_f2(sct + (sb * kSkRows + g + 8) * 8);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) fold(acc[nt], c[q][nt], pa, pb, ldsn_f2(xst + ((sb * NT + nt) * 8 + 2 * t) * 4));
            }
        }
    }
};

template <int NT> struct SkRecord<QT_Q8_0, NT> {
    static constexpr int QB = 8 / NT;
    // record = [8 x 32 int8][8 x fp16 d]; p = d, q = 2304 d (128 for the sign flip, 128 + 2048 for the two planes)
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t, int lane, uint32_t sct) {
        const int row = lane >> 1, half = lane & 1;
        const uint2 dd = ldsn64(rec_row + 256 + 8 * half);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t wv = i < 2 ? dd.x : dd.y;
            const float d = half_bits_to_float(wv >> (16 * (i & 1)));
            sts_f2(sct + ((4 * half + i) * kSkRows + row) * 8, d, -2304.f * d);
        }
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
#pragma unroll
        for (int b0 = 0; b0 < 8; b0 += QB) {
            uint2 wa[QB], wb[QB];
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                wa[q] = ldsn64(recA + 32 * (b0 + q) + 8 * t);
                wb[q] = ldsn64(recB + 32 * (b0 + q) + 8 * t);
                wa[q].x ^= 0x80808080u, wa[q].y ^= 0x80808080u, wb[q].x ^= 0x80808080u, wb[q].y ^= 0x80808080u;   // q + 128 = 16 hi + lo
            }
            float c[QB][NT][4];
#pragma unroll
            for (int s = 0; s < 2; ++s) {
#pragma unroll
                for (int plane = 0; plane < 2; ++plane) {
#pragma unroll
                    for (int q = 0; q < QB; ++q) {
                        const int sb = b0 + q;
                        const uint32_t ra = s ? wa[q].y : wa[q].x, rb = s ? wb[q].y : wb[q].x;
                        uint32_t a0, a1, a2, a3;
                        if (plane == 0) {
                            a0 = pair02<0x43004300u>(ra), a2 = pair02<0x43004300u>(ra >> 8);
                            a1 = pair02<0x43004300u>(rb), a3 = pair02<0x43004300u>(rb >> 8);
                        } else {
                            a0 = pair02<0x45004500u>(ra >> 4), a2 = pair02<0x45004500u>(ra >> 12);
                            a1 = pair02<0x45004500u>(rb >> 4), a3 = pair02<0x45004500u>(rb >> 12);
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const int bi = ((nt * 8 + sb) * 2 + s) * 2;
                            if (s == 0 && plane == 0) mma_first(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                            else mma_more(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < QB; ++q) {
                const int sb = b0 + q;
                const float2 pa = ldsn_f2(sct + (sb * kSkRows + g) * 8), pb = ldsn_f2(sct + (sb * kSkRows + g + 8) * 8);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) fold(acc[nt], c[q][nt], pa, pb, ldsn_f2(xst + ((sb * NT + nt) * 8 + 2 * t) * 4));
            }
        }
    }
};

template <int NT> struct SkRecord<QT_Q6_K, NT> {
    static constexpr int QB = 8 / NT;
    // record = [ql 128][qh 64][16 int8 scales], the row's fp16 d at d_row; sub-blocks of 16 weights:
    // p = d sc, q = 160 p (128 from the bf16 trick, 32 from the format's offset)
    static __device__ __forceinline__ void scales(uint32_t rec_row, uint32_t d_row, int lane, uint32_t sct) {
        const int row = lane >> 1, half = lane & 1;
        const uint2 s8 = ldsn64(rec_row + 192 + 8 * half);
        const float d = half_bits_to_float(ldsn32(d_row & ~3u) >> (8 * (d_row & 2)));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t wv = i < 4 ? s8.x : s8.y;
            const float p = d * (float)(int)(int8_t)(wv >> (8 * (i & 3)));
            sts_f2(sct + ((8 * half + i) * kSkRows + row) * 8, p, -160.f * p);
        }
    }
    // 6-bit values of four weights: low nibbles (after shift) of lw, bit pair `qd` of hw
    static __device__ __forceinline__ uint32_t six(uint32_t lw, uint32_t hw, int qd) {
        const uint32_t lo = (qd >= 2 ? lw >> 4 : lw) & 0x0F0F0F0Fu;
        const uint32_t hb = qd == 0 ? hw << 4 : qd == 1 ? hw << 2 : qd == 2 ? hw : hw >> 2;
        return lo | (hb & 0x30303030u);
    }
    static __device__ __forceinline__ void run(uint32_t recA, uint32_t recB, int g, int t, const uint32_t (&B)[32 * NT],
                                               uint32_t sct, uint32_t xst, float (&acc)[NT][4]) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            uint32_t la[4], lb[4], ha[2], hb[2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                la[i] = ldsn32(recA + 64 * hf + 16 * i + 4 * t);
                lb[i] = ldsn32(recB + 64 * hf + 16 * i + 4 * t);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                ha[i] = ldsn32(recA + 128 + 32 * hf + 16 * i + 4 * t);
                hb[i] = ldsn32(recB + 128 + 32 * hf + 16 * i + 4 * t);
            }
#pragma unroll
            for (int b0 = 0; b0 < 8; b0 += QB) {
                float c[QB][NT][4];
#pragma unroll
                for (int q = 0; q < QB; ++q) {
                    const int qd = (b0 + q) >> 1, bb = (b0 + q) & 1, sb = 8 * hf + b0 + q;
                    // weights 128 hf + 32 qd + 16 bb + 4 t .. + 3: ql byte 64 hf + 32 (qd & 1) + 16 bb + 4 t, nibble qd >> 1
                    const uint32_t va = six(la[2 * (qd & 1) + bb], ha[bb], qd), vb = six(lb[2 * (qd & 1) + bb], hb[bb], qd);
                    const uint32_t a0 = __byte_perm(va, 0x43434343u, 0x4140), a2 = __byte_perm(va, 0x43434343u, 0x4342);
                    const uint32_t a1 = __byte_perm(vb, 0x43434343u, 0x4140), a3 = __byte_perm(vb, 0x43434343u, 0x4342);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int bi = (nt * 8 + (sb >> 1)) * 4 + 2 * (sb & 1);
                        mma_first(c[q][nt], a0, a1, a2, a3, B[bi], B[bi + 1]);
                    }
                }
#pragma unroll
                for (int q = 0; q < QB; ++q) {
                    const int sb = 8 * hf + b0 + q;
                    const float2 pa = ldsn_f2(sct + (sb * kSkRows + g) * 8), pb = ldsn_f2(sct + (sb * kSkRows + g + 8) * 8);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) fold(acc[nt], c[q][nt], pa, pb, ldsn_f2(xst + ((sb * NT + nt) * 8 + 2 * t) * 4));
                }
            }
        }
    }
};

// Walks a CTA's items in order: (job, chunk, row block) of the current item, stepped without dividing.
struct SkCursor {
    int ji, c, rb;
    __device__ __forceinline__ void start(const SkJob *jobs, int njobs, int it) {
        ji = 0;
        while (ji + 1 < njobs && it >= jobs[ji + 1].item0) ++ji;
        const int local = it - jobs[ji].item0;
        c = local / jobs[ji].n_rb;
        rb = local - c * jobs[ji].n_rb;
    }
    __device__ __forceinline__ void next(const SkJob *jobs) {
        if (++rb == jobs[ji].n_rb) {
            rb = 0;
            if (++c == jobs[ji].nchunks) c = 0, ++ji;
        }
    }
};

// This warp's B fragments and activation sums for record `rec` of the row, straight from X.
// Q4_K / Q8_0: per 32-weight block sb, lane (g, t) holds the eight values x0..x7 at 32 sb + 8 t of
// token slot g as the pairs (x0, x2) (x1, x3) | (x4, x6) (x5, x7) - the order in which the bytes of a
// weight word meet them.  Q6_K: per 16-weight block, four values at 16 sb + 4 t in natural order.
template <int QT, int NT>
__device__ __forceinline__ void sk_load_b(const SkJob &J, int rec, int g, int t, uint32_t (&B)[32 * NT], float *xst_p) {
    constexpr bool Q6 = QT == QT_Q6_K;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int tok = J.pairsum ? g : nt * 8 + g;
        const bool low_part = J.pairsum && nt == 1;
        const bool valid = tok < J.M;
        // all loads of the tile are issued before the first value is used (one trip to L2, not eight)
        uint32_t w4[8][4];      // per run pair v: bf16 pairs (x0 x1) (x2 x3) | (x4 x5) (x6 x7)
        if (J.x_is_bf16 && J.x_vec_ok) {
            const __nv_bfloat16 *xr = reinterpret_cast<const __nv_bfloat16 *>(J.x) + (long long)tok * J.ldx;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                // two runs of four values: Q6_K blocks 2 v and 2 v + 1, otherwise the halves of block v's eight
                const int kA = rec * SB + (Q6 ? 32 * v + 4 * t : 32 * v + 8 * t);
                const bool in = valid && kA < J.K;
                if (Q6) {
                    const uint2 a = in ? __ldcg(reinterpret_cast<const uint2 *>(xr + kA)) : make_uint2(0, 0);
                    const uint2 b = in ? __ldcg(reinterpret_cast<const uint2 *>(xr + kA + 16)) : make_uint2(0, 0);
                    w4[v][0] = a.x, w4[v][1] = a.y, w4[v][2] = b.x, w4[v][3] = b.y;
                } else {
                    const uint4 a = in ? __ldcg(reinterpret_cast<const uint4 *>(xr + kA)) : make_uint4(0, 0, 0, 0);
                    w4[v][0] = a.x, w4[v][1] = a.y, w4[v][2] = a.z, w4[v][3] = a.w;
                }
            }
        } else {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const int kA = rec * SB + (Q6 ? 32 * v + 4 * t : 32 * v + 8 * t);
                const int kB = Q6 ? kA + 16 : kA + 4;
#pragma unroll
                for (int i = 0; i < 4; ++i) w4[v][i] = 0;
                if (valid && kA < J.K) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int k = (i < 4 ? kA : kB - 4) + i;
                        uint32_t bits;
                        if (J.x_is_bf16) {
                            bits = reinterpret_cast<const unsigned short *>(J.x)[(long long)tok * J.ldx + k];
                        } else {
                            const float f = reinterpret_cast<const float *>(J.x)[(long long)tok * J.ldx + k];
                            bits = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                            if (low_part) bits = __bfloat16_as_ushort(__float2bfloat16_rn(f - __uint_as_float(bits << 16)));
                        }
                        w4[v][i >> 1] |= bits << (16 * (i & 1));
                    }
                }
            }
        }
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            float s0 = (__uint_as_float(w4[v][0] << 16) + __uint_as_float(w4[v][0] & 0xFFFF0000u)) +
                       (__uint_as_float(w4[v][1] << 16) + __uint_as_float(w4[v][1] & 0xFFFF0000u));
            float s1 = (__uint_as_float(w4[v][2] << 16) + __uint_as_float(w4[v][2] & 0xFFFF0000u)) +
                       (__uint_as_float(w4[v][3] << 16) + __uint_as_float(w4[v][3] & 0xFFFF0000u));
            const int bi = (nt * 8 + v) * 4;
            if (Q6) {
                B[bi] = w4[v][0], B[bi + 1] = w4[v][1], B[bi + 2] = w4[v][2], B[bi + 3] = w4[v][3];
            } else {
                B[bi] = __byte_perm(w4[v][0], w4[v][1], 0x5410), B[bi + 1] = __byte_perm(w4[v][0], w4[v][1], 0x7632);
                B[bi + 2] = __byte_perm(w4[v][2], w4[v][3], 0x5410), B[bi + 3] = __byte_perm(w4[v][2], w4[v][3], 0x7632);
                s0 += s1;
            }
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 1);
            s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 2);
            if (Q6) {
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
                s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 2);
            }
            if (t == 0) {
                if (Q6) {
                    xst_p[((2 * v) * NT + nt) * 8 + g] = s0;
                    xst_p[((2 * v + 1) * NT + nt) * 8 + g] = s1;
                } else {
                    xst_p[(v * NT + nt) * 8 + g] = s0;
                }
            }
        }
    }
}

// one bounded wait of a role; on expiry (or when another role already gave up) the role leaves
__device__ __forceinline__ bool sk_wait(uint32_t bar, uint32_t parity, volatile int *fail_flag, int *status) {
    if (*fail_flag) return false;
    if (mbar_wait_bounded_fast(bar, parity)) return true;
    atomicMax(status, DEV_ERR_PIPE_TIMEOUT);
    *fail_flag = 1;
    return false;
}

template <int QT, int NT>
__global__ void __launch_bounds__(sk_threads(NT), sk_ctas_per_sm(NT)) skinny_kernel(const __grid_constant__ SkParams p) {
    using L = SkLayout<QT, NT>;
    constexpr int SBK = L::SBK, GS = L::GS;
    extern __shared__ __align__(128) uint8_t smem[];
    SkHead &head = *reinterpret_cast<SkHead *>(smem);
    const uint32_t full0 = smem_u32(head.full), empty0 = smem_u32(head.empty);
    const uint32_t rfull0 = smem_u32(head.redfull), rempty0 = smem_u32(head.redempty);
    const uint32_t ring0 = smem_u32(smem + L::kRingOff);
    float *red = reinterpret_cast<float *>(smem + L::kRedOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.depth;
    const int it_begin = p.begin[blockIdx.x], it_end = p.begin[blockIdx.x + 1];

    if (threadIdx.x == 0) {
        for (int i = 0; i < D; ++i) {
            mbar_init(full0 + 8 * i, 1);
            mbar_init(empty0 + 8 * i, kSkWarps);
        }
        for (int i = 0; i < kRedDepth; ++i) {
            mbar_init(rfull0 + 8 * i, kSkWarps);
            mbar_init(rempty0 + 8 * i, NT);
        }
        head.fail = 0;
        mbar_fence_init();
        fence_proxy_async();
    }
    {   // job table -> shared memory
        const int words = p.njobs * (int)(sizeof(SkJob) / 4);
        const int *src = p.jobs ? reinterpret_cast<const int *>(p.jobs) : reinterpret_cast<const int *>(&p.inl[0]);
        int *dst = reinterpret_cast<int *>(head.jobs);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = src[i];
    }
    pdl_launch_dependents();
    __syncthreads();
    if (threadIdx.x == 0) SK_TRACE(0);
    const SkJob *jobs = head.jobs;
    volatile int *fail_flag = &head.fail;

    // ===== producer: lane q copies row group q (four rows) of every item of this CTA into the ring ===
    if (warp == kSkWarps) {
        int n = 0, slot = 0;
        uint32_t phase = 0;        // parity of the ring pass in progress (no division in the loop)
        SkCursor cur;
        cur.start(jobs, p.njobs, it_begin);
        for (int it = it_begin; it < it_end; ++it, ++n, cur.next(jobs)) {
            const int c = cur.c, rb = cur.rb;
            const SkJob &J = jobs[cur.ji];
            bool ok = true;
            if (n >= D) {
                if (lane == 0) ok = sk_wait(empty0 + 8 * slot, phase ^ 1u, fail_flag, p.status);
                ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            }
            if (!ok) break;
            const uint32_t crb = (c == J.nchunks - 1) ? (uint32_t)J.crb_tail : (uint32_t)J.crb_full;
            const int ng = min(kSkRows / kRowGroup, J.groups - rb * (kSkRows / kRowGroup));     // groups present in device memory
            const uint32_t bar = full0 + 8 * slot;
            if (lane == 0) {
                fence_proxy_async();     // the consumers' reads of this slot precede the copy engine's writes
                mbar_expect_tx(bar, ng * kRowGroup * crb);
            }
            __syncwarp();
            if (lane < ng) {
                const uint8_t *src = J.w + tile_off(QT, rb * (kSkRows / kRowGroup) + lane, c, 0, J.nsb);
                bulk_g2s(ring0 + slot * L::kStageBytes + lane * GS, src, kRowGroup * crb, bar);
            }
            if (lane == 0) SK_TRACE(10 + (n & 63));
            if (++slot == D) slot = 0, phase ^= 1u;
        }
        // After a failure the consumers may have stopped short of the copies already issued: those must
        // land before the CTA's shared memory is released.  (A slot whose phase has long completed
        // answers at once.)
        if (*fail_flag && lane == 0)
            for (int k = max(0, n - D); k < n; ++k)
                if (!mbar_wait_bounded(full0 + 8 * (k % D), (uint32_t)(k / D) & 1u)) break;
        return;
    }

    // ===== reducers: add the eight warps' partial tiles of every item and store the item's sums; =====
    // ===== reducer r takes the token pairs i = r, r + NT, ... of the tile                        =====
    if (warp > kSkWarps) {
        const int r = warp - (kSkWarps + 1);
        int n = 0;
        bool waited = false;
        SkCursor cur;
        cur.start(jobs, p.njobs, it_begin);
        for (int it = it_begin; it < it_end; ++it, ++n, cur.next(jobs)) {
            const int c = cur.c, rb = cur.rb;
            const SkJob &J = jobs[cur.ji];
            const int nrec = min(kChunkRecs, J.nsb - c * kChunkRecs);
            const int rs = n % kRedDepth;
            bool ok = true;
            if (lane == 0) ok = sk_wait(rfull0 + 8 * rs, (uint32_t)(n / kRedDepth) & 1u, fail_flag, p.status);
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) break;
            if (!waited) {       // outputs and the workspace belong to earlier launches until they have finished
                pdl_wait();
                waited = true;
            }
            const float *rbase = red + (size_t)rs * kSkWarps * L::kRedFloats;
            const size_t npad = (size_t)J.n_rb * kSkRows;
            const int row = lane & 15;                                           // MMA row of the partial tiles
            const int grow = rb * kSkRows + (row & 3) * kRowGroup + (row >> 2);    // = row (row >> 2) of group (row & 3)
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const int i = ii * NT + r;
                const int tok = 2 * i + (lane >> 4);      // element (tok, row): tok * 16 + row = lane + 32 i
                if (tok >= J.M) continue;
                const float *rsrc = rbase + tok * kRedStride + row;
                float tv[kSkWarps], v = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < kSkWarps; ++w2) tv[w2] = w2 < nrec ? rsrc[w2 * L::kRedFloats] : 0.f;
#pragma unroll
                for (int w2 = 0; w2 < kSkWarps; ++w2) v += tv[w2];
                if (NT == 2 && J.pairsum) {
#pragma unroll
                    for (int w2 = 0; w2 < kSkWarps; ++w2) tv[w2] = w2 < nrec ? rsrc[w2 * L::kRedFloats + 8 * kRedStride] : 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < kSkWarps; ++w2) v += tv[w2];
                }
                if (J.nchunks > 1) {
                    J.part[((size_t)c * J.M + tok) * npad + grow] = v;
                } else if (grow < J.N) {
                    const long long idx = (long long)tok * J.ldy + grow;
                    if (J.y_is_bf16) reinterpret_cast<__nv_bfloat16 *>(J.y)[idx] = __float2bfloat16_rn(v);
                    else reinterpret_cast<float *>(J.y)[idx] = v;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(rempty0 + 8 * rs);
            if (lane == 0) SK_TRACE(300 + (n & 63));
        }
        return;
    }

    // ===== consumers ==================================================================================
    const int g = lane >> 2, t = lane & 3;
    const uint32_t sct0 = smem_u32(smem + L::kSctOff) + warp * (SBK * kSkRows * 8);
    float *xst_p = reinterpret_cast<float *>(smem + L::kXstOff) + warp * (SBK * 8 * NT);
    uint32_t xst = smem_u32(xst_p);
    uint32_t B[32 * NT];
#pragma unroll
    for (int i = 0; i < 32 * NT; ++i) B[i] = 0;
    int cur_key = -1, n = 0, slot = 0;
    uint32_t phase = 0;
    SkCursor cur;
    cur.start(jobs, p.njobs, it_begin);
    if (threadIdx.x == 0) SK_TRACE(100);
    pdl_wait();     // the activations (written by an earlier launch) are visible from here
    if (threadIdx.x == 0) SK_TRACE(101);

#pragma unroll 1
    for (int it = it_begin; it < it_end; ++it, ++n, cur.next(jobs)) {
        const int c = cur.c;
        const SkJob &J = jobs[cur.ji];
        const int nrec = min(kChunkRecs, J.nsb - c * kChunkRecs);
        const bool active = warp < nrec;
        if (cur.ji * 65536 + c != cur_key) {     // a new K range: this warp's activation fragments and sums
            cur_key = cur.ji * 65536 + c;
            __syncwarp();
            if (active) sk_load_b<QT, NT>(J, c * kChunkRecs + warp, g, t, B, xst_p);
            __syncwarp();
            xst = hold_after_wait(smem_u32(xst_p));
        }
        bool ok = sk_wait(full0 + 8 * slot, phase, fail_flag, p.status);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        if (threadIdx.x == 0) SK_TRACE(200 + 4 * (n & 31));
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
        if (active) {
            const uint32_t stage = hold_after_wait(ring0 + slot * L::kStageBytes);
            const uint32_t crb = (c == J.nchunks - 1) ? (uint32_t)J.crb_tail : (uint32_t)J.crb_full;
            const uint32_t roff = QT == QT_Q6_K ? warp * 208 : warp * rec_bytes(QT);
            const uint32_t doff = nrec * 208 + 2 * warp;                      // Q6_K: the row's fp16 d of this record
            // MMA row f lies in group f & 3 as its row f >> 2
            const uint32_t srow = stage + ((lane >> 1) & 3) * GS + (lane >> 3) * crb;
            SkRecord<QT, NT>::scales(srow + roff, srow + doff, lane, sct0);
            __syncwarp();
            const uint32_t sct = hold_after_wait(sct0);
            const uint32_t recA = stage + (g & 3) * GS + (g >> 2) * crb + roff;
            SkRecord<QT, NT>::run(recA, recA + 2 * crb, g, t, B, sct, xst, acc);
            keep_before<NT>(acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * slot);
        if (threadIdx.x == 0) SK_TRACE(201 + 4 * (n & 31));
        if (++slot == D) slot = 0, phase ^= 1u;

        // this warp's partial tile [token][row] -> the reducer
        const int rs = n % kRedDepth;
        if (n >= kRedDepth) {
            ok = sk_wait(rempty0 + 8 * rs, ((uint32_t)(n / kRedDepth) & 1u) ^ 1u, fail_flag, p.status);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
        }
        if (active) {
            float *rd = red + ((size_t)rs * kSkWarps + warp) * L::kRedFloats;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                rd[(nt * 8 + 2 * t) * kRedStride + g] = acc[nt][0];
                rd[(nt * 8 + 2 * t + 1) * kRedStride + g] = acc[nt][1];
                rd[(nt * 8 + 2 * t) * kRedStride + g + 8] = acc[nt][2];
                rd[(nt * 8 + 2 * t + 1) * kRedStride + g + 8] = acc[nt][3];
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(rfull0 + 8 * rs);
        if (threadIdx.x == 0) SK_TRACE(202 + 4 * (n & 31));
    }
    if (threadIdx.x == 0) SK_TRACE(900);
}

// Y = sum over chunks of the chunk sums, in chunk order, for every product of the set whose K spans
// several chunks.  Launched right behind skinny_kernel (programmatic stream serialization).
__global__ void __launch_bounds__(256) skinny_chunk_sum_kernel(const __grid_constant__ SkParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if (p.njobs <= kSkInline) {        // a call's few products, one after another: one output per thread and pass
        for (int ji = 0; ji < p.njobs; ++ji) {
            const SkJob &J = p.jobs ? p.jobs[ji] : p.inl[ji];
            if (J.nchunks <= 1) continue;
            const size_t npad = (size_t)J.n_rb * kSkRows;
            const int total = J.M * J.N;
            for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
                const int tok = e / J.N, row = e - tok * J.N;
                float v = 0.f;
                for (int cc = 0; cc < J.nchunks; ++cc) v += __ldcg(&J.part[((size_t)cc * J.M + tok) * npad + row]);
                const long long idx = (long long)tok * J.ldy + row;
                if (J.y_is_bf16) reinterpret_cast<__nv_bfloat16 *>(J.y)[idx] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(J.y)[idx] = v;
            }
        }
        return;
    }
    // A plan's many products share the grid side by side (a share of the blocks each), and a thread
    // reads the chunk sums of several outputs before it stores the first: taken one after another,
    // every product and every output would cost a trip to L2.
    constexpr int U = 4;
    const int bpj = max(1, (int)gridDim.x / p.njobs);          // blocks per product
    for (int slot = blockIdx.x; slot < p.njobs * bpj; slot += gridDim.x) {
        const int ji = slot / bpj, lb = slot - ji * bpj;
        const SkJob &J = p.jobs[ji];
        if (J.nchunks <= 1) continue;
        const size_t npad = (size_t)J.n_rb * kSkRows;
        const int total = J.M * J.N, stride = bpj * blockDim.x;
        for (int e0 = lb * blockDim.x + threadIdx.x; e0 < total; e0 += U * stride) {
            float v[U];
            long long idx[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int e = e0 + u * stride;
                v[u] = 0.f;
                idx[u] = -1;
                if (e < total) {
                    const int tok = e / J.N, row = e - tok * J.N;
                    idx[u] = (long long)tok * J.ldy + row;
#pragma unroll 2
                    for (int cc = 0; cc < J.nchunks; ++cc) v[u] += __ldcg(&J.part[((size_t)cc * J.M + tok) * npad + row]);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (idx[u] >= 0) {
                    if (J.y_is_bf16) reinterpret_cast<__nv_bfloat16 *>(J.y)[idx[u]] = __float2bfloat16_rn(v[u]);
                    else reinterpret_cast<float *>(J.y)[idx[u]] = v[u];
                }
            }
        }
    }
}

template <int QT, int NT>
cudaError_t sk_launch_t(const SkParams &p, int grid, size_t smem_limit, cudaStream_t st) {
    using L = SkLayout<QT, NT>;
    SkParams q = p;
    // co-resident CTAs share the SM's shared memory (1 KB per CTA is the system's)
    constexpr int kPerSm = sk_ctas_per_sm(NT);
    if (kPerSm > 1) smem_limit = (smem_limit + 1024) / kPerSm - 1024;
    int depth = (int)((smem_limit - L::kRingOff) / L::kStageBytes);
    if (depth > kSkMaxDepth) depth = kSkMaxDepth;
    if (depth < 2) return cudaErrorInvalidValue;
    q.depth = depth;
    const size_t smem = L::kRingOff + (size_t)depth * L::kStageBytes;
    auto kern = skinny_kernel<QT, NT>;
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
    cfg.blockDim = dim3(sk_threads(NT));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, q);
}

}  // namespace

int skinny_max_m() { return 16; }

size_t skinny_part_bytes(const SkinnyProduct &a) {
    const size_t nchunks = ((size_t)a.Kpad / SB + kChunkRecs - 1) / kChunkRecs;
    if (nchunks <= 1) return 0;
    const size_t n_rb = (padded_rows(a.N) / kRowGroup + 3) / 4;
    return ((nchunks * a.M * n_rb * kSkRows * sizeof(float)) + 255) & ~size_t(255);
}

// A prepared call: the kernel parameters of `n` products of one block type and one M (fp32
// activations: M <= 8) and the CTA partition.  Built once (per call, or per plan) on the host;
// launching it touches no host memory the caller could have freed.
struct SkinnySet {
    SkParams p;
    int qt = 0, NT = 1, grid = 0, sum_grid = 0;
    size_t smem_limit = 0;
};

cudaError_t skinny_set_create(const SkinnyProduct *prods, int n, const SkinnyBuffers &buf, SkinnySet **out) {
    if (!out) return cudaErrorInvalidValue;
    *out = nullptr;
    if (n < 1 || n > kSkMaxJobs || !prods) return cudaErrorInvalidValue;
    const int M = prods[0].M, qt = prods[0].qt;
    const bool any_f32 = !prods[0].x_is_bf16;
    if (M < 1 || M > 16 || (any_f32 && M > 8)) return cudaErrorInvalidValue;
    const int NT = (M > 8 || any_f32) ? 2 : 1;
    SkinnySet *set = new (std::nothrow) SkinnySet();
    if (!set) return cudaErrorMemoryAllocation;
    SkParams &p = set->p;
    p = SkParams{};
    std::vector<SkJob> jobs((size_t)n);
    size_t ws_off = 0;
    int items = 0;
    long long sum_elems = 0;
    auto bad = [&]() {
        delete set;
        return cudaErrorInvalidValue;
    };
    for (int i = 0; i < n; ++i) {
        const SkinnyProduct &a = prods[i];
        if (a.qt != qt || a.M != M || (!a.x_is_bf16) != any_f32 || a.N < 1 || a.K < 1) return bad();
        SkJob &J = jobs[i];
        J = SkJob{};
        J.w = a.w;
        J.x = a.x;
        J.ldx = a.ldx;
        J.x_is_bf16 = a.x_is_bf16;
        J.x_vec_ok = a.x_is_bf16 && !(reinterpret_cast<uintptr_t>(a.x) & 15) && (a.ldx * 2) % 16 == 0;
        J.y = a.y;
        J.ldy = a.ldy;
        J.N = a.N;
        J.M = M;
        J.K = a.K;
        J.nsb = a.Kpad / SB;
        J.nchunks = (J.nsb + kChunkRecs - 1) / kChunkRecs;
        J.groups = (int)(padded_rows(a.N) / kRowGroup);
        J.n_rb = (J.groups + 3) / 4;
        J.crb_full = (int)chunk_row_bytes(qt, 0, J.nsb);
        J.crb_tail = (int)chunk_row_bytes(qt, J.nchunks - 1, J.nsb);
        J.y_is_bf16 = a.y_is_bf16;
        J.pairsum = any_f32 ? 1 : 0;
        J.item0 = items;
        items += J.nchunks * J.n_rb;
        if (J.nchunks > 1) {
            if (ws_off + skinny_part_bytes(a) > buf.ws_bytes) return bad();
            J.part = reinterpret_cast<float *>(buf.ws + ws_off);
            ws_off += skinny_part_bytes(a);
            sum_elems += (long long)M * a.N;
        }
    }
    // contiguous runs of items of (nearly) equal weight per CTA; an item's weight is its chunk's
    // record count plus a constant for the per-item work that does not shrink with a short chunk
    const int grid = std::min(std::min(buf.sm_count * sk_ctas_per_sm(NT), kSkMaxCtas), items);
    {
        double total = 0;
        for (const SkJob &J : jobs)
            for (int c = 0; c < J.nchunks; ++c) total += (double)J.n_rb * (std::min(kChunkRecs, J.nsb - c * kChunkRecs) + 2);
        int b = 1;
        double cum = 0;
        p.begin[0] = 0;
        for (const SkJob &J : jobs) {
            for (int c = 0; c < J.nchunks && b < grid; ++c) {
                const double wt = std::min(kChunkRecs, J.nsb - c * kChunkRecs) + 2;
                const double blk_end = cum + wt * J.n_rb;
                while (b < grid && total * b / grid < blk_end) {
                    const double target = total * b / grid;
                    int idx = (int)((target - cum) / wt + 0.5);
                    idx = std::max(0, std::min(idx, J.n_rb));
                    p.begin[b] = std::max(p.begin[b - 1], J.item0 + c * J.n_rb + idx);
                    ++b;
                }
                cum = blk_end;
            }
        }
        for (; b < grid; ++b) p.begin[b] = items;
        p.begin[grid] = items;
    }
    p.njobs = n;
    p.status = buf.status;
    if (n <= kSkInline) {
        p.jobs = nullptr;
        for (int i = 0; i < n; ++i) p.inl[i] = jobs[i];
    } else {
        if (!buf.jobs_dev) return bad();
        cudaError_t e = cudaMemcpy(buf.jobs_dev, jobs.data(), sizeof(SkJob) * (size_t)n, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            delete set;
            return e;
        }
        p.jobs = reinterpret_cast<const SkJob *>(buf.jobs_dev);
    }
    set->qt = qt;
    set->NT = NT;
    set->grid = grid;
    set->sum_grid = sum_elems > 0 ? (int)std::min<long long>((sum_elems + 255) / 256, (n <= kSkInline ? 2LL : 8LL) * buf.sm_count) : 0;
    set->smem_limit = buf.smem_limit;
    *out = set;
    return cudaSuccess;
}

void skinny_set_destroy(SkinnySet *set) { delete set; }

// The product launch, then (when some K spans several chunks) the chunk-sum launch; both with
// programmatic stream serialization.
cudaError_t skinny_set_launch(const SkinnySet *set, cudaStream_t st) {
    if (!set) return cudaErrorInvalidValue;
    cudaError_t e;
    switch (set->qt * 4 + set->NT) {
    case QT_Q4_K * 4 + 1: e = sk_launch_t<QT_Q4_K, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q4_K * 4 + 2: e = sk_launch_t<QT_Q4_K, 2>(set->p, set->grid, set->smem_limit, st); break;
    case QT_MXFP4 * 4 + 1: e = sk_launch_t<QT_MXFP4, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_MXFP4 * 4 + 2: e = sk_launch_t<QT_MXFP4, 2>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q4_0 * 4 + 1: e = sk_launch_t<QT_Q4_0, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q4_0 * 4 + 2: e = sk_launch_t<QT_Q4_0, 2>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q5_K * 4 + 1: e = sk_launch_t<QT_Q5_K, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q5_K * 4 + 2: e = sk_launch_t<QT_Q5_K, 2>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q6_K * 4 + 1: e = sk_launch_t<QT_Q6_K, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q6_K * 4 + 2: e = sk_launch_t<QT_Q6_K, 2>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q8_0 * 4 + 1: e = sk_launch_t<QT_Q8_0, 1>(set->p, set->grid, set->smem_limit, st); break;
    case QT_Q8_0 * 4 + 2: e = sk_launch_t<QT_Q8_0, 2>(set->p, set->grid, set->smem_limit, st); break;
    default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || set->sum_grid == 0) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)set->sum_grid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, skinny_chunk_sum_kernel, set->p);
}

int skinny_set_launches(const SkinnySet *set) { return set ? 1 + (set->sum_grid > 0 ? 1 : 0) : 0; }

cudaError_t skinny_run(const SkinnyProduct *prods, int n, const SkinnyBuffers &buf, cudaStream_t st, int *launches) {
    if (n > kSkInline) return cudaErrorInvalidValue;     // larger sets go through a plan, whose job table is uploaded once
    SkinnySet *set = nullptr;
    cudaError_t e = skinny_set_create(prods, n, buf, &set);
    if (e != cudaSuccess) return e;
    e = skinny_set_launch(set, st);
    if (launches) *launches += skinny_set_launches(set);
    skinny_set_destroy(set);
    return e;
}

#ifdef B200Q_SKINNY_TRACE
extern "C" int b200q_debug_skinny_trace(unsigned long long *out_4096) {
    return (int)cudaMemcpyFromSymbol(out_4096, g_sk_trace, sizeof(unsigned long long) * 4096);
}
#endif

size_t skinny_job_table_bytes() { return sizeof(SkJob) * kSkMaxJobs; }
int skinny_max_products() { return kSkMaxJobs; }

cudaError_t skinny_set_wait_limit_ns(unsigned long long ns) { return cudaMemcpyToSymbol(s_wait_limit_ns, &ns, sizeof(ns)); }

}  // namespace b200q
