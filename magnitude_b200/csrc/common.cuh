// Shared definitions for the b200q kernels: the device ("streaming") weight layout, PTX
// wrappers for mbarrier / bulk-copy / dp4a, and the status codes kernels can raise.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

// ---------------------------------------------------------------------------------------------
// Streaming layout.
//
// A weight W[N][K] is cut into "superblock records" of 256 weights (Kpad = K rounded up to 256;
// only Q8_0 can need padding, its pad blocks are d = 0, q = 0):
//
//   Q4_K : the native 144-byte block                    [d:2][dmin:2][scales:12][qs:128]
//   Q8_0 : eight native 34-byte blocks regrouped as     [qs:8x32][d:8x2]            = 272 bytes
//   Q6_K : the native 210-byte block without its d      [ql:128][qh:64][scales:16]  = 208 bytes,
//          and after every eight records ("octet") one 16-byte group of their eight fp16 d
//          (a trailing partial octet of r records is r*208 + 16 bytes).
//
// Records are stored tile by tile.  A tile is a group of kRowGroup = 4 consecutive rows x one
// chunk of kChunkRecs = 8 consecutive records: inside a row group the chunks follow each other,
// and inside a chunk the group's rows follow each other.  One tile (4 rows x 2048 weights, 4.5 KB
// for Q4_K) is therefore one contiguous, 16-byte aligned byte range, which the streaming kernels
// fetch with a single bulk copy.  The tensor is padded with zero rows to a multiple of 4 rows, so
// every row group is whole and tiles sit at regular strides (which also lets a tiled TMA
// descriptor address them); the last chunk of a row may hold fewer than 8 records.
//
// The byte count equals GGUF's except for the Q8_0 K padding and at most 14 bytes per Q6_K row.
// ---------------------------------------------------------------------------------------------

enum : int { QT_Q4_0 = B200Q_TYPE_Q4_0, QT_Q8_0 = B200Q_TYPE_Q8_0, QT_Q4_K = B200Q_TYPE_Q4_K, QT_Q5_K = B200Q_TYPE_Q5_K, QT_Q6_K = B200Q_TYPE_Q6_K, QT_MXFP4 = B200Q_TYPE_MXFP4 };

constexpr int SB = 256;  // weights per superblock record

__host__ __device__ constexpr int rec_bytes(int qt) {
    return (qt == QT_Q4_K || qt == QT_Q4_0 || qt == QT_MXFP4) ? 144 : qt == QT_Q5_K ? 176 : qt == QT_Q8_0 ? 272 : 208;
}
__host__ __device__ constexpr int gguf_block_elems(int qt) { return (qt == QT_Q8_0 || qt == QT_Q4_0 || qt == QT_MXFP4) ? 32 : 256; }
__host__ __device__ constexpr int gguf_block_bytes(int qt) {
    return qt == QT_Q4_K ? 144 : qt == QT_Q5_K ? 176 : qt == QT_Q8_0 ? 34 : qt == QT_Q4_0 ? 18 : qt == QT_MXFP4 ? 17 : 210;
}

// byte offset of superblock record `sb` inside a row
__host__ __device__ inline int64_t rec_off(int qt, int64_t sb) {
    if (qt == QT_Q6_K) return (sb >> 3) * 1680 + (sb & 7) * 208;
    return sb * rec_bytes(qt);
}
// byte offset of the fp16 d of Q6_K superblock `sb` (nsb = records in the row)
__host__ __device__ inline int64_t q6k_d_off(int64_t sb, int64_t nsb) {
    int64_t base = sb & ~int64_t(7);
    int64_t in_octet = nsb - base < 8 ? nsb - base : 8;
    return (sb >> 3) * 1680 + in_octet * 208 + 2 * (sb & 7);
}
// bytes of a row of nsb records; also the offset of the end of record range [0, nsb)
__host__ __device__ inline int64_t row_bytes_for(int qt, int64_t nsb) {
    if (qt == QT_Q6_K) return (nsb >> 3) * 1680 + ((nsb & 7) ? (nsb & 7) * 208 + 16 : 0);
    return nsb * rec_bytes(qt);
}
// bytes of the contiguous record range [sb0, sb1) of a row (sb0 a multiple of 8 for Q6_K)
__host__ __device__ inline int64_t range_bytes(int qt, int64_t sb0, int64_t sb1, int64_t nsb) {
    int64_t end = (sb1 >= nsb) ? row_bytes_for(qt, nsb) : rec_off(qt, sb1);
    return end - rec_off(qt, sb0);
}

constexpr int kRowGroup = 4;    // rows per tile
constexpr int kChunkRecs = 8;   // records per tile row

// bytes one row contributes to chunk c (records [8c, min(8c+8, nsb)))
__host__ __device__ inline int64_t chunk_row_bytes(int qt, int64_t c, int64_t nsb) {
    const int64_t sb1 = (c + 1) * kChunkRecs < nsb ? (c + 1) * kChunkRecs : nsb;
    return range_bytes(qt, c * kChunkRecs, sb1, nsb);
}
// rows of row group g that exist in an N-row tensor (the rest of the group is zero padding)
__host__ __device__ inline int group_rows(int64_t g, int64_t N) {
    const int64_t left = N - g * kRowGroup;
    return left < kRowGroup ? (int)left : kRowGroup;
}
// rows a tensor of N rows occupies in device memory
__host__ __device__ inline int64_t padded_rows(int64_t N) { return (N + kRowGroup - 1) / kRowGroup * kRowGroup; }
// byte offset of tile (row group g, chunk c) from the start of the tensor
__host__ __device__ inline int64_t tile_off(int qt, int64_t g, int64_t c, int64_t, int64_t nsb) {
    return g * kRowGroup * row_bytes_for(qt, nsb) + kRowGroup * rec_off(qt, c * kChunkRecs);
}
// byte offset of record `sb` of row `row` (for Q6_K: of its 208-byte part)
__host__ __device__ inline int64_t record_off(int qt, int64_t row, int64_t sb, int64_t N, int64_t nsb) {
    const int64_t g = row / kRowGroup, c = sb / kChunkRecs;
    return tile_off(qt, g, c, N, nsb) + (row - g * kRowGroup) * chunk_row_bytes(qt, c, nsb) +
           (rec_off(qt, sb) - rec_off(qt, c * kChunkRecs));
}
// byte offset of the fp16 d of Q6_K record `sb` of row `row`
__host__ __device__ inline int64_t q6k_d_record_off(int64_t row, int64_t sb, int64_t N, int64_t nsb) {
    const int64_t g = row / kRowGroup, c = sb / kChunkRecs;
    return tile_off(QT_Q6_K, g, c, N, nsb) + (row - g * kRowGroup) * chunk_row_bytes(QT_Q6_K, c, nsb) +
           (q6k_d_off(sb, nsb) - rec_off(QT_Q6_K, c * kChunkRecs));
}

// MXFP4 helpers.  Scale byte e (e8m0) -> 2^(e - 128), the halved scale ggml pairs with its doubled e2m1
// values {0, 1, 2, 3, 4, 6, 8, 12} and their negatives (codes 8..15).
__host__ __device__ inline uint32_t e8m0_half_bits(uint32_t e) { return e < 2 ? (0x00200000u << e) : ((e - 1) << 23); }
#ifdef __CUDACC__
// four e2m1 codes (the four nibbles of sel's low 16 bits) -> four bytes 64 + value, by table look-up:
// prmt copies a table byte, or, when the selector nibble's bit 3 is set, replicates that byte's top
// bit (0 here): non-negative codes hit the first table, negative ones (sign bit flipped) the second.
__device__ __forceinline__ uint32_t mxfp4_bytes(uint32_t sel) {
    uint32_t pos, neg;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(pos) : "r"(0x43424140u), "r"(0x4C484644u), "r"(sel));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(neg) : "r"(0x3D3E3F40u), "r"(0x34383A3Cu), "r"(sel ^ 0x8888u));
    return pos | neg;
}
#endif

// Device status word values (atomicMax'ed, so larger = more severe).
enum : int {
    DEV_OK = 0,
    DEV_ERR_PIPE_TIMEOUT = 1,   // a bounded mbarrier wait ran out
    DEV_ERR_TMEM = 2,           // tensor-memory allocation handshake failed
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// non-blocking probe (try_wait may suspend the thread for a while; a polling loop that serves
// several barriers must not)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// both barriers' phases complete?  One instruction sequence, so the two probes' latencies overlap.
__device__ __forceinline__ bool mbar_test_wait_both(uint32_t bar0, uint32_t parity0, uint32_t bar1, uint32_t parity1) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
        "and.pred p, p, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar0), "r"(parity0), "r"(bar1), "r"(parity1)
        : "memory");
    return ok != 0;
}

// Wait limit for every device-side spin: after this long the waiter gives up, raises the status
// word and the kernel drains and returns instead of hanging the GPU.  A variable (one copy per
// source file and device; the context option B200Q_OPT_WAIT_LIMIT_MS sets them all) so that a host
// can choose its own deadline and a test can make a wait run out quickly.
static __device__ unsigned long long s_wait_limit_ns = 2000000000ull;
#define kWaitLimitNs s_wait_limit_ns

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
    }
}

// try_wait with a cap (ns) on how long the hardware may keep the thread suspended.  Without the hint
// a suspended waiter may resume only about a microsecond after the phase completes, which is most
// of an item's time in the pipelines that wait once per item.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// bounded wait for waits on a pipeline's critical path: re-checks every few dozen nanoseconds
__device__ __forceinline__ bool mbar_wait_bounded_fast(uint32_t bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < (1 << 12); ++i)
        if (mbar_try_wait_hint(bar, parity, 32)) return true;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbar_try_wait_hint(bar, parity, 64)) return true;
        if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.  No cluster multicast anywhere.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Shared-memory reads go through 32-bit shared-window addresses: the hot loop then spends no
// instructions on 64-bit pointer arithmetic.  (volatile keeps them after the barrier waits.)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs; it must call pdl_wait() before it
// reads anything the predecessor writes or writes anything the predecessor may still read.
// Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// dp4a: d = c + sum_i a.b[i] * b.b[i] with per-operand signedness
__device__ __forceinline__ int dp4a_us(uint32_t a_u8, uint32_t b_s8, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_s8), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a_u8, uint32_t b_u8, int c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_u8), "r"((uint32_t)c));
    return (int)d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a_s8, uint32_t b_s8, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_s8), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a_s8, uint32_t b_u8, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_u8), "r"(c));
    return d;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half((unsigned short)(h16 & 0xFFFFu)));
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// Q4_K 6-bit scale / min of sub-block `is` (0..7) from the three scale words of the header.
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int is, int &sc,
                                              int &mn) {
    // bytes 0..3 = s0, 4..7 = s1, 8..11 = s2
    if (is < 4) {
        sc = (s0 >> (8 * is)) & 63;
        mn = (s1 >> (8 * is)) & 63;
    } else {
        const int sh = 8 * (is - 4);
        const uint32_t a = (s2 >> sh) & 0xFF, lo = (s0 >> sh) & 0xFF, hi = (s1 >> sh) & 0xFF;
        sc = (a & 0xF) | ((lo >> 6) << 4);
        mn = (a >> 4) | ((hi >> 6) << 4);
    }
}

}  // namespace b200q
