// Streaming-layout conversion (host) and bit-exact dequantization (device).
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

void repack_host(int qt, int64_t K, const uint8_t *gguf, int64_t r0, int64_t n, int64_t sb0,
                 int64_t sb1, uint8_t *dst, int64_t ra, int64_t rb) {
    const int64_t src_row = K / gguf_block_elems(qt) * gguf_block_bytes(qt);
    const int64_t nsb = sb1 - sb0;
    for (int64_t r = ra; r < rb; ++r) {   // r: row of the shard, r0 + r: row of the full tensor
        const uint8_t *s = gguf + (r0 + r) * src_row;
        for (int64_t sb = 0; sb < nsb; ++sb) {
            uint8_t *rec = dst + record_off(qt, r, sb, n, nsb);
            if (qt == QT_Q4_K) {
                memcpy(rec, s + (sb0 + sb) * 144, 144);
            } else if (qt == QT_Q5_K) {
                // [d dmin scales | nibbles | fifth bits]: the first 144 bytes read like a Q4_K record
                const uint8_t *blk = s + (sb0 + sb) * 176;
                memcpy(rec, blk, 16);
                memcpy(rec + 16, blk + 48, 128);
                memcpy(rec + 144, blk + 16, 32);
            } else if (qt == QT_Q4_0) {
                // eight native blocks -> [8 x fp16 d][128 bytes of nibbles in the Q4_K arrangement: block 2j in the
                // low nibbles of bytes 32j .. 32j + 31, block 2j + 1 in their high nibbles]; K padding: zero blocks
                const int64_t nblk = K / 32;
                memset(rec, 0, 144);
                for (int b = 0; b < 8; ++b) {
                    const int64_t blk = (sb0 + sb) * 8 + b;
                    if (blk >= nblk) continue;
                    const uint8_t *src = s + blk * 18;
                    memcpy(rec + 2 * b, src, 2);
                    uint8_t *q = rec + 16 + 32 * (b >> 1);
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t v = l < 16 ? (src[2 + l] & 0xF) : (src[2 + l - 16] >> 4);
                        q[l] |= (b & 1) ? (uint8_t)(v << 4) : v;
                    }
                }
            } else if (qt == QT_MXFP4) {
                // eight native blocks -> [8 scale bytes][8 zero bytes][per block four words of eight codes each, code n
                // of word i = weight 8 i + n]: the order a table look-up by prmt wants; K padding: zero codes
                const int64_t nblk = K / 32;
                memset(rec, 0, 144);
                for (int b = 0; b < 8; ++b) {
                    const int64_t blk = (sb0 + sb) * 8 + b;
                    if (blk >= nblk) continue;
                    const uint8_t *src = s + blk * 17;
                    rec[b] = src[0];
                    uint8_t *q = rec + 16 + 16 * b;
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t v = l < 16 ? (src[1 + l] & 0xF) : (src[1 + l - 16] >> 4);
                        q[l >> 1] |= (l & 1) ? (uint8_t)(v << 4) : v;
                    }
                }
            } else if (qt == QT_Q8_0) {
                const int64_t nblk = K / 32;
                for (int b = 0; b < 8; ++b) {
                    const int64_t blk = (sb0 + sb) * 8 + b;
                    if (blk < nblk) {
                        memcpy(rec + 32 * b, s + blk * 34 + 2, 32);
                        memcpy(rec + 256 + 2 * b, s + blk * 34, 2);
                    } else {   // K padding: zero blocks contribute nothing
                        memset(rec + 32 * b, 0, 32);
                        memset(rec + 256 + 2 * b, 0, 2);
                    }
                }
            } else {
                const uint8_t *blk = s + (sb0 + sb) * 210;
                memcpy(rec, blk, 208);
                memcpy(dst + q6k_d_record_off(r, sb, n, nsb), blk + 208, 2);
            }
        }
    }
}

namespace {

// One CTA per (row, superblock record); thread t produces weight t of the record.
template <int QT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ w, int64_t N, int64_t K,
                                                      int nsb, float *__restrict__ out) {
    const int sb = blockIdx.x % nsb;
    const int64_t row = blockIdx.x / nsb;
    const int t = threadIdx.x;
    const int64_t k = (int64_t)sb * 256 + t;
    if (k >= K) return;
    float v;
    if (QT == QT_Q4_K || QT == QT_Q5_K) {
        const uint8_t *rec = w + record_off(QT, row, sb, N, nsb);
        const uint32_t *hw = reinterpret_cast<const uint32_t *>(rec);
        const float d = half_bits_to_float(hw[0]), dmin = half_bits_to_float(hw[0] >> 16);
        int sc, mn;
        q4k_scale_min(hw[1], hw[2], hw[3], t >> 5, sc, mn);
        const uint8_t byte = rec[16 + 32 * (t >> 6) + (t & 31)];
        int q = (t & 32) ? (byte >> 4) : (byte & 0xF);
        if (QT == QT_Q5_K) q += ((rec[144 + (t & 31)] >> (t >> 5)) & 1) << 4;      // bit j of byte l: sub-block j, weight l
        const float d1 = __fmul_rn(d, (float)sc);
        const float m1 = __fmul_rn(dmin, (float)mn);
        v = __fsub_rn(__fmul_rn(d1, (float)q), m1);
    } else if (QT == QT_Q4_0) {
        const uint8_t *rec = w + record_off(QT, row, sb, N, nsb);
        const int b = t >> 5;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rec + 2 * b));
        const uint8_t byte = rec[16 + 32 * (b >> 1) + (t & 31)];
        const int q = (b & 1) ? (byte >> 4) : (byte & 0xF);
        v = __fmul_rn((float)(q - 8), d);
    } else if (QT == QT_MXFP4) {
        const uint8_t *rec = w + record_off(QT, row, sb, N, nsb);
        const int b = t >> 5, l = t & 31;
        const float d = __uint_as_float(e8m0_half_bits(rec[b]));
        const uint8_t byte = rec[16 + 16 * b + (l >> 1)];
        const int code = (l & 1) ? (byte >> 4) : (byte & 0xF);
        const int mag = (0x0C08060403020100ull >> (8 * (code & 7))) & 0xFF;
        v = __fmul_rn((float)((code & 8) ? -mag : mag), d);
    } else if (QT == QT_Q8_0) {
        const uint8_t *rec = w + record_off(QT, row, sb, N, nsb);
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(rec + 256 + 2 * (t >> 5)));
        const int q = (int)(int8_t)rec[t];
        v = __fmul_rn(d, (float)q);
    } else {
        const uint8_t *rec = w + record_off(QT, row, sb, N, nsb);
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(w + q6k_d_record_off(row, sb, N, nsb)));
        const int h = t >> 7, l = t & 127, c = l >> 5, pos = l & 31;
        const uint8_t qlb = rec[64 * h + 32 * (c & 1) + pos];
        const uint8_t qhb = rec[128 + 32 * h + pos];
        const int q = (int)(((c & 2) ? (qlb >> 4) : (qlb & 0xF)) | (((qhb >> (2 * c)) & 3) << 4)) - 32;
        const int sc = (int)(int8_t)rec[192 + (t >> 4)];
        v = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
    out[row * K + k] = v;
}

}  // namespace

cudaError_t dequant_launch(int qt, const uint8_t *w, int64_t N, int64_t K, int64_t Kpad,
                           int64_t row_bytes, float *out, cudaStream_t st) {
    const int nsb = (int)(Kpad / SB);
    const int64_t blocks = N * nsb;
    if (blocks == 0) return cudaSuccess;
    if (blocks > 0x7FFFFFFF) return cudaErrorInvalidValue;
    switch (qt) {
    case QT_Q4_K: dequant_kernel<QT_Q4_K><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    case QT_Q5_K: dequant_kernel<QT_Q5_K><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    case QT_Q8_0: dequant_kernel<QT_Q8_0><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    case QT_Q4_0: dequant_kernel<QT_Q4_0><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    case QT_MXFP4: dequant_kernel<QT_MXFP4><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    case QT_Q6_K: dequant_kernel<QT_Q6_K><<<(unsigned)blocks, 256, 0, st>>>(w, N, K, nsb, out); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace b200q
