// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200q {

// ---- layout.cu ------------------------------------------------------------------------------
// Host: re-lay GGUF rows [r0, r1) x superblocks [sb0, sb1) of a tensor into the streaming layout.
// K is the full tensor's row length; dst receives (r1-r0) rows of row_bytes_for(qt, sb1-sb0).
void repack_host(int qt, int64_t K, const uint8_t *gguf, int64_t r0, int64_t r1, int64_t sb0,
                 int64_t sb1, uint8_t *dst);
// Device: fp32 values of rows of a streaming-layout weight (bit-exact, no fused multiply-add).
cudaError_t dequant_launch(int qt, const uint8_t *w, int64_t N, int64_t K, int64_t Kpad,
                           int64_t row_bytes, float *out, cudaStream_t st);

// ---- gemv.cu --------------------------------------------------------------------------------
struct GemvLaunch {
    int qt;
    int nseg;                 // 1..4 weights sharing x
    const uint8_t *w[4];
    void *y[4];
    long long ldy[4];
    int n[4];
    const void *x;
    long long ldx;
    int x_is_bf16, y_is_bf16;
    int M;                    // 1..4
    int K, Kpad;
    long long row_bytes;
    int *status;              // device status word
    int sm_count;
    size_t smem_limit;        // opt-in shared memory per block
    size_t smem_sm;           // shared memory per SM
    int pdl;                  // launch with programmatic stream serialization
    int warps, depth, grid;   // 0 = default
    int rows_per_item;        // 0 = choose, else 2 or 4
    int debug;                // experiments only (see gemv.cu)
};
int gemv_max_m();
cudaError_t gemv_launch(const GemvLaunch &a, cudaStream_t st);

}  // namespace b200q
