// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200q {

// ---- device wait limit (one variable per source file with bounded waits; all set together) --------
cudaError_t gemv_set_wait_limit_ns(unsigned long long ns);
cudaError_t skinny_set_wait_limit_ns(unsigned long long ns);
cudaError_t gemm_set_wait_limit_ns(unsigned long long ns);
cudaError_t peer_set_wait_limit_ns(unsigned long long ns);

// ---- layout.cu ------------------------------------------------------------------------------
// Host: re-lay rows [r0, r0 + n) x superblocks [sb0, sb1) of a GGUF tensor (row length K) into the
// streaming layout at dst (n * row_bytes_for(qt, sb1 - sb0) bytes).  Only shard rows [ra, rb) are
// written, so several threads can share one call's work.
void repack_host(int qt, int64_t K, const uint8_t *gguf, int64_t r0, int64_t n, int64_t sb0,
                 int64_t sb1, uint8_t *dst, int64_t ra, int64_t rb);
// Device: fp32 values of rows of a streaming-layout weight (bit-exact, no fused multiply-add).
cudaError_t dequant_launch(int qt, const uint8_t *w, int64_t N, int64_t K, int64_t Kpad,
                           int64_t row_bytes, float *out, cudaStream_t st);

// ---- gemv.cu --------------------------------------------------------------------------------
// The streaming kernel runs a list of jobs in one launch.  A job is 1..4 weights of one type and
// K applied to one activation (M <= 4 rows, the same M for every job of a launch).
constexpr int kStreamMaxSeg = 4;
enum : int {
    STREAM_JOB_WAITS = 1,       // the job reads what earlier jobs of the launch wrote
    STREAM_JOB_SUM_RANKS = 2,   // the job's outputs are summed over the attached peer ranks inside the launch
    STREAM_JOB_SWIGLU = 4,      // two segments (gate, up) of equal rows: seg[0].y receives silu(gate x) * (up x)
    STREAM_JOB_ACCUM = 8,       // the results are added to what the output holds (residual connection)
};

struct StreamSeg {
    const uint8_t *w;   // streaming-layout rows
    void *y;            // output base (row m at y + m*ldy elements)
    long long ldy;
    int n;              // rows
    int group_begin;    // first virtual 4-row group of this segment (filled by stream_job_finish)
};

struct StreamJob {
    StreamSeg seg[kStreamMaxSeg];
    int nseg;
    int total_groups;                  // filled by stream_job_finish: 4-row groups over all segments
    int qt;
    int K, Kpad;
    int nsb, nchunks;                  // filled by stream_job_finish
    long long row_bytes;
    unsigned bytes_full, bytes_tail;   // filled: bytes one row adds to a chunk, all but the last / the last
    long long tile_group_stride;       // filled: bytes between the tiles of consecutive row groups (same chunk)
    int tile_chunk_stride;             // filled: bytes between the tiles of consecutive chunks (same row group)
    const void *x;
    long long ldx;
    int x_is_bf16, x_vec_ok, y_is_bf16;
    int flags;                         // STREAM_JOB_*
    int team;                          // which half of the consumer warps runs the job (see stream_assign_teams)
    const float *gamma;                // RMSNorm weight [K]: the activation is normalised on the load (null = none)
    float norm_eps;
    const uint8_t *xq;                 // device buffer for the activation in fixed point, filled by stream_xprep_launch
                                       // before the streaming launch (stream_xq_bytes); null = converted inside the kernel
};

struct StreamLaunch {
    const StreamJob *jobs_host;   // always: the descriptors, readable by the host
    const StreamJob *jobs_dev;    // the same table in device memory, or nullptr for a single job
    int njobs;
    int M;                        // 1..4
    int *status;                  // device status word
    unsigned *counter;            // device word for grid-wide completion counting
    int sm_count;
    size_t smem_limit;            // opt-in shared memory per block
    int warps, depth, grid;       // 0 = default
    int debug;                    // experiments only (see gemv.cu)
    int pdl;                      // launch with programmatic stream serialization
    int teams;                    // 1 = never split the consumer warps into two teams
    int producer_nap;             // ns the producer warp sleeps when it finds nothing to do (0 = spin)
    uint8_t *peer_base[8];        // every rank's exchange buffer (jobs flagged STREAM_JOB_SUM_RANKS); null = none
    int peer_rank, peer_world;
};
int gemv_max_m();
void stream_job_finish(StreamJob &job);
// Spreads the jobs of a plan over the two consumer-warp teams of a CTA, balancing streamed bytes.
void stream_assign_teams(StreamJob *jobs, int n);
size_t stream_xq_bytes(const StreamJob &J, int M);
cudaError_t stream_xprep_launch(const StreamJob *jobs_dev, int njobs, int M, cudaStream_t st);
cudaError_t stream_launch(const StreamLaunch &a, cudaStream_t st);

// ---- skinny.cu ------------------------------------------------------------------------------
// 2..16 activation rows against one or more weights of one block type: the packed weights stream
// through shared memory once and meet the exact bf16 activations in mma.sync with fp32 accumulation;
// products whose K spans several 2048-weight chunks end with a small chunk-sum launch.
struct SkinnyProduct {
    int qt;
    const uint8_t *w;        // streaming-layout weights
    int N, K, Kpad;
    const void *x;           // activations [M][K], bf16 (M <= 16) or fp32 (M <= 8: hi/lo halves take two token slots)
    long long ldx;
    int x_is_bf16;
    void *y;
    long long ldy;
    int y_is_bf16;
    int M;
};
struct SkinnyBuffers {
    uint8_t *ws;             // chunk sums of the call (skinny_part_bytes per product)
    size_t ws_bytes;
    void *jobs_dev;          // skinny_job_table_bytes() of device memory for calls with more than one product
    int *status;
    int sm_count;
    size_t smem_limit;
};
int skinny_max_m();
int skinny_max_products();
size_t skinny_part_bytes(const SkinnyProduct &a);
size_t skinny_job_table_bytes();
// at most four products (their descriptions travel in the kernel parameters): prepare, launch, forget
cudaError_t skinny_run(const SkinnyProduct *prods, int n, const SkinnyBuffers &buf, cudaStream_t st, int *launches);
// up to skinny_max_products() products prepared once and launched many times (plans): buf.jobs_dev,
// and buf.ws stay owned by the caller and must outlive the set
struct SkinnySet;
cudaError_t skinny_set_create(const SkinnyProduct *prods, int n, const SkinnyBuffers &buf, SkinnySet **out);
cudaError_t skinny_set_launch(const SkinnySet *set, cudaStream_t st);
int skinny_set_launches(const SkinnySet *set);
void skinny_set_destroy(SkinnySet *set);

// ---- gemm_tc.cu -----------------------------------------------------------------------------
struct GemmLaunch {
    int qt;
    const uint8_t *w;        // streaming-layout weights
    int N, K, Kpad;
    const void *x;           // fp16 activations [M][K], rows 16-byte aligned
    long long ldx;
    int M;
    void *y;
    long long ldy;
    int y_is_bf16;
    int *status;
    int sm_count;
    int bn_override;         // 0 = choose the token tile
    int debug;               // timing experiments (see GemmParams::debug); 0 in production
    int pair;                // 1 = large products use the two-CTA kernel (256-row tiles)
    float *part;             // workspace for K-split partial products of skinny batches (null = never split)
    size_t part_bytes;
};
size_t gemm_x_scratch_bytes(int M, int K);
// K ranges x rows never exceed SMs x 128 (one work unit per SM), tokens < 128: 148 x 128 x 127 x 4 bytes < 16 MB
constexpr size_t kGemmPartBytes = size_t(16) << 20;
// activations (bf16 or fp32) -> fp16 rows of ((K + 7) & ~7) elements in `scratch`
cudaError_t gemm_convert_x(const void *x, int x_is_bf16, long long ldx, void *scratch, int M, int K, cudaStream_t st);
cudaError_t gemm_launch(const GemmLaunch &a, cudaStream_t st);
// the same product with the activation copy in the library's built-in scratch array: a.x / a.ldx
// describe the caller's activations (bf16 or fp32), nothing is allocated
size_t gemm_static_scratch_elems();
cudaError_t gemm_launch_static(GemmLaunch a, int x_is_bf16, cudaStream_t st);

// ---- peer.cu --------------------------------------------------------------------------------
// Exchange buffer of one GPU.  Every element travels as an 8-byte (value, call number) pair written
// with one store, so the reader needs no separate flag and the writer no fence: a pair whose
// number is the current call's is complete.  Two regions (the stand-alone all-reduce kernel, and
// the sums inside the streaming kernel), each: call counters, then slots [2 sets][ranks][elements].
constexpr int kPeerMaxWorld = 8;
constexpr int kPeerBlocks = 16;                        // blocks of the stand-alone kernel
constexpr int kPeerThreads = 128;
constexpr int kPeerCtas = 160;                         // CTAs of the streaming kernel (one per SM)
constexpr int kPeerSlotFloats = 16384;                 // largest vector summed over ranks
constexpr size_t kPeerSlotBytes = size_t(kPeerSlotFloats) * 8;
constexpr size_t kPeerRegionSlots = size_t(2) * kPeerMaxWorld * kPeerSlotBytes;      // 2 MB
constexpr size_t kPeerEpochOff = 0;                    // [kPeerBlocks] u32
constexpr size_t kPeerSlotOff = 4096;
constexpr size_t kPeerFusedEpochOff = kPeerSlotOff + kPeerRegionSlots;               // [2 teams][kPeerCtas] u32
constexpr size_t kPeerFusedSlotOff = kPeerFusedEpochOff + 4096;                      // [2 teams][2 sets][ranks][elements]
constexpr size_t kPeerBufferBytes = kPeerFusedSlotOff + 2 * kPeerRegionSlots;
struct PeerLaunch {
    float *y;                       // in place: partial sums in, sums over ranks out
    int count;
    int rank, world;
    uint8_t *base[kPeerMaxWorld];   // every rank's exchange buffer as mapped in this process
    int *status;
};
cudaError_t peer_allreduce_launch(const PeerLaunch &a, cudaStream_t st);

}  // namespace b200q
