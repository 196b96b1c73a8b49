// Decode GEMV (M = 1) and M <= 4 product: the HBM-bound streaming kernel.
//
// Y[m][n] = sum_k X[m][k] * dequant(W)[n][k]   for the streaming layout of common.cuh.
//
// One launch runs a list of projection jobs (one job for b200q_matmul, a whole decode step for a
// plan) on persistent CTAs, one per SM, no CPU fallback, no cluster multicast:
//   * CW consumer warps and one producer warp.  Every consumer warp owns a private ring of
//     shared-memory slots; lane w of the producer warp keeps consumer w's ring full with 1-D
//     bulk copies (cp.async.bulk, completion counted on a "full" mbarrier) and learns that a slot
//     was consumed from an "empty" mbarrier.  A work item is one tile of the streaming layout
//     (4 rows x 8 superblock records = 4 x 2048 weights), fetched with a single bulk copy.  The rings run on across job boundaries, so the weights of
//     the next job stream in while the consumers still finish, reduce and store the current one:
//     HBM reads never wait for a launch, a prologue or a grid-wide barrier.
//   * per job each CTA owns a contiguous range of 4-row groups; items are dealt round-robin to
//     the consumer warps and each item's result goes to its own shared-memory cell, so the final
//     sum over K-chunks runs in a fixed order (bit-reproducible results).
//   * the activation is converted once per CTA and job into a 16-bit fixed-point form in shared
//     memory: per 32 weights one fp32 scale sx and per weight two signed bytes (x ~= sx * (256*hi
//     + lo), lo in [-128, 127]; relative step 2^-15 of the block maximum).  The packed 4/6/8-bit
//     weights multiply the two byte planes with dp4a, four weights per instruction, and block
//     results are scaled and accumulated in fp32.
//   * sub-block scales and mins are unpacked in registers; the min term of Q4_K and the -32
//     offset of Q6_K use per-block integer sums of the activation computed in the prologue.
//   * one lane handles one 64-weight unit of each of the item's 4 rows, so the activation bytes
//     it loads are reused 4 times; a row's partial sums live in the lanes of one warp and are
//     combined by warp shuffles.
//   * a job may declare that it reads what earlier jobs of the same launch wrote; the CTAs then
//     meet at a counter in global memory before converting that job's activation.
//   * every wait (mbarrier, counter) is bounded; on expiry the waiter raises the status word and
//     the kernel drains and returns.
#include <stdlib.h>

#include <algorithm>
#include <atomic>

#include "gemv_units.cuh"
#include "kernels.h"

namespace b200q {

namespace {

// timing experiments (parts of the pipeline switched off; results invalid) exist only in builds that ask for them
#ifdef B200Q_TIMING_EXPERIMENTS
#define GEMV_DBG(bit) (p.debug & (bit))
#else
#define GEMV_DBG(bit) (false)
#endif

constexpr int kMaxWarps = 15;    // consumer warps (+1 producer = 512 threads, 128 registers each)
constexpr int kMaxDepth = 8;
constexpr int KC = kChunkRecs;   // superblock records per chunk: 32 units of 64 weights, one per lane
constexpr int R = kRowGroup;     // rows per item

constexpr int chunk_bytes(int qt) { return (qt == QT_Q4_K || qt == QT_Q4_0 || qt == QT_MXFP4) ? KC * 144 : qt == QT_Q5_K ? KC * 176 : qt == QT_Q8_0 ? KC * 272 : 1680; }

struct StreamParams {
    const StreamJob *jobs;   // device table, or nullptr when the single job is `inl`
    StreamJob inl;
    int njobs;
    int M;
    int depth;               // ring slots per warp
    int chunk_stride;        // bytes between the rows of a slot (largest chunk of the launch's types)
    int jobs_bytes;          // shared-memory bytes of the job table
    int x_bytes;             // ... reserved for the fixed-point activation
    int partial_bytes;       // ... for the per-(row, chunk) partial sums
    int has_dep;             // some job waits for earlier jobs: CTAs count completions
    int teams;               // 2: the consumer warps work as two teams on different jobs at the same time
    int has_xq;              // some job's activation arrives already in fixed point (StreamJob::xq)
    int producer_nap;        // ns the producer warp sleeps when no ring slot is free (0 = spin)
    int debug;               // experiments only: 1 stream without computing, 2 compute without
                             // streaming, 4 skip the activation prologue, 8 skip the final pass,
                             // 64 do not wait for the peers' partial sums
    int *status;
    unsigned *counter;       // grid-wide completion counter (zeroed before the launch)
    uint8_t *peer_base[kPeerMaxWorld];   // exchange buffers of the tensor-parallel ranks (peer memory)
    int peer_rank, peer_world;           // peer_world <= 1: jobs flagged SUM_RANKS store their own sums
};

// shared-memory header: barriers and failure bookkeeping (the job table follows it)
struct SmemHead {
    uint64_t full[kMaxWarps * kMaxDepth];
    uint64_t empty[kMaxWarps * kMaxDepth];
    uint64_t xfull[2];       // per team: the job's pre-quantized activation has landed in the team's area
    int fail;                // raised by any warp that gave up a wait; everybody then drains and leaves
    int decide[2];           // per team: its first thread's sample of `fail`, taken before a barrier so all its warps agree
    int prod_done;           // the producer warp has stopped issuing copies
    int issued[kMaxWarps];   // ... after issuing this many items into each consumer's ring
    unsigned xepoch[2];      // per team: exchanges posted so far (loaded from the exchange buffer)
    int xfail;               // a wait for a peer's partial sums ran out
    int xdone[2];            // per team: warps x jobs finished so far (a job's activation area may be refilled once all
                             // the team's warps have left the job before it)
};

// (value, exchange number) pairs of the in-launch rank sums: one 8-byte store / load each
__device__ __forceinline__ void st_pair(unsigned long long *p, float v, unsigned e) {
    const unsigned long long w = ((unsigned long long)e << 32) | __float_as_uint(v);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_pair(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
constexpr size_t kHeadBytes = (sizeof(SmemHead) + 127) & ~size_t(127);

// (segment, row group inside it) of virtual group vg; segments are concatenated in launch order.
// A SWIGLU job interleaves its two segments instead (even groups gate, odd groups up), so that a
// CTA's contiguous range holds the gate rows and the up rows of the same outputs.
// (`glu`: the job's SWIGLU flag, read once per job by the caller: this runs once per work item.)
__device__ __forceinline__ void locate_group(const StreamJob &J, int vg, int &s, int &g, bool glu) {
    if (glu) {
        s = vg & 1;
        g = vg >> 1;
        return;
    }
    s = 0;
#pragma unroll
    for (int i = 1; i < kStreamMaxSeg; ++i)
        if (i < J.nseg && vg >= J.seg[i].group_begin) s = i;
    g = vg - J.seg[s].group_begin;
}

// virtual groups [gb, ge) of job J that CTA b of `grid` works on (whole gate/up pairs for SWIGLU)
template <bool FUSED = true>
__host__ __device__ __forceinline__ void cta_groups(const StreamJob &J, int b, int grid, int &gb, int &ge) {
    if (FUSED && (J.flags & STREAM_JOB_SWIGLU)) {
        const long long pairs = J.total_groups >> 1;
        gb = 2 * (int)(pairs * b / grid);
        ge = 2 * (int)(pairs * (b + 1) / grid);
    } else if (J.total_groups < (1 << 21)) {
        // (32-bit division: this runs once per job in every warp, the producer's included)
        gb = (int)((unsigned)J.total_groups * (unsigned)b / (unsigned)grid);
        ge = (int)((unsigned)J.total_groups * (unsigned)(b + 1) / (unsigned)grid);
    } else {
        gb = (int)((long long)J.total_groups * b / grid);
        ge = (int)((long long)J.total_groups * (b + 1) / grid);
    }
}

// barrier of one consumer team (hardware barrier 1 + team; barrier 0 is __syncthreads)
__device__ __forceinline__ void team_sync(int team, int T) { asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(T) : "memory"); }

// one item (a tile: up to 4 rows x one chunk) of one job for this lane's 64-weight unit;
// `sl` = shared address of the tile, `stride` = byte distance between its rows
template <int QT, int MT, typename Flush>
__device__ __forceinline__ void item_dot(int nsb, uint32_t sl, int stride, int sb0, int lsb, int j, int nr,
                                         const XView (&xv)[MT], int units16, bool whole, float (&acc)[R][MT],
                                         Flush &&flush_pending) {
    const int gsb = sb0 + lsb;
    const int gu = gsb * 4 + j;
    const uint32_t rec0 = sl + lsb * rec_bytes(QT);
    float d6[R];
    if constexpr (QT == QT_Q6_K) {
        const uint32_t doff = sl + (uint32_t)(q6k_d_off(gsb, nsb) - rec_off(QT, sb0));
#pragma unroll
        for (int r = 0; r < R; ++r) d6[r] = (r < nr) ? half_bits_to_float(lds16(doff + r * stride)) : 0.f;
    }
    auto load_w = [&](WRegs<QT> &w, int r) {
        if constexpr (QT == QT_Q6_K) w.load(rec0 + r * stride, j, d6[r]);
        else w.load(rec0 + r * stride, j);
    };
    if constexpr (MT <= 1 || (MT == 2 && QT != QT_Q6_K)) {
        // one or two activation rows: keep their bytes in registers, stream the weight rows past them
        XRegs<QT> xr[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) xr[m].load(xv[m], gu, gsb, j, units16);
        if (whole) flush_pending();
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r < nr) {
                WRegs<QT> w;
                load_w(w, r);
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[r][m] += w.dot(xr[m]);
            }
        }
    } else if constexpr (QT != QT_Q6_K && MT >= 3) {
        // three or four activation rows: two passes over the tile, two rows resident in each
        if (whole) flush_pending();
#pragma unroll 1
        for (int m0 = 0; m0 < MT; m0 += 2) {
            XRegs<QT> xa, xb;
            xa.load(xv[m0], gu, gsb, j, units16);
            const bool two = m0 + 1 < MT;
            if (two) xb.load(xv[m0 + 1 < MT ? m0 + 1 : m0], gu, gsb, j, units16);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (r < nr) {
                    WRegs<QT> w;
                    load_w(w, r);
                    const float va = w.dot(xa);
                    const float vb = two ? w.dot(xb) : 0.f;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        if (m == m0) acc[r][m] += va;
                        if (m == m0 + 1) acc[r][m] += vb;
                    }
                }
            }
        }
    } else {
        // more activation rows than registers can hold: one weight row at a time, activations re-read
        if (whole) flush_pending();
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            WRegs<QT> w;
            load_w(w, r);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                XRegs<QT> xr;
                xr.load(xv[m], gu, gsb, j, units16);
                const float v = w.dot(xr);
#pragma unroll
                for (int rr = 0; rr < R; ++rr)
                    if (rr == r) acc[rr][m] += v;
            }
        }
    }
}

// TYPES is the set of block types the launch's jobs use (bit 0 Q4_K, bit 1 Q6_K, bit 2 Q8_0): a
// single-type launch compiles only that type's unpacking, which keeps it free of register spills.
constexpr int TY_Q4K = 1, TY_Q6K = 2, TY_Q80 = 4, TY_Q5K = 8, TY_Q40 = 16, TY_MX4 = 32;

// VAR: which optional code the instantiation carries.  Bit 0: the fused epilogues (SWIGLU, ACCUM, norm on
// the load) for launches that hold such jobs; bit 1: the rank-sum exchange, for launches of attached
// tensor-parallel ranks.  Every form carries only what it needs: the kernel is sensitive to the
// registers and code of what it does not use.
template <int MT, int TYPES, int VAR>
__global__ void __launch_bounds__((kMaxWarps + 1) * 32, 1) stream_kernel(const StreamParams p) {
    constexpr bool FUSED = (VAR & 1) != 0, PEER = (VAR & 2) != 0;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int CW = (blockDim.x >> 5) - 1;     // consumer warps; warp CW is the producer
    const int D = p.depth;
    const int cw0 = p.teams == 2 ? (CW + 1) / 2 : CW;     // team 0 = consumer warps [0, cw0), team 1 = [cw0, CW)

    // shared-memory carve-up: header, activation planes, partial sums, rings
    SmemHead &head = *reinterpret_cast<SmemHead *>(smem);
    const uint32_t full0 = smem_u32(head.full), empty0 = smem_u32(head.empty);
    StreamJob *jobs_s = reinterpret_cast<StreamJob *>(smem + kHeadBytes);
    uint8_t *xbase0 = smem + kHeadBytes + p.jobs_bytes;                       // one activation area per team
    float *partial0 = reinterpret_cast<float *>(xbase0 + p.teams * p.x_bytes); // [row][chunk][MT], one per team
    uint8_t *rings = reinterpret_cast<uint8_t *>(partial0) + p.teams * p.partial_bytes;
    // Two teams: while one team sums, stores and prepares the next activation (the per-job work
    // that keeps no data moving), the other is in the middle of its own job, so the SM always has
    // warps doing block dots.  Team 0 = consumer warps [0, cw0), team 1 = [cw0, CW).

    const int slot_bytes = R * p.chunk_stride;
    const int ring_bytes = D * slot_bytes;

    if (threadIdx.x < CW) {
        for (int i = 0; i < D; ++i) {
            mbar_init(full0 + (threadIdx.x * kMaxDepth + i) * 8, 1);
            mbar_init(empty0 + (threadIdx.x * kMaxDepth + i) * 8, 1);
        }
        mbar_fence_init();
        fence_proxy_async();
    }
    if (threadIdx.x == 0) {
        head.fail = 0; head.prod_done = 0; head.xfail = 0;
        head.xdone[0] = head.xdone[1] = 0;
        for (int t = 0; t < 2; ++t) mbar_init(smem_u32(&head.xfull[t]), 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    // the job table (written by the host when the plan was made) moves to shared memory once
    if (p.jobs) {
        const int words = p.njobs * (int)(sizeof(StreamJob) / 4);
        const int *src = reinterpret_cast<const int *>(p.jobs);
        int *dst = reinterpret_cast<int *>(jobs_s);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = src[i];
    } else if (threadIdx.x == 0) {
        jobs_s[0] = p.inl;
    }
    // let the next kernel in the stream start early (it waits in pdl_wait before touching data)
    pdl_launch_dependents();
    __syncthreads();

    // =========================================================================================
    // producer warp: lane w feeds consumer warp w.  All lanes poll together (no lane blocks the
    // others): a lane issues its next item as soon as its consumer has released the slot.
    // =========================================================================================
    if (warp == CW) {
        const unsigned mask = 0xFFFFFFFFu;
        const bool feeder = lane < CW && !GEMV_DBG(2);
        const uint32_t ring_s = smem_u32(rings + lane * ring_bytes);
        const uint32_t fbar = full0 + lane * kMaxDepth * 8, ebar = empty0 + lane * kMaxDepth * 8;
        // the consumer this lane feeds: its team, its index and the number of warps in that team
        const int my_team = lane >= cw0 ? 1 : 0;
        const int twarp = lane - (my_team ? cw0 : 0), tcw = my_team ? CW - cw0 : cw0;
        int slot = 0, k = 0;
        uint32_t phase = 0;            // parity of the release this slot's next reuse waits for
        bool dead = false;
        // every lane walks its own team's jobs: job cursor, item cursor inside the job
        int jb = -1, n_items = 0, item = 0, g = 0, c = 0, gb = 0;
        bool glu = false;
        auto next_job = [&]() {
            do { ++jb; } while (jb < p.njobs && p.teams == 2 && jobs_s[jb].team != my_team);
            if (!feeder) jb = p.njobs;
            if (jb >= p.njobs) return;
            const StreamJob &J = jobs_s[jb];
            glu = FUSED && (J.flags & STREAM_JOB_SWIGLU) != 0;
            int ge;
            cta_groups<FUSED>(J, blockIdx.x, gridDim.x, gb, ge);
            n_items = (ge - gb) * J.nchunks;
            item = twarp;
            g = 0, c = twarp;          // item = g * nchunks + c, kept without dividing
            while (c >= J.nchunks) { c -= J.nchunks; ++g; }
        };
        next_job();
        // Lanes 30 and 31 feed the activation areas of team 0 and team 1: one bulk copy per job whose
        // activation was converted to fixed point by the prep launch, as soon as the team has left
        // the area's previous contents behind.
        const bool xfeeder = p.has_xq && lane >= 30 && (lane - 30) < p.teams && !GEMV_DBG(2);
        const int xteam = lane - 30;
        int xjb = -1, xseq = 0;        // job cursor; how many of the team's jobs lie before it
        auto next_xjob = [&]() {
            if (xjb >= 0) ++xseq;
            do { ++xjb; } while (xjb < p.njobs && p.teams == 2 && jobs_s[xjb].team != xteam);
        };
        if (xfeeder) next_xjob();
        else xjb = p.njobs;
        if (p.has_xq) pdl_wait();      // the prep launch's output is visible from here
        uint64_t t_first = 0;
        bool timing = false;
        int idle = 0;
#pragma unroll 1
        while (true) {
            bool progressed = false;
            if (*reinterpret_cast<volatile int *>(&head.fail)) { dead = true; break; }
            if (jb < p.njobs) {
                if (item >= n_items) {
                    next_job();
                    progressed = true;
                } else {
                    const StreamJob &J = jobs_s[jb];
                    const bool free_slot = (k < D) || mbar_test_wait(ebar + 8 * slot, phase ^ 1u);
                    if (free_slot) {
                        int sg, lg;
                        locate_group(J, gb + g, sg, lg, glu);
                        const uint32_t bytes = R * ((c == J.nchunks - 1) ? J.bytes_tail : J.bytes_full);   // whole tile, padding rows included
                        const uint32_t bar = fbar + 8 * slot;
                        fence_proxy_async();   // the consumer's reads of this slot precede the engine's writes
                        mbar_expect_tx(bar, bytes);
                        // tile (row group lg, chunk c): both strides were worked out when the job was made, so the
                        // producer's per-item path has no type logic
                        bulk_g2s(ring_s + slot * slot_bytes, J.seg[sg].w + (long long)lg * J.tile_group_stride + c * J.tile_chunk_stride,
                                 bytes, bar);
                        item += tcw;
                        c += tcw;
                        while (c >= J.nchunks) { c -= J.nchunks; ++g; }
                        ++k;
                        if (++slot == D) { slot = 0; phase ^= 1u; }
                        progressed = true;
                    }
                }
            }
            if (xjb < p.njobs) {
                const StreamJob &J = jobs_s[xjb];
                // Every job, with or without an image, is passed only once all warps of the team have
                // finished the job before it (a plain count: nothing to confuse however far either side
                // runs ahead).  Passing earlier would overwrite the activation area of a job still in
                // progress and arrive twice in one phase of the image barrier.
                const int xwarps = xteam ? CW - cw0 : cw0;
                if (xseq != 0 && *reinterpret_cast<volatile int *>(&head.xdone[xteam]) < xseq * xwarps) {
                    // the previous job of the team is still running
                } else if (!J.xq) {
                    next_xjob();
                    progressed = true;
                } else {
                    const int n_isum = (J.qt == QT_Q6_K) ? (J.Kpad >> 4) : (J.Kpad >> 5);
                    const uint32_t bytes = (uint32_t)p.M * (uint32_t)(2 * J.Kpad + (J.Kpad >> 5) * 4 + n_isum * 4);
                    const uint32_t bar = smem_u32(&head.xfull[xteam]);
                    fence_proxy_async();
                    mbar_expect_tx(bar, bytes);
                    bulk_g2s(smem_u32(xbase0 + xteam * p.x_bytes), J.xq, bytes, bar);
                    next_xjob();
                    progressed = true;
                }
            }
            if (__all_sync(mask, jb >= p.njobs && xjb >= p.njobs)) break;
            if (__any_sync(mask, progressed)) {
                idle = 0;
                timing = false;
                continue;
            }
            // nothing to do right now: step aside for a moment instead of taking issue slots from the
            // consumer warps that share this scheduler (a slot frees up every ~150 ns on average)
            if (p.producer_nap) __nanosleep(p.producer_nap);
            if (++idle >= 1024) {   // nobody moved for a while: look at the clock
                idle = 0;
                const uint64_t now = globaltimer_ns();
                if (!timing) {
                    timing = true;
                    t_first = now;
                } else if (now - t_first > kWaitLimitNs) {
                    if (lane == 0) atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                    *reinterpret_cast<volatile int *>(&head.fail) = 1;
                    dead = true;
                    break;
                }
            }
        }
        (void)dead;
        // tell the consumers how much is (or was) in flight, so a failing CTA can wait for exactly
        // those copies before its shared memory is released
        if (lane < CW) head.issued[lane] = k;
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            *reinterpret_cast<volatile int *>(&head.prod_done) = 1;
        }
        return;
    }

    // =========================================================================================
    // consumer warps
    // =========================================================================================
    const int team = warp >= cw0 ? 1 : 0;
    const int tw0 = team ? cw0 : 0;                 // first warp of this thread's team
    const int tcw = team ? CW - cw0 : cw0;          // warps in the team
    const int T = tcw * 32;                         // threads in the team
    const int tid = threadIdx.x - tw0 * 32;         // thread index inside the team
    const int twarp = warp - tw0;
    uint8_t *xbase = xbase0 + team * p.x_bytes;
    float *partial_t = partial0 + team * (p.partial_bytes >> 2);      // two copies, used by alternate jobs
    int tjobs = 0, xq_seen = 0;                                         // the team's jobs so far; those with a pre-quantized activation
    const uint32_t ring_sa = smem_u32(rings + warp * ring_bytes);
    const uint32_t fbar = full0 + warp * kMaxDepth * 8, ebar = empty0 + warp * kMaxDepth * 8;
    const int lsb = lane >> 2, j = lane & 3;   // this lane's record and 64-weight group in a chunk
    volatile int *fail_flag = &head.fail;
    int slot = 0, consumed = 0;
    uint32_t phase = 0;
    XRaw xraw;                 // the next job's activation, loaded early (M = 1, bf16)
    bool have_raw = false;
    auto job_xsrc = [&](const StreamJob &Jx) {
        XSrc xs;
        xs.x = Jx.x; xs.ldx = Jx.ldx; xs.x_is_bf16 = Jx.x_is_bf16; xs.x_vec_ok = Jx.x_vec_ok;
        xs.K = Jx.K; xs.Kpad = Jx.Kpad;
        xs.gamma = FUSED ? Jx.gamma : nullptr;
        xs.rs = 1.f;
        return xs;
    };

    // ---- sums over tensor-parallel ranks, inside the launch -----------------------------------
    // A job flagged SUM_RANKS does not store its row sums: every CTA writes them, as (value,
    // exchange number) pairs, into its slot of every rank's exchange buffer (peer stores over
    // NVLink) and later adds up, in rank order, what the same CTA of every rank delivered, into y;
    // a pair that carries the current exchange number is complete, so there is no flag and no
    // fence.  "Later" is just before the CTA posts its next exchange (or at the end of the launch),
    // so the transfer hides behind the jobs in between; launches whose jobs wait for one another
    // complete it at once.  Two slot sets alternate; a CTA posts exchange e + 1 only after it has
    // read exchange e, and can only read e + 1 after the peers posted it, i.e. after they read e:
    // no pair is overwritten before it has been read.  All ranks run the same plan on the same grid.
    const bool xenabled = PEER && p.peer_world > 1;
    unsigned xe = 0;
    bool xe_loaded = false;
    int xpending = -1;
    auto exchange_complete = [&](int job, unsigned e) {
        const StreamJob &Jc = jobs_s[job];
        const unsigned long long *slots = reinterpret_cast<const unsigned long long *>(p.peer_base[p.peer_rank] + kPeerFusedSlotOff) +
                                          (size_t)(team * 2 + (e & 1)) * kPeerMaxWorld * kPeerSlotFloats;
        int gbc, gec;
        cta_groups<FUSED>(Jc, blockIdx.x, gridDim.x, gbc, gec);
        const int n = Jc.seg[0].n;
        const bool accum = FUSED && (Jc.flags & STREAM_JOB_ACCUM) != 0;
        const int cells = (gec - gbc) * R * MT;
        // Eight lanes share one output: lane r of the group fetches rank r's pair (and waits for it, with the
        // usual limit), so all ranks' pairs travel at the same time; lane 0 then adds them in rank order.
        const bool dead = *reinterpret_cast<volatile int *>(&head.xfail) != 0;
        for (int base = 0; base < cells; base += T / kPeerMaxWorld) {
            const int t = base + (tid >> 3), r = lane & 7;
            const int rl = t / MT, m = t - rl * MT;
            const int row = gbc * R + rl;
            const bool valid = t < cells && row < n && m < p.M;
            const int si = m * n + row;
            unsigned long long w = 0;
            bool ok = !dead;
            if (valid && r < p.peer_world && ok) {
                const unsigned long long *q = slots + (size_t)r * kPeerSlotFloats + si;
                w = ld_pair(q);
                if ((unsigned)(w >> 32) != e && !GEMV_DBG(64)) {
                    const uint64_t t0 = globaltimer_ns();
                    int spins = 0;
                    while ((unsigned)((w = ld_pair(q)) >> 32) != e) {
                        if ((++spins & 63) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
                            ok = false;
                            head.xfail = 1;
                            atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                            break;
                        }
                    }
                }
            }
            const float v = __uint_as_float((unsigned)w);
            const int lane0 = lane & ~7;
            float acc = __shfl_sync(0xFFFFFFFFu, v, lane0);
#pragma unroll
            for (int rr = 1; rr < kPeerMaxWorld; ++rr) {
                const float o = __shfl_sync(0xFFFFFFFFu, v, lane0 + rr);
                if (rr < p.peer_world) acc += o;
            }
            const unsigned okmask = __ballot_sync(0xFFFFFFFFu, ok);
            if (valid && r == 0 && ((okmask >> lane0) & 0xFFu) == 0xFFu) {
                float *yp = reinterpret_cast<float *>(Jc.seg[0].y) + (long long)m * Jc.seg[0].ldy + row;
                *yp = accum ? *yp + acc : acc;
            }
        }
    };

    bool first_job = true;
#pragma unroll 1
    for (int jb = 0; jb < p.njobs; ++jb) {
        const StreamJob &J = jobs_s[jb];
        if (p.teams == 2 && J.team != team) continue;      // the other team's job

        // ---- dependencies --------------------------------------------------------------------
        if (first_job) pdl_wait();   // the previous kernel's writes (activations) are visible from here
        first_job = false;
        if (J.flags & STREAM_JOB_WAITS) {
            // every CTA has stored all earlier jobs' outputs once the counter reaches grid * jb
            if (tid == 0) {
                const unsigned target = gridDim.x * (unsigned)jb;
                const uint64_t t0 = globaltimer_ns();
                unsigned seen;
                int spins = 0;
                while (true) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counter) : "memory");
                    if (seen >= target || *fail_flag) break;
                    if ((++spins & 255) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
                        atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                        *fail_flag = 1;
                        break;
                    }
                }
            }
            team_sync(team, T);
        }

        // ---- this job's geometry -------------------------------------------------------------
        int gb, ge;
        cta_groups<FUSED>(J, blockIdx.x, gridDim.x, gb, ge);
        const int n_items = (ge - gb) * J.nchunks;
        const int nchunks = J.nchunks, nsb = J.nsb, qt = J.qt;
        const bool glu = FUSED && (J.flags & STREAM_JOB_SWIGLU) != 0;
        const int units16 = (J.Kpad >> 6) * 16;
        const int plane = J.Kpad;
        const int n_isum = (qt == QT_Q6_K) ? (J.Kpad >> 4) : (J.Kpad >> 5);
        const int per_m = 2 * plane + (J.Kpad >> 5) * 4 + n_isum * 4;        // xh, xl, sx, isum

        // ---- prologue: activation rows -> fixed point ----------------------------------------
        // partial sums alternate between two copies: the previous job's are still being added up by
        // slower threads of the team when this job's first items are flushed
        float *partial = partial_t + (tjobs & 1) * (p.partial_bytes >> 3);
        ++tjobs;
        const bool pre_x = J.xq != nullptr && !GEMV_DBG(2);
        XView xv[MT];
        {
            XSrc xs = job_xsrc(J);
            const bool norm = FUSED && xs.gamma != nullptr && !pre_x;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (norm && m < p.M) {
                    // RMSNorm on the load: the team adds up the row's squares first (partials through the
                    // partial-sum table, which no item of this job has touched yet)
                    float ss = row_square_share(xs, m, tid, T);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                    team_sync(team, T);
                    if (lane == 0) partial[twarp] = ss;
                    team_sync(team, T);
                    float tot = 0.f;
                    for (int w = 0; w < tcw; ++w) tot += partial[w];
                    xs.rs = rsqrtf(tot / (float)xs.K + J.norm_eps);
                }
                uint8_t *b = xbase + m * per_m;
                float *sxp = reinterpret_cast<float *>(b + 2 * plane);
                int *isp = reinterpret_cast<int *>(b + 2 * plane + (J.Kpad >> 5) * 4);
                xv[m].xh = smem_u32(b);
                xv[m].xl = smem_u32(b + plane);
                xv[m].sx = smem_u32(sxp);
                xv[m].isum = smem_u32(isp);
                if (m < p.M && !GEMV_DBG(4) && !pre_x) {
                    const bool q6 = (TYPES & TY_Q6K) && (TYPES == TY_Q6K || qt == QT_Q6_K);
                    if (MT == 1 && have_raw && !norm) {
                        if (q6) prep_from_raw<QT_Q6_K>(xs, tid, T, xraw, b, b + plane, sxp, isp, units16);
                        else if (TYPES & ~TY_Q6K) prep_from_raw<QT_Q4_K>(xs, tid, T, xraw, b, b + plane, sxp, isp, units16);
                    } else {
                        if (q6) prep_row<QT_Q6_K, FUSED>(xs, m, tid, T, b, b + plane, sxp, isp, units16);
                        else if (TYPES & ~TY_Q6K) prep_row<QT_Q4_K, FUSED>(xs, m, tid, T, b, b + plane, sxp, isp, units16);
                    }
                }
            }
        }
        if (pre_x) {
            // the fixed-point image arrives by bulk copy: every thread waits for it itself, no team barrier
            bool okx = mbar_wait_bounded(smem_u32(&head.xfull[team]), (uint32_t)xq_seen & 1u);
            ++xq_seen;
            if (!okx) {
                atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                *fail_flag = 1;
            }
        } else {
            team_sync(team, T);
        }

        // ---- items ---------------------------------------------------------------------------
        // The cross-lane sum of an item's results is taken one iteration late, after the next
        // item's shared-memory loads have been issued, so its shuffle chain hides behind them.
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
                if ((lane & (32 / R - 1)) == 0 && r < pend_nr) partial[pend_cell + r * nchunks] = v;
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float v = pend[r][m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                        if (lane == 0 && r < pend_nr) partial[(pend_cell + r * nchunks) * MT + m] = v;
                    }
                }
            }
            pend_cell = -1;
        };

        // item = g * nchunks + c; stepping by CW items without dividing in the loop
        const int step_g = tcw / nchunks, step_c = tcw - step_g * nchunks;
        int g = twarp / nchunks, c = twarp - g * nchunks;
#pragma unroll 1
        for (int item = GEMV_DBG(16) ? n_items : twarp; item < n_items; item += tcw) {
            // the common case is a slot that is already full: one probe, and the abort flag is only looked at
            // when the warp has to wait
            bool ok = GEMV_DBG(2) || mbar_test_wait(fbar + 8 * slot, phase);
            if (!__all_sync(0xFFFFFFFFu, ok)) {
                ok = mbar_wait_bounded(fbar + 8 * slot, phase);
                ok = __all_sync(0xFFFFFFFFu, ok && !*fail_flag);
            }
            if (!ok) {
                if (lane == 0) {
                    atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);
                    *fail_flag = 1;
                }
                break;
            }
            int sg, lg;
            locate_group(J, gb + g, sg, lg, glu);
            const int nr = group_rows(lg, J.seg[sg].n);
            const int cb = (c == nchunks - 1) ? (int)J.bytes_tail : (int)J.bytes_full;   // bytes per tile row
            const int sb0 = c * KC;
            float acc[R][MT];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

            // the pending sum uses full-warp shuffles, so it may sit inside the branch below only
            // when every lane takes that branch (a chunk of 8 whole records)
            const bool whole = (sb0 + KC <= nsb) && !GEMV_DBG(1);
            if (!whole) flush_pending();
            if (sb0 + lsb < nsb && !GEMV_DBG(1)) {
                const uint32_t sl = ring_sa + slot * slot_bytes;
                if ((TYPES & TY_Q4K) && (TYPES == TY_Q4K || qt == QT_Q4_K))
                    item_dot<QT_Q4_K, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
                else if ((TYPES & TY_Q6K) && (TYPES == TY_Q6K || qt == QT_Q6_K))
                    item_dot<QT_Q6_K, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
                else if ((TYPES & TY_Q5K) && (TYPES == TY_Q5K || qt == QT_Q5_K))
                    item_dot<QT_Q5_K, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
                else if ((TYPES & TY_Q40) && (TYPES == TY_Q40 || qt == QT_Q4_0))
                    item_dot<QT_Q4_0, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
                else if ((TYPES & TY_MX4) && (TYPES == TY_MX4 || qt == QT_MXFP4))
                    item_dot<QT_MXFP4, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
                else if (TYPES & TY_Q80)
                    item_dot<QT_Q8_0, MT>(nsb, sl, cb, sb0, lsb, j, nr, xv, units16, whole, acc, flush_pending);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(ebar + 8 * slot);   // slot may be refilled
            if (++slot == D) { slot = 0; phase ^= 1u; }
            ++consumed;

            // one shared-memory cell per (row, chunk, m): the final sum over chunks runs in a
            // fixed order whatever warp produced which cell
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) pend[r][m] = acc[r][m];
            pend_cell = GEMV_DBG(32) ? -1 : (g * R) * nchunks + c;
            pend_nr = nr;
            if constexpr (MT > 1) flush_pending();   // several activation rows: registers are scarce, sum at once
            g += step_g;
            c += step_c;
            if (c >= nchunks) { c -= nchunks; ++g; }
        }
        flush_pending();
        // start loading the next job's activation now: the loads fly while this job is summed and
        // stored (not possible when that activation is still being produced by this launch)
        // this warp is done with the activation area: the next pre-quantized image may overwrite it
        if (p.has_xq) {
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                atomicAdd(&head.xdone[team], 1);
            }
        }
        have_raw = false;
        if (MT == 1 && !GEMV_DBG(4)) {
            int jn = jb + 1;
            while (jn < p.njobs && p.teams == 2 && jobs_s[jn].team != team) ++jn;
            if (jn < p.njobs) {
                const StreamJob &Jn = jobs_s[jn];
                const XSrc xn = job_xsrc(Jn);
                if (!(Jn.flags & STREAM_JOB_WAITS) && !Jn.xq && !xn.gamma && prep_can_prefetch(xn, T)) {
                    prep_prefetch(xn, tid, T, xraw);
                    have_raw = true;
                }
            }
        }
        if (tid == 0) head.decide[team] = *fail_flag;
        team_sync(team, T);

        if (head.decide[team]) {
            // Some wait ran out.  Copies already issued into this warp's ring must land before
            // the CTA's shared memory is released: learn from the producer how many were issued
            // and wait for exactly those, each wait again with a limit.
            const uint64_t t0 = globaltimer_ns();
            while (!*reinterpret_cast<volatile int *>(&head.prod_done) && globaltimer_ns() - t0 < kWaitLimitNs) {}
            const int outstanding = *reinterpret_cast<volatile int *>(&head.issued[warp]) - consumed;
            for (int i = 0; i < outstanding && i < D; ++i) {
                if (!mbar_wait_bounded(fbar + 8 * slot, phase)) break;
                if (++slot == D) { slot = 0; phase ^= 1u; }
            }
            return;
        }

        // ---- final pass: sum the chunks of every row of this CTA in order and store ------------
        const bool xsum = xenabled && (J.flags & STREAM_JOB_SUM_RANKS);
        if (xsum) {
            if (!xe_loaded) {   // exchanges posted by earlier launches (after pdl_wait: their last write is visible)
                if (tid == 0)
                    head.xepoch[team] = *(reinterpret_cast<const unsigned *>(p.peer_base[p.peer_rank] + kPeerFusedEpochOff) + team * kPeerCtas + blockIdx.x);
                team_sync(team, T);
                xe = head.xepoch[team];
                xe_loaded = true;
            }
            if (xpending >= 0) {
                exchange_complete(xpending, xe);
                xpending = -1;
            }
            ++xe;
        }
        const bool accum = FUSED && (J.flags & STREAM_JOB_ACCUM) != 0;
        auto store_out = [&](const StreamSeg &S, long long idx, float v) {
            if (J.y_is_bf16) {
                __nv_bfloat16 *yp = reinterpret_cast<__nv_bfloat16 *>(S.y) + idx;
                *yp = __float2bfloat16_rn(accum ? __bfloat162float(*yp) + v : v);
            } else {
                float *yp = reinterpret_cast<float *>(S.y) + idx;
                *yp = accum ? *yp + v : v;
            }
        };
        if (glu) {
            // local groups alternate gate, up: output row = silu(gate row) * up row, to the first segment's y
            const int outs = GEMV_DBG(8) ? 0 : ((ge - gb) >> 1) * R * MT;
            for (int t = tid; t < outs; t += T) {
                const int ro = t / MT, m = t - ro * MT;          // ro = local pair * 4 + row in group
                const int pair = ro / R, r = ro & (R - 1);
                const int row = ((gb >> 1) + pair) * R + r;
                if (row < J.seg[0].n && m < p.M) {
                    float gv = 0.f, uv = 0.f;
                    const int cg = ((2 * pair) * R + r) * nchunks, cu = ((2 * pair + 1) * R + r) * nchunks;
                    for (int cc = 0; cc < nchunks; ++cc) {
                        gv += partial[(cg + cc) * MT + m];
                        uv += partial[(cu + cc) * MT + m];
                    }
                    store_out(J.seg[0], (long long)m * J.seg[0].ldy + row, gv / (1.f + __expf(-gv)) * uv);
                }
            }
        }
        const int cells = (GEMV_DBG(8) || glu) ? 0 : (ge - gb) * R * MT;
        for (int t = tid; t < cells; t += T) {
            const int rl = t / MT, m = t - rl * MT;      // rl = local group * 4 + row in group
            int sg, lg;
            locate_group(J, gb + rl / R, sg, lg, false);
            const int row = lg * R + (rl & (R - 1));
            if (row < J.seg[sg].n && m < p.M) {
                float v = 0.f;
                for (int cc = 0; cc < nchunks; ++cc) v += partial[(rl * nchunks + cc) * MT + m];
                if (xsum) {     // one segment, fp32 output (checked when the plan was made)
                    const size_t si = (size_t)((team * 2 + (xe & 1)) * kPeerMaxWorld + p.peer_rank) * kPeerSlotFloats + m * J.seg[0].n + row;
                    for (int r = 0; r < p.peer_world; ++r)
                        st_pair(reinterpret_cast<unsigned long long *>(p.peer_base[r] + kPeerFusedSlotOff) + si, v, xe);
                    continue;
                }
                store_out(J.seg[sg], (long long)m * J.seg[sg].ldy + row, v);
            }
        }
        if (xsum) {
            if (p.has_dep) exchange_complete(jb, xe);   // a later job may read y: finish now
            else xpending = jb;
        }
        if (p.has_dep) {
            // publish: this CTA's outputs of job jb are stored
            team_sync(team, T);
            if (tid == 0) {
                __threadfence();
                atomicAdd(p.counter, 1u);
            }
        }
    }
    if (xpending >= 0) exchange_complete(xpending, xe);
    if (xe_loaded && tid == 0)
        *(reinterpret_cast<unsigned *>(p.peer_base[p.peer_rank] + kPeerFusedEpochOff) + team * kPeerCtas + blockIdx.x) = xe;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

int gemv_max_m() { return 4; }

namespace {

// Converts the activation of every job that has an image buffer (StreamJob::xq) to the fixed-point
// form the streaming kernel works on, once per job instead of once per CTA and job: block (job, part)
// handles every `parts`-th run of 8 elements.  The image has the layout of the kernel's
// shared-memory activation area ([row][xh | xl | sx | isum]), so a CTA fetches it with one bulk copy.
__global__ void __launch_bounds__(256) xprep_kernel(const StreamJob *jobs, int M) {
    pdl_launch_dependents();       // the streaming launch may start (it waits before reading the images)
    const StreamJob &J = jobs[blockIdx.x];
    if (!J.xq) return;
    XSrc xs;
    xs.x = J.x; xs.ldx = J.ldx; xs.x_is_bf16 = J.x_is_bf16; xs.x_vec_ok = J.x_vec_ok;
    xs.K = J.K; xs.Kpad = J.Kpad;
    xs.gamma = J.gamma;
    xs.rs = 1.f;
    __shared__ float warp_ss[8];
    const int units16 = (J.Kpad >> 6) * 16, plane = J.Kpad;
    const int n_isum = (J.qt == QT_Q6_K) ? (J.Kpad >> 4) : (J.Kpad >> 5);
    const int per_m = 2 * plane + (J.Kpad >> 5) * 4 + n_isum * 4;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, T = gridDim.y * blockDim.x;
    for (int m = 0; m < M; ++m) {
        uint8_t *b = const_cast<uint8_t *>(J.xq) + (size_t)m * per_m;
        float *sxp = reinterpret_cast<float *>(b + 2 * plane);
        int *isp = reinterpret_cast<int *>(b + 2 * plane + (J.Kpad >> 5) * 4);
        if (xs.gamma) {
            // RMSNorm on the load: every block of the job adds up the whole row's squares itself
            float ss = row_square_share(xs, m, threadIdx.x, blockDim.x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_ss[w];
            xs.rs = rsqrtf(tot / (float)xs.K + J.norm_eps);
        }
        if (J.qt == QT_Q6_K) prep_row<QT_Q6_K, true>(xs, m, tid, T, b, b + plane, sxp, isp, units16);
        else prep_row<QT_Q4_K, true>(xs, m, tid, T, b, b + plane, sxp, isp, units16);
    }
}

}  // namespace

size_t stream_xq_bytes(const StreamJob &J, int M) {
    const size_t n_isum = J.qt == QT_Q6_K ? J.Kpad / 16 : J.Kpad / 32;
    const size_t per_m = 2 * (size_t)J.Kpad + (J.Kpad / 32) * 4 + n_isum * 4;
    return ((size_t)M * per_m + 255) & ~size_t(255);
}

cudaError_t stream_xprep_launch(const StreamJob *jobs_dev, int njobs, int M, cudaStream_t st) {
    if (njobs < 1) return cudaSuccess;
    xprep_kernel<<<dim3((unsigned)njobs, 4), 256, 0, st>>>(jobs_dev, M);
    return cudaGetLastError();
}

namespace {

template <int MT, int TYPES, int VAR = 0>
cudaError_t launch_t(const StreamLaunch &a, StreamParams &p, int grid, cudaStream_t st) {
    int warps = a.warps > 0 ? a.warps : kMaxWarps;
    if (warps > kMaxWarps) warps = kMaxWarps;
    // shared-memory needs: the largest activation form and partial-sum table over the jobs
    size_t x_bytes = 0, partial = 0;
    int stride = 0;
    for (int i = 0; i < a.njobs; ++i) {
        const StreamJob &J = a.jobs_host[i];
        const size_t n_isum = J.qt == QT_Q6_K ? J.Kpad / 16 : J.Kpad / 32;
        const size_t per_m = 2 * (size_t)J.Kpad + (J.Kpad / 32) * 4 + n_isum * 4;
        x_bytes = std::max(x_bytes, (MT * per_m + 127) & ~size_t(127));
        int groups = (J.total_groups + grid - 1) / grid;
        if (J.flags & STREAM_JOB_SWIGLU) groups = 2 * ((J.total_groups / 2 + grid - 1) / grid);
        partial = std::max(partial, (((size_t)groups * R * J.nchunks * MT * 4) + 127) & ~size_t(127));
        stride = std::max(stride, chunk_bytes(J.qt));
    }
    p.x_bytes = (int)x_bytes;
    p.partial_bytes = (int)(2 * partial);          // two copies per team, used by alternate jobs
    p.chunk_stride = stride;
    p.jobs_bytes = (int)(((size_t)a.njobs * sizeof(StreamJob) + 127) & ~size_t(127));
    const size_t budget = a.smem_limit;
    // two consumer teams need two activation areas; keep them only while two ring slots per warp still fit
    if (p.teams == 2 && kHeadBytes + p.jobs_bytes + 2 * (x_bytes + 2 * partial) + (size_t)warps * 2 * R * stride > budget) p.teams = 1;
    if (warps < 4) p.teams = 1;
    const size_t fixed = kHeadBytes + p.jobs_bytes + p.teams * (x_bytes + 2 * partial);
    // fewer consumer warps when two slots each do not fit (very long rows, several activation rows)
    while (warps > 4 && fixed + (size_t)warps * 2 * R * stride > budget) --warps;
    if (fixed + (size_t)warps * 2 * R * stride > budget) return cudaErrorInvalidValue;
    int depth = (int)((budget - fixed) / ((size_t)warps * R * stride));
    if (depth > kMaxDepth) depth = kMaxDepth;
    if (a.depth > 0 && a.depth < depth) depth = a.depth;
    p.depth = depth;
    const size_t smem = fixed + (size_t)warps * depth * R * stride;

    if (VAR == 0) {      // pick the form once, from the plain entry
        bool fused = false, sums = false;
        for (int i = 0; i < a.njobs; ++i) {
            fused = fused || (a.jobs_host[i].flags & (STREAM_JOB_SWIGLU | STREAM_JOB_ACCUM)) != 0 || a.jobs_host[i].gamma != nullptr;
            sums = sums || (a.jobs_host[i].flags & STREAM_JOB_SUM_RANKS) != 0;
        }
        const bool peer = sums && p.peer_world > 1;
        if (peer && fused) return launch_t<MT, TYPES, (VAR == 0 ? 3 : VAR)>(a, p, grid, st);
        if (peer) return launch_t<MT, TYPES, (VAR == 0 ? 2 : VAR)>(a, p, grid, st);
        if (fused) return launch_t<MT, TYPES, (VAR == 0 ? 1 : VAR)>(a, p, grid, st);
    }
    auto kern = stream_kernel<MT, TYPES, VAR>;
    static std::atomic<size_t> configured{0};   // per instantiation; a context on another device re-sets it
    static std::atomic<int> configured_dev{-1};  // (contexts on several threads may launch at once)
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > configured.load() || dev != configured_dev.load()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
        configured_dev = dev;
    }
    if (p.has_dep) {
        cudaError_t e = cudaMemsetAsync(p.counter, 0, sizeof(unsigned), st);
        if (e != cudaSuccess) return e;
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
    cfg.numAttrs = (a.pdl && !p.has_dep) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int TYPES>
cudaError_t launch_m(const StreamLaunch &a, StreamParams &p, int grid, cudaStream_t st) {
    switch (a.M) {
    case 1: return launch_t<1, TYPES>(a, p, grid, st);
    case 2: return launch_t<2, TYPES>(a, p, grid, st);
    case 3: return launch_t<3, TYPES>(a, p, grid, st);
    default: return launch_t<4, TYPES>(a, p, grid, st);
    }
}

constexpr int kMaxJobsPerLaunch = 64;   // the job table lives in shared memory

cudaError_t stream_launch_one(const StreamLaunch &a, cudaStream_t st) {
    if (a.njobs < 1 || a.M < 1 || a.M > 4 || !a.jobs_host) return cudaErrorInvalidValue;
    StreamParams p{};
    p.jobs = a.jobs_dev;
    if (!a.jobs_dev) {
        if (a.njobs != 1) return cudaErrorInvalidValue;
        p.inl = a.jobs_host[0];
    }
    p.njobs = a.njobs;
    p.M = a.M;
    p.debug = a.debug;
    p.producer_nap = a.producer_nap;
    p.status = a.status;
    p.counter = a.counter;
    p.peer_rank = a.peer_rank;
    p.peer_world = a.peer_world;
    for (int r = 0; r < kPeerMaxWorld; ++r) p.peer_base[r] = a.peer_base[r];
    p.has_dep = 0;
    for (int i = 0; i < a.njobs; ++i)
        if (a.jobs_host[i].flags & STREAM_JOB_WAITS) p.has_dep = 1;
    p.has_xq = 0;
    for (int i = 0; i < a.njobs; ++i)
        if (a.jobs_host[i].xq) p.has_xq = 1;
    // two teams when the launch holds jobs for both and no job waits for another
    p.teams = 1;
    if (!p.has_dep && a.teams != 1) {
        bool t0 = false, t1 = false;
        for (int i = 0; i < a.njobs; ++i) (a.jobs_host[i].team ? t1 : t0) = true;
        if (t0 && t1) p.teams = 2;
    }
    const int grid = a.grid > 0 ? a.grid : a.sm_count;
    if (p.has_dep && grid > a.sm_count) return cudaErrorInvalidValue;   // the counter wait needs every CTA resident
    if (p.peer_world > 1) {
        for (int i = 0; i < a.njobs; ++i) {
            const StreamJob &J = a.jobs_host[i];
            if (!(J.flags & STREAM_JOB_SUM_RANKS)) continue;
            // in-launch sums: per-CTA flags, one segment, fp32 outputs that fit one slot
            if (grid > kPeerCtas || J.nseg != 1 || J.y_is_bf16 || (long long)a.M * J.seg[0].n > kPeerSlotFloats)
                return cudaErrorInvalidValue;
        }
    }
    int types = 0;
    for (int i = 0; i < a.njobs; ++i) {
        const int qt = a.jobs_host[i].qt;
        types |= qt == QT_Q4_K ? TY_Q4K : qt == QT_Q6_K ? TY_Q6K : qt == QT_Q8_0 ? TY_Q80 : qt == QT_Q5_K ? TY_Q5K : qt == QT_Q4_0 ? TY_Q40 : qt == QT_MXFP4 ? TY_MX4 : 64;
    }
    if (types & 64) return cudaErrorInvalidValue;
    switch (types) {
    case TY_Q4K: return launch_m<TY_Q4K>(a, p, grid, st);
    case TY_Q6K: return launch_m<TY_Q6K>(a, p, grid, st);
    case TY_Q80: return launch_m<TY_Q80>(a, p, grid, st);
    case TY_Q5K: return launch_m<TY_Q5K>(a, p, grid, st);
    case TY_Q40: return launch_m<TY_Q40>(a, p, grid, st);
    case TY_MX4: return launch_m<TY_MX4>(a, p, grid, st);
    default:
        if (!(types & (TY_Q5K | TY_Q40 | TY_MX4))) return launch_m<TY_Q4K | TY_Q6K | TY_Q80>(a, p, grid, st);
        return launch_m<TY_Q4K | TY_Q6K | TY_Q80 | TY_Q5K | TY_Q40 | TY_MX4>(a, p, grid, st);
    }
}

}  // namespace

void stream_job_finish(StreamJob &J) {
    int groups = 0;
    for (int i = 0; i < J.nseg; ++i) {
        J.seg[i].group_begin = groups;
        groups += (J.seg[i].n + R - 1) / R;
    }
    J.total_groups = groups;
    J.nsb = J.Kpad / SB;
    J.nchunks = (J.nsb + KC - 1) / KC;
    J.bytes_full = (unsigned)chunk_row_bytes(J.qt, 0, J.nsb);
    J.bytes_tail = (unsigned)chunk_row_bytes(J.qt, J.nchunks - 1, J.nsb);
    J.tile_group_stride = tile_off(J.qt, 1, 0, 0, J.nsb);              // both offsets are linear in their index
    J.tile_chunk_stride = (int)tile_off(J.qt, 0, 1, 0, J.nsb);
}

void stream_assign_teams(StreamJob *jobs, int n) {
    // greedy: each job goes to the team whose streamed bytes per warp are lower so far
    // (team 0 has 8 of the 15 consumer warps, team 1 has 7)
    const double warps[2] = {(kMaxWarps + 1) / 2, kMaxWarps / 2};
    double load[2] = {0, 0};
    for (int i = 0; i < n; ++i) {
        double bytes = 0;
        for (int s = 0; s < jobs[i].nseg; ++s) bytes += (double)jobs[i].seg[s].n * jobs[i].row_bytes;
        const int t = (load[1] + bytes) / warps[1] < (load[0] + bytes) / warps[0] ? 1 : 0;
        jobs[i].team = t;
        load[t] += bytes;
    }
}

// Returns cudaSuccess, or cudaErrorInvalidValue when the shapes cannot be staged in shared memory.
cudaError_t stream_launch(const StreamLaunch &a, cudaStream_t st) {
    if (a.njobs <= kMaxJobsPerLaunch) return stream_launch_one(a, st);
    if (!a.jobs_dev || !a.jobs_host) return cudaErrorInvalidValue;
    for (int j0 = 0; j0 < a.njobs; j0 += kMaxJobsPerLaunch) {   // long plans: several launches in a row
        StreamLaunch part = a;
        part.jobs_host = a.jobs_host + j0;
        part.jobs_dev = a.jobs_dev + j0;
        part.njobs = std::min(kMaxJobsPerLaunch, a.njobs - j0);
        cudaError_t e = stream_launch_one(part, st);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t gemv_set_wait_limit_ns(unsigned long long ns) { return cudaMemcpyToSymbol(s_wait_limit_ns, &ns, sizeof(ns)); }

}  // namespace b200q
