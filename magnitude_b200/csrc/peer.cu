// One-shot all-reduce over NVLink peer memory for the small vectors of a row-parallel decode
// projection (a few thousand floats per token): every rank stores its partial sums straight into
// a slot of every rank's exchange buffer and then adds up, in rank order, what all ranks stored into
// its own buffer, so all ranks get bit-identical sums.  Plain peer stores and loads only: no
// multimem, no TMA, no NCCL.  A ring all-reduce moves fewer bytes, but at this size the cost is
// latency, and one store per peer is the shortest path.
//
// Each element is stored as one 8-byte pair (value bits, call number).  The reader polls the pair
// until it carries the current call's number; there is no flag to raise and no fence to wait for.
// Calls alternate between two slot sets: block b of a rank stores call e + 2 only after it has read
// block b's range of call e + 1 from every rank, and a rank stores call e + 1 only after reading
// call e, so a pair is never overwritten before it has been read.  The call number lives in device
// memory (one counter per block), which keeps a launch replayable from a CUDA graph.  Block b owns a
// fixed element range and every block counts every call, so counts may change from call to call.
// Every rank must make the same sequence of calls with the same counts.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace b200q {

namespace {

struct PeerParams {
    float *y;
    int count;
    int rank, world;
    uint8_t *base[kPeerMaxWorld];
    int *status;
};

__device__ __forceinline__ void st_pair(unsigned long long *p, float v, unsigned e) {
    const unsigned long long w = ((unsigned long long)e << 32) | __float_as_uint(v);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_pair(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerParams p) {
    const int b = blockIdx.x;
    uint8_t *local = p.base[p.rank];
    unsigned *epochs = reinterpret_cast<unsigned *>(local + kPeerEpochOff);
    __shared__ unsigned s_epoch;
    __shared__ int s_fail;
    if (threadIdx.x == 0) {
        s_epoch = epochs[b] + 1;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned e = s_epoch;
    const size_t set_off = (size_t)(e & 1) * kPeerMaxWorld * kPeerSlotFloats;
    // Block b always owns elements [1024 b, 1024 b + 1024), whatever the call's count, and every
    // block counts every call: a pair found under the current number can then only have been
    // stored by the same block of a peer for this very call.
    constexpr int per = kPeerSlotFloats / kPeerBlocks;
    const int lo = b * per, hi = min(lo + per, p.count);

    // 1. my partial sums -> slot [set][my rank] of every rank
    for (int i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
        const float v = p.y[i];
        for (int r = 0; r < p.world; ++r)
            st_pair(reinterpret_cast<unsigned long long *>(p.base[r] + kPeerSlotOff) + set_off + (size_t)p.rank * kPeerSlotFloats + i, v, e);
    }
    // 2. sum what every rank delivered here, in rank order (bounded wait per element)
    const unsigned long long *slots = reinterpret_cast<const unsigned long long *>(local + kPeerSlotOff) + set_off;
    for (int i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
        float acc = 0.f;
        bool ok = true;
        // all ranks' pairs are requested before the first is looked at: one trip to memory, not one per rank
        unsigned long long w[kPeerMaxWorld];
#pragma unroll
        for (int r = 0; r < kPeerMaxWorld; ++r)
            if (r < p.world) w[r] = ld_pair(slots + (size_t)r * kPeerSlotFloats + i);
#pragma unroll
        for (int r = 0; r < kPeerMaxWorld; ++r) {
            if (r >= p.world || !ok) continue;
            if ((unsigned)(w[r] >> 32) != e) {
                const unsigned long long *q = slots + (size_t)r * kPeerSlotFloats + i;
                const uint64_t t0 = globaltimer_ns();
                int spins = 0;
                while ((unsigned)((w[r] = ld_pair(q)) >> 32) != e) {
                    if ((++spins & 63) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
                        ok = false;
                        break;
                    }
                }
            }
            acc = r == 0 ? __uint_as_float((unsigned)w[r]) : acc + __uint_as_float((unsigned)w[r]);
        }
        if (ok) p.y[i] = acc;
        else s_fail = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_fail) atomicMax(p.status, DEV_ERR_PIPE_TIMEOUT);   // results of this call are invalid
        epochs[b] = e;                                            // also then: the ranks stay in step
    }
}

}  // namespace

cudaError_t peer_allreduce_launch(const PeerLaunch &a, cudaStream_t st) {
    if (a.world < 1 || a.world > kPeerMaxWorld || a.rank < 0 || a.rank >= a.world) return cudaErrorInvalidValue;
    if (a.count < 1 || a.count > kPeerSlotFloats) return cudaErrorInvalidValue;
    PeerParams p{};
    p.y = a.y;
    p.count = a.count;
    p.rank = a.rank;
    p.world = a.world;
    for (int r = 0; r < a.world; ++r) {
        if (!a.base[r]) return cudaErrorInvalidValue;
        p.base[r] = a.base[r];
    }
    p.status = a.status;
    // always the full grid, so that every block's call counter advances on every call
    peer_allreduce_kernel<<<kPeerBlocks, kPeerThreads, 0, st>>>(p);
    return cudaGetLastError();
}

cudaError_t peer_set_wait_limit_ns(unsigned long long ns) { return cudaMemcpyToSymbol(s_wait_limit_ns, &ns, sizeof(ns)); }

}  // namespace b200q
