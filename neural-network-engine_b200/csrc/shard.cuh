// Shared between shard.cu (group management, push kernel) and the forward kernels that store
// their results into every rank's window themselves: the per-launch description of the peers and
// the device-side arrival protocol.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#ifdef __CUDACC__
#include "ptx.cuh"
#endif

namespace nne {

constexpr int SHARD_MAX_RANKS = 8;

// What a kernel needs to reach the other ranks' windows.  world == 0: no exchange.
struct PeerSet {
    int world = 0, rank = 0;
    unsigned long long target = 0;        // every arrival word reaches this when the run is complete
    long long delta[SHARD_MAX_RANKS] = {};  // byte distance from an address in this rank's window to the
                                            // same place in rank p's window as mapped here (0 for itself)
    unsigned long long *flags = nullptr;  // this rank's arrival words [world], in its own window
};

// One slice to copy out: rows x width floats at y (inside this rank's window), row stride ldy.
struct PushSeg {
    float *y;
    size_t ldy;
    unsigned int rows, width;
    int vec;  // y, ldy and width allow 16-byte accesses
};

#ifdef __CUDACC__
// Announces this rank's runs up to number `upto` (epoch * 2^32) to every rank: raises the word
// "from ps.rank" in every window.  Called by one thread of a kernel that runs AFTER the producing kernels have
// completed (stream order), so their stores - local and remote - are already performed; the fence
// makes the announcement a release that carries them.
__device__ __forceinline__ void shard_publish(const PeerSet &ps, unsigned long long upto) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
#pragma unroll
    for (int p = 0; p < SHARD_MAX_RANKS; ++p) {
        if (p < ps.world) {
            unsigned long long *word = reinterpret_cast<unsigned long long *>(
                                           reinterpret_cast<char *>(ps.flags) + ps.delta[p]) + ps.rank;
            asm volatile("red.relaxed.sys.global.max.u64 [%0], %1;" ::"l"(word), "l"(upto) : "memory");
        }
    }
}

// Waits until every source's arrival word in THIS rank's window has reached the run's target.
// Bounded like every wait in this library; on expiry sets the context's error word and returns false.
__device__ __forceinline__ bool shard_wait_all(const PeerSet &ps, volatile int *abort_flag, int *err,
                                               int where, unsigned long long limit_ns = WAIT_LIMIT_NS) {
    const unsigned long long t0 = globaltimer_ns();
    for (int s = 0; s < ps.world; ++s) {
        unsigned int spins = 0;
        for (;;) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ps.flags + s) : "memory");
            if (v >= ps.target) break;
            if ((++spins & 0xff) == 0) {
                if (*abort_flag) return false;
                if (globaltimer_ns() - t0 > limit_ns) {
                    *abort_flag = 1;
                    *reinterpret_cast<volatile int *>(err) = 0x100 + where;
                    __threadfence_system();
                    return false;
                }
            }
        }
    }
    return true;
}
#endif

}  // namespace nne

struct nne_shard_group {
    nne_ctx *ctx = nullptr;
    int rank = 0, world = 1;
    uint8_t *base = nullptr;   // this rank's window (+ arrival words behind it)
    size_t bytes = 0;          // whole allocation
    size_t flag_off = 0;       // offset of the arrival words = usable window size
    uint8_t *peer[nne::SHARD_MAX_RANKS] = {};  // every rank's window as mapped in this process
    bool ipc = false, connected = false;
    void *nccl_comm = nullptr;
    std::atomic<unsigned long long> epoch{0};  // sharded runs issued on this group so far
};

namespace nne {

PeerSet shard_peerset(const nne_shard_group *g, unsigned long long epoch);
int shard_push(nne_shard_group *g, const PushSeg *segs_dev, int count, size_t floats_total,
               unsigned long long epoch, cudaStream_t s);
int shard_wait(nne_shard_group *g, unsigned long long epoch, cudaStream_t s);
int shard_nccl_all_gather(nne_shard_group *g, const void *send, void *recv, size_t count_floats,
                          cudaStream_t s);
int shard_nccl_group_start();
int shard_nccl_group_end();
int shard_interleave(nne_ctx *ctx, const float *staged, float *y, int world, size_t m, size_t w,
                     size_t ldy, cudaStream_t s);

}  // namespace nne
