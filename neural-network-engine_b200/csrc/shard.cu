// Column shards over the GPUs of one node: the exchange of output slices.
//
// The path shards by output channel (reference src/nn/quantized.rs:184-192: channel j reads only
// row j of qweight, scales[j] and bias[j]), so rank g of G computes columns [b_g, e_g) of
// y [m, N_total] and every rank needs all of them afterwards - an all-gather.  Two routes:
//
//  * peer stores (the default).  Every rank owns a WINDOW of device memory that all peers map
//    (CUDA IPC between processes, peer access inside one process).  Outputs live at the same
//    offset in every window, so "gather" means: write your slice into all G windows.  For decode
//    shapes the streaming GEMV does that itself - its finishing lanes store each result to every
//    window (gemv_tma.cu) - and for every other shape shard_push_kernel below copies the slice
//    out after the local forward.  Plain st.global to peer-mapped memory only: no multicast
//    object, no TMA to or from a peer.  A run is split in two, like a non-blocking collective:
//    the producing kernels only store (they neither announce nor wait); nne_shard_group_wait then
//    enqueues a one-warp kernel that announces this rank's completed runs in every window (one
//    64-bit word per source rank) and waits, bounded at about 2 s, until every rank has announced
//    as much - at which point this rank's window holds every slice.  Every rank must call it.
//  * NCCL (north star's baseline): ncclAllGather on a communicator the host created.  The library
//    resolves the NCCL entry points at run time from the copy the process has already loaded.
//
// Ordering rules for callers: all ranks issue the same sequence of sharded runs and waits on a
// group, like collectives; a wait goes on a stream that is ordered after the runs it completes.  A
// rank may overwrite an output area only when every peer has finished READING what the area held.
// With run, wait and the reads in one stream, "a peer has announced run e+1" implies "it has read
// run e", so two areas that alternate are enough; a caller that keeps d runs in flight before it
// waits needs 2 d areas.
#include <dlfcn.h>
#include <string.h>

#include <atomic>
#include <memory>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"
#include "shard.cuh"

namespace nne {
namespace {

// ---- push kernel ----------------------------------------------------------------------------
// Copies this rank's slices (rows x width floats at row stride ldy) from its own window to the
// same place in every other window.
__global__ void __launch_bounds__(256)
shard_push_kernel(const PushSeg *__restrict__ segs, int count, const PeerSet ps) {
    // the slices are the output of the previous kernels in the stream
    grid_dependency_wait();
    grid_launch_dependents();
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    for (int si = 0; si < count; ++si) {
        const PushSeg sg = segs[si];
        if (sg.rows == 0 || sg.width == 0) continue;
        if (sg.vec) {
            const size_t w4 = sg.width >> 2;
            const size_t total = (size_t)sg.rows * w4;
            for (size_t i = tid; i < total; i += nthreads) {
                const size_t r = i / w4, c = i - r * w4;
                float *p = sg.y + r * sg.ldy + 4 * c;
                const float4 v = *reinterpret_cast<const float4 *>(p);
#pragma unroll
                for (int q = 0; q < SHARD_MAX_RANKS; ++q)
                    if (q < ps.world && q != ps.rank)
                        *reinterpret_cast<float4 *>(reinterpret_cast<char *>(p) + ps.delta[q]) = v;
            }
        } else {
            const size_t total = (size_t)sg.rows * sg.width;
            for (size_t i = tid; i < total; i += nthreads) {
                const size_t r = i / sg.width, c = i - r * sg.width;
                float *p = sg.y + r * sg.ldy + c;
                const float v = *p;
#pragma unroll
                for (int q = 0; q < SHARD_MAX_RANKS; ++q)
                    if (q < ps.world && q != ps.rank)
                        *reinterpret_cast<float *>(reinterpret_cast<char *>(p) + ps.delta[q]) = v;
            }
        }
    }
}

// The second half of the exchange, one warp: announces this rank's runs up to ps.target to every
// rank - the producing kernels precede this kernel in stream order, so their stores, local and
// remote, are complete - and then waits (bounded) until every rank has announced as much, i.e.
// until this rank's window holds every slice of those runs.  Small enough to sit on an SM beside a
// CTA of the persistent decode kernel, so on a second stream it overlaps the next run.
// (Announcing from inside the producing kernels was measured and dropped: a fence that waits for
// the NVLink acknowledgements in every CTA cost 8 us on a 72 us launch, and an announcing kernel
// between two forwards in one stream as much.)
__global__ void __launch_bounds__(32)
shard_wait_kernel(const PeerSet ps, int *err) {
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        shard_publish(ps, ps.target);
        (void)shard_wait_all(ps, &abort_flag, err, 0x51);
    }
}

// [G][m][w] (what an all-gather of per-rank [m, w] blocks returns) -> row-major [m, G*w] at row
// stride ldy.
__global__ void __launch_bounds__(256)
shard_interleave_kernel(const float *__restrict__ staged, float *__restrict__ y, int world, size_t m,
                        size_t w, size_t ldy) {
    const size_t total = (size_t)world * m * w;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t g = i / (m * w), rem = i - g * (m * w);
        const size_t r = rem / w, c = rem - r * w;
        y[r * ldy + g * w + c] = staged[i];
    }
}

// Failure-path check, no fault involved: one CTA waits on something that will never happen - an
// mbarrier nobody arrives at (which = 0), or an arrival word that nothing raises (which = 1) - with
// a short limit.  The wait must give up, set the context's error word and let the kernel return.
__global__ void __launch_bounds__(32)
wait_selftest_kernel(int which, unsigned long long limit_ns, unsigned long long *never_raised, int *err) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        if (which == 0) {
            (void)mbar_wait(smem_u32(&bar), 0, &abort_flag, err, 0x7e, limit_ns);
        } else {
            PeerSet ps;
            ps.world = 1;
            ps.rank = 0;
            ps.target = ~0ull;
            ps.flags = never_raised;
            (void)shard_wait_all(ps, &abort_flag, err, 0x7f, limit_ns);
        }
    }
}

// ---- NCCL, resolved at run time ----------------------------------------------------------------
struct NcclApi {
    int (*all_gather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*group_start)() = nullptr;
    int (*group_end)() = nullptr;
    const char *(*error_string)(int) = nullptr;
    bool ok = false;
};

const NcclApi &nccl_api() {
    static const NcclApi api = [] {
        NcclApi a;
        // The copy the process already uses (the one that made the caller's communicator) first;
        // NNE_NCCL_LIB names another.
        const char *env = getenv("NNE_NCCL_LIB");
        void *h = env ? dlopen(env, RTLD_NOW | RTLD_GLOBAL) : nullptr;
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return a;
        a.all_gather = reinterpret_cast<decltype(a.all_gather)>(dlsym(h, "ncclAllGather"));
        a.group_start = reinterpret_cast<decltype(a.group_start)>(dlsym(h, "ncclGroupStart"));
        a.group_end = reinterpret_cast<decltype(a.group_end)>(dlsym(h, "ncclGroupEnd"));
        a.error_string = reinterpret_cast<decltype(a.error_string)>(dlsym(h, "ncclGetErrorString"));
        a.ok = a.all_gather && a.group_start && a.group_end;
        return a;
    }();
    return api;
}

int nccl_fail(int rc, const char *what) {
    const NcclApi &a = nccl_api();
    return fail(NNE_ERR_NCCL, "%s failed: %s", what, a.error_string ? a.error_string(rc) : "NCCL error");
}

constexpr int NCCL_FLOAT32 = 7;

}  // namespace

PeerSet shard_peerset(const nne_shard_group *g, unsigned long long epoch) {
    PeerSet ps;
    ps.world = g->world;
    ps.rank = g->rank;
    ps.target = epoch << 32;
    ps.flags = reinterpret_cast<unsigned long long *>(g->base + g->flag_off);
    for (int p = 0; p < SHARD_MAX_RANKS; ++p)
        ps.delta[p] = (p < g->world && g->peer[p]) ? (long long)(g->peer[p] - g->base) : 0;
    return ps;
}

int shard_push(nne_shard_group *g, const PushSeg *segs_dev, int count, size_t floats_total,
               unsigned long long epoch, cudaStream_t s) {
    const PeerSet ps = shard_peerset(g, epoch);
    size_t blocks = (floats_total / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    // A copy to G - 1 peers is bound by NVLink, not by SMs: for the small slices of decode-sized
    // forwards one CTA per SM keeps the links busy.  A large slice (tens of MB: a prefill output) needs
    // more stores in flight than that - 148 CTAs moved 205 MB to seven peers at 320 GB/s - so it gets
    // four CTAs per SM.
    size_t cap = (size_t)(g->ctx->sm_count > 4 ? g->ctx->sm_count / 4 : 1) * 4;
    if (floats_total * sizeof(float) >= ((size_t)16 << 20)) cap *= 4;
    if (blocks > cap) blocks = cap;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = pdl;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, shard_push_kernel, segs_dev, count, ps);
    count_launch();
    if (e != cudaSuccess) return fail(NNE_ERR_CUDA, "slice push launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

int shard_wait(nne_shard_group *g, unsigned long long epoch, cudaStream_t s) {
    if (g->world <= 1 || epoch == 0) return NNE_OK;
    const PeerSet ps = shard_peerset(g, epoch);
    shard_wait_kernel<<<1, 32, 0, s>>>(ps, g->ctx->err_word);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

int shard_nccl_all_gather(nne_shard_group *g, const void *send, void *recv, size_t count_floats,
                          cudaStream_t s) {
    const NcclApi &a = nccl_api();
    if (!a.ok) return fail(NNE_ERR_NCCL, "no NCCL library could be resolved in this process");
    if (!g->nccl_comm) return fail(NNE_ERR_NCCL, "the group has no NCCL communicator (nne_shard_group_set_nccl)");
    const int rc = a.all_gather(send, recv, count_floats, NCCL_FLOAT32, g->nccl_comm, s);
    if (rc != 0) return nccl_fail(rc, "ncclAllGather");
    return NNE_OK;
}
int shard_nccl_group_start() {
    const NcclApi &a = nccl_api();
    if (!a.ok) return fail(NNE_ERR_NCCL, "no NCCL library could be resolved in this process");
    const int rc = a.group_start();
    return rc == 0 ? NNE_OK : nccl_fail(rc, "ncclGroupStart");
}
int shard_nccl_group_end() {
    const NcclApi &a = nccl_api();
    const int rc = a.group_end();
    return rc == 0 ? NNE_OK : nccl_fail(rc, "ncclGroupEnd");
}

int shard_interleave(nne_ctx *ctx, const float *staged, float *y, int world, size_t m, size_t w,
                     size_t ldy, cudaStream_t s) {
    const size_t total = (size_t)world * m * w;
    if (total == 0) return NNE_OK;
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    shard_interleave_kernel<<<(unsigned)blocks, 256, 0, s>>>(staged, y, world, m, w, ldy);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

}  // namespace nne

using namespace nne;

extern "C" {

int nne_cuda_ctx_selftest_wait(nne_ctx *ctx, int which, unsigned int limit_us) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (which != 0 && which != 1) return fail(NNE_ERR_INVALID_ARGUMENT, "which must be 0 or 1");
    if (limit_us == 0 || limit_us > 1000000u)
        return fail(NNE_ERR_INVALID_ARGUMENT, "limit must be 1..1000000 microseconds");
    // the context's 256-byte scratch block is zero beyond its first word: bytes 8..15 serve as the
    // arrival word that never reaches its target
    wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(which, (unsigned long long)limit_us * 1000ull,
                                                   reinterpret_cast<unsigned long long *>(ctx->absmax_word + 2),
                                                   ctx->err_word);
    NNE_LAUNCH_CHECK();
    NNE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_shard_group_create(nne_ctx *ctx, int rank, int world, size_t window_bytes,
                           nne_shard_group **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    if (world < 1 || world > SHARD_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NNE_ERR_INVALID_ARGUMENT, "rank %d of %d: a group holds 1..%d ranks", rank, world,
                    SHARD_MAX_RANKS);
    if (window_bytes > ((size_t)1 << 46)) return fail(NNE_ERR_INVALID_ARGUMENT, "window too large");
    std::unique_ptr<nne_shard_group> g(new nne_shard_group());
    g->ctx = ctx;
    g->rank = rank;
    g->world = world;
    g->flag_off = (window_bytes + 255) & ~(size_t)255;
    g->bytes = g->flag_off + 256;
    // cudaMalloc, not the stream-ordered pool: the allocation is exported to other processes.
    NNE_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&g->base), g->bytes));
    cudaError_t e = cudaMemset(g->base, 0, g->bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(g->base);
        return fail(NNE_ERR_CUDA, "window set-up failed: %s", cudaGetErrorString(e));
    }
    g->peer[rank] = g->base;
    g->connected = (world == 1);
    *out = g.release();
    return NNE_OK;
    NNE_GUARD_END
}

int nne_shard_group_handle(const nne_shard_group *g, void *handle_out) {
    NNE_GUARD_BEGIN
    if (!g || !handle_out) return fail(NNE_ERR_INVALID_ARGUMENT, "null group or handle buffer");
    NNE_TRY(use_ctx(g->ctx));
    static_assert(sizeof(cudaIpcMemHandle_t) == NNE_SHARD_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    NNE_CUDA_TRY(cudaIpcGetMemHandle(&h, g->base));
    memcpy(handle_out, &h, sizeof(h));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_shard_group_connect(nne_shard_group *g, const void *all_handles) {
    NNE_GUARD_BEGIN
    if (!g || !all_handles) return fail(NNE_ERR_INVALID_ARGUMENT, "null group or handle table");
    if (g->connected) return fail(NNE_ERR_INVALID_ARGUMENT, "the group is already connected");
    NNE_TRY(use_ctx(g->ctx));
    const char *tab = static_cast<const char *>(all_handles);
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, tab + (size_t)p * NNE_SHARD_HANDLE_BYTES, sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int q = 0; q < p; ++q)
                if (q != g->rank && g->peer[q]) {
                    cudaIpcCloseMemHandle(g->peer[q]);
                    g->peer[q] = nullptr;
                }
            return fail(NNE_ERR_CUDA, "mapping rank %d's window failed: %s", p, cudaGetErrorString(e));
        }
        g->peer[p] = static_cast<uint8_t *>(ptr);
    }
    g->ipc = true;
    g->connected = true;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_shard_group_connect_local(nne_shard_group *g, nne_shard_group *const *all_groups) {
    NNE_GUARD_BEGIN
    if (!g || !all_groups) return fail(NNE_ERR_INVALID_ARGUMENT, "null group or group table");
    if (g->connected) return fail(NNE_ERR_INVALID_ARGUMENT, "the group is already connected");
    NNE_TRY(use_ctx(g->ctx));
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank) continue;
        const nne_shard_group *o = all_groups[p];
        if (!o || o->rank != p || o->world != g->world || o->bytes != g->bytes)
            return fail(NNE_ERR_INVALID_ARGUMENT, "entry %d of the group table does not match", p);
        int can = 0;
        NNE_CUDA_TRY(cudaDeviceCanAccessPeer(&can, g->ctx->device, o->ctx->device));
        if (!can)
            return fail(NNE_ERR_UNSUPPORTED, "device %d cannot map device %d's memory", g->ctx->device,
                        o->ctx->device);
        cudaError_t e = cudaDeviceEnablePeerAccess(o->ctx->device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
            return fail(NNE_ERR_CUDA, "enabling peer access failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        g->peer[p] = o->base;
    }
    g->ipc = false;
    g->connected = true;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_shard_group_window(const nne_shard_group *g, void **base, size_t *bytes) {
    if (!g) return fail(NNE_ERR_INVALID_ARGUMENT, "null group");
    if (base) *base = g->base;
    if (bytes) *bytes = g->flag_off;
    return NNE_OK;
}

int nne_shard_group_wait(nne_shard_group *g, void *stream) {
    NNE_GUARD_BEGIN
    if (!g) return fail(NNE_ERR_INVALID_ARGUMENT, "null group");
    NNE_TRY(use_ctx(g->ctx));
    return shard_wait(g, g->epoch.load(), (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_shard_group_set_nccl(nne_shard_group *g, void *nccl_comm) {
    if (!g) return fail(NNE_ERR_INVALID_ARGUMENT, "null group");
    g->nccl_comm = nccl_comm;
    return NNE_OK;
}

int nne_shard_group_destroy(nne_shard_group *g) {
    NNE_GUARD_BEGIN
    if (!g) return NNE_OK;
    cudaSetDevice(g->ctx->device);
    cudaDeviceSynchronize();
    if (g->ipc)
        for (int p = 0; p < g->world; ++p)
            if (p != g->rank && g->peer[p]) cudaIpcCloseMemHandle(g->peer[p]);
    if (g->base) cudaFree(g->base);
    cudaGetLastError();
    delete g;
    return NNE_OK;
    NNE_GUARD_END
}

}  // extern "C"
