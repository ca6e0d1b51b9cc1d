// Shared host-side plumbing of the nne_cuda library: status/error text, the per-device context,
// the layer handle, and the launch counter.  Kernels live in quantize.cu, gemv.cu, prefill.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <atomic>
#include <mutex>
#include <string>

#include "../../include/nne_cuda.h"

namespace nne {

// ---- thread-local error text -------------------------------------------------------------
std::string &last_error_ref();
int fail(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define NNE_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) {                                                            \
            int st__ = (e__ == cudaErrorMemoryAllocation) ? NNE_ERR_OUT_OF_MEMORY            \
                                                          : NNE_ERR_CUDA;                    \
            return ::nne::fail(st__, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                               __FILE__, __LINE__);                                          \
        }                                                                                    \
    } while (0)

#define NNE_TRY(expr)                      \
    do {                                   \
        int st__ = (expr);                 \
        if (st__ != NNE_OK) return st__;   \
    } while (0)

// Every extern "C" body is wrapped so that no C++ exception can cross the boundary.
#define NNE_GUARD_BEGIN try {
#define NNE_GUARD_END                                                              \
    }                                                                              \
    catch (const std::bad_alloc &) {                                               \
        return ::nne::fail(NNE_ERR_OUT_OF_MEMORY, "host allocation failed");       \
    }                                                                              \
    catch (const std::exception &ex) {                                             \
        return ::nne::fail(NNE_ERR_INVALID_ARGUMENT, "exception: %s", ex.what());  \
    }                                                                              \
    catch (...) {                                                                  \
        return ::nne::fail(NNE_ERR_INVALID_ARGUMENT, "unknown exception");         \
    }

// Longest row the integer tensor-core kernels take: |q| <= 128 times a digit |d| <= 128 is 2^14, and
// an int32 accumulator in TMEM adds in_features of those, so sums stay exact below 2^17 terms.
constexpr size_t NNE_TENSOR_INT_MAX_K = ((size_t)1 << 17) - 1;

// ---- launch counter ----------------------------------------------------------------------
extern std::atomic<uint64_t> g_launches;
// Programmatic dependent launch is on unless NNE_PDL=0.
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNE_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}
inline void count_launch(int n = 1) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// Checks the launch that was just issued.
#define NNE_LAUNCH_CHECK()                                                               \
    do {                                                                                 \
        ::nne::count_launch();                                                           \
        cudaError_t e__ = cudaGetLastError();                                            \
        if (e__ != cudaSuccess)                                                          \
            return ::nne::fail(NNE_ERR_CUDA, "kernel launch failed: %s (%s:%d)",         \
                               cudaGetErrorString(e__), __FILE__, __LINE__);             \
    } while (0)

// Raises a kernel's MaxDynamicSharedMemorySize to at least `bytes` on `device` (the attribute is
// per device, so it is tracked per (device, kernel) and only ever raised; safe from any thread).
// The device must be the calling thread's current one.
int ensure_dynamic_smem(int device, const void *func, size_t bytes);
template <typename K>
inline int ensure_dynamic_smem(int device, K *kernel, size_t bytes) {
    return ensure_dynamic_smem(device, reinterpret_cast<const void *>(kernel), bytes);
}

// A device buffer that only ever grows; used for host-call staging and kernel workspaces.
struct GrowBuf {
    void *ptr = nullptr;
    size_t cap = 0;
    int reserve(size_t bytes);
    void release();
};

}  // namespace nne

// ---- opaque handles ------------------------------------------------------------------------
struct nne_ctx {
    int device = 0;
    int sm_count = 0;
    int reserved_sms = 0;  // SMs the persistent streaming kernel leaves free (nne_cuda_ctx_reserve_sms)
    int cc_major = 0, cc_minor = 0;
    size_t total_mem = 0;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;  // used by the *_host entry points
    std::mutex mu;                  // serialises *_host calls and workspace growth
    nne::GrowBuf stage_a, stage_b, stage_c;  // host-call staging (inputs / outputs)
    unsigned int *absmax_word = nullptr;     // 4-byte scratch for the per-tensor absmax
    int *err_word = nullptr;                 // device address of the error word: a kernel's bounded wait ran out
    volatile int *err_host = nullptr;        // the same word as the host sees it (mapped pinned memory)
};

struct nne_qlinear {
    nne_ctx *ctx = nullptr;
    int device = 0;           // copy of ctx->device, so destroy works after the context is gone
    size_t n = 0, k = 0;
    int8_t *q = nullptr;      // [n, k] row-major codes
    float *scales = nullptr;  // [n]
    float *bias = nullptr;    // [n] or null
    bool own = true;
    void *tmap_w = nullptr;   // host copy of the TMA descriptor of q (bf16 tensor path), or null
    void *tmap_w8 = nullptr;  // host copy of the swizzled TMA descriptor of q (int8 tensor path)
    void *tmap_wsk = nullptr; // same with 128-row boxes (small-batch tensor path)
};

namespace nne {

// Sets the calling thread's current device to the context's.
inline int use_ctx(const nne_ctx *ctx) {
    if (!ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null context");
    NNE_CUDA_TRY(cudaSetDevice(ctx->device));
    return NNE_OK;
}

// kernels' host launchers (defined next to the kernels) ---------------------------------------
struct PeerSet;  // shard.cuh: the other ranks' windows, for a column shard's launch
int launch_quantize_rows(nne_ctx *ctx, const float *w, size_t rows, size_t cols, int8_t *q,
                         float *scales, cudaStream_t s);
int launch_quantize_tensor(nne_ctx *ctx, const float *v, size_t n, int8_t *q, float *scale_dev,
                           unsigned int *absmax_word, cudaStream_t s);
int launch_dequantize_rows(nne_ctx *ctx, const int8_t *q, const float *scales, size_t rows,
                           size_t cols, float *out, cudaStream_t s);

bool gemv_supports(size_t n, size_t k, size_t m);
int launch_gemv(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                cudaStream_t s);
// One layer of a streaming launch (gemv_tma.cu).  x [m, k] and y [m, .] row stride ldy floats.
struct StreamLayer {
    const int8_t *q;
    const float *scales;
    const float *bias;  // or null
    const float *x;
    float *y;
    size_t ldy;
    int n, k;
    int rw;  // weight rows per ring stage: stream_rows_per_stage(k)
    // What the layer multiplies is x' = x (both null), RMSNorm(x) = (x * rrms) * gamma (gamma set), or
    // silu(x) * x2 (x2 set, [m, k]); what it writes is forward(x') + residual (residual set, laid out
    // like y).  The steps either side of a QLinear in a decoder block, done where x and y pass anyway.
    float eps = 0.0f;
    const float *gamma = nullptr;
    const float *x2 = nullptr;
    const float *residual = nullptr;
    // 1: the layer reads or overwrites something an earlier layer of the same launch writes (or
    // overwrites something one reads); the grid meets before its activations are prepared
    int sync = 0;
    // 1: x, its transform and k are those of the layer before it in the list (and nothing wrote x in
    // between): the kernel reuses that layer's prepared activations
    int same_input = 0;
};
// The decode kernels (streaming GEMV, small-batch tensor-core kernel) put an activation row on the
// grid 2^-e with |v| = |rint(x * 2^e)| < 2^ACT_GRID_BITS and split v into ACT_PLANES balanced int8
// digits of base 2^ACT_DIGIT_BITS.  Two base-256 digits (16 bits): the rounding of x to the grid is
// then at most 2^-15 of the row's largest |x| per element, i.e. a result error of at most 3 % of the
// path's tolerance (1e-3 * ||x||inf * scale_j * sum|q_jk|) and typically 0.1 % of it, for two dot
// products per weight instead of three.  (Three base-128 digits, 2^-21, were the first form.)
#ifndef NNE_DIGIT_PLANES
#define NNE_DIGIT_PLANES 2
#endif
constexpr int ACT_PLANES = NNE_DIGIT_PLANES;
constexpr int ACT_DIGIT_BITS = ACT_PLANES == 3 ? 7 : 8;
constexpr int ACT_GRID_BITS = ACT_PLANES == 3 ? 20 : 15;
// Exponent e of the grid for a row whose largest |x| is `big` (> 0, finite): big * 2^e lies in
// [2^(ACT_GRID_BITS-1), 2^ACT_GRID_BITS); with two planes the top digit must stay below 128 after
// the low one has been split off, hence the margin at the top of the binade.
__host__ __device__ inline int act_grid_exponent(float big) {
    int e = ACT_GRID_BITS - 1 - ((big > 0.0f) ? ilogbf(big) : 0);
    if (ACT_PLANES == 2 && scalbnf(big, e) > 32639.0f) --e;
    return e;
}
constexpr int STREAM_INLINE_LAYERS = 8;  // descriptors passed in the kernel's parameter block
struct StreamBatch {
    int count;
    int reuse;  // the same weights appear again later in the list: do not mark them evict-first
    const StreamLayer *dev;  // device copy of the descriptors when count > STREAM_INLINE_LAYERS
    int chain;     // some layer has `sync` or `same_input` set: the launch takes the kernel instance with those paths
    int pf_bytes;  // how far the weight stream's L2 look-ahead runs in front of the ring (0: off)
#ifdef NNE_TRACE
    unsigned long long *trace;  // debug builds: time stamps
#endif
    unsigned long long *gsync;  // arrival counter of the launch's rendezvous, or null (no chained layer)
    StreamLayer inl[STREAM_INLINE_LAYERS];
};
int stream_rows_per_stage(size_t k);
bool gemv_tma_supports(size_t n, size_t k, size_t m);  // m = rows of one launch, 1..2
int launch_gemv_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                    const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                    cudaStream_t s);
int launch_gemv_tma_passes(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                           const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                           cudaStream_t s);
int launch_stream_batch(nne_ctx *ctx, const StreamLayer *host, const StreamLayer *dev, int count,
                        size_t m, bool reuse, cudaStream_t s, const PeerSet *peers = nullptr,
                        unsigned long long *gsync = nullptr);
int launch_generic(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                   const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                   cudaStream_t s);

int launch_rmsnorm(nne_ctx *ctx, const float *x, const float *gamma, float eps, size_t rows, size_t cols,
                   float *y, cudaStream_t s);
int launch_silu_mul(nne_ctx *ctx, const float *gate, const float *up, size_t n, float *out, cudaStream_t s);
int launch_add(nne_ctx *ctx, const float *a, const float *b, size_t n, float *out, cudaStream_t s);
// Copies between pinned host memory and device buffers done by a kernel (elementwise.cu).
constexpr int HOST_COPY_SEGS = 8;
struct HostCopySegs {
    int count;
    struct {
        const float *src;
        float *dst;
        size_t n4;  // float4 elements
    } seg[HOST_COPY_SEGS];
};
int launch_host_copy(nne_ctx *ctx, const HostCopySegs &segs, bool results_of_previous_kernel, cudaStream_t s);

bool prefill_supports(const nne_qlinear *ql, size_t m);
int prefill_prepare_layer(nne_qlinear *ql);  // builds the weight TMA descriptor
void prefill_release_layer(nne_qlinear *ql);
int launch_prefill(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy,
                   cudaStream_t s);
bool skinny_supports(const nne_qlinear *ql, size_t m);
int skinny_prepare_layer(nne_qlinear *ql);
void skinny_release_layer(nne_qlinear *ql);
int launch_skinny(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy, cudaStream_t s);
struct SkPlan;  // several small-batch forwards as one launch (skinny.cu)
bool skinny_plan_supports(nne_qlinear *const *layers, const float *const *x, float *const *y,
                          size_t count, size_t m);
int skinny_plan_create(nne_ctx *ctx, nne_qlinear *const *layers, const float *const *x, float *const *y,
                       const size_t *ldy_or_null, size_t count, size_t m, SkPlan **out);
int skinny_plan_run(SkPlan *plan, cudaStream_t s);
void skinny_plan_destroy(SkPlan *plan);
bool prefill_i8_supports(const nne_qlinear *ql, size_t m);
int prefill_i8_prepare_layer(nne_qlinear *ql);
void prefill_i8_release_layer(nne_qlinear *ql);
int launch_prefill_i8(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy,
                      cudaStream_t s, const PeerSet *peers = nullptr);

}  // namespace nne

#include <vector>

struct nne_shard_group;
namespace nne {
struct PushSeg;
}

struct nne_plan {
    nne_ctx *ctx = nullptr;
    size_t m = 0;
    bool fused = false;  // the whole list runs as one streaming launch
    std::vector<nne_qlinear *> layers;
    std::vector<const float *> x;
    std::vector<float *> y;      // where this plan's kernels write layer i (a shard: its slice of y_full)
    std::vector<size_t> ldy;     // row stride of y[i] in floats
    std::vector<nne::StreamLayer> descs;
    nne::StreamLayer *descs_dev = nullptr;
    // Items that consume earlier items' outputs: one streaming launch whose grid meets between them
    // (gsync_dev: its arrival counter), or - other kernels - sub-plans run one after another.
    unsigned long long *gsync_dev = nullptr;
    std::vector<nne_plan *> phases;
    nne::SkPlan *skinny = nullptr;  // 2 <= m <= 16: the whole list as one small-batch launch
    // Input transforms and residual adds (nne_qlinear_plan_create_fused) where the forward kernels
    // of this plan do not do them themselves: standalone launches before / after, into plan-owned
    // buffers.  Empty for a streaming plan, whose kernel takes them in its stride.
    struct PreOp {
        int kind;  // 1 = RMSNorm, 2 = silu(x) * x2
        const float *x, *aux;  // aux: gamma or x2
        float eps;
        float *dst;
        size_t rows, cols;
    };
    struct PostOp {
        float *y;
        const float *residual;
        size_t count;
    };
    std::vector<PreOp> pre_ops;
    std::vector<PostOp> post_ops;
    float *xform_buf = nullptr;
    // column shards (nne_qlinear_plan_create_sharded); group == nullptr for an ordinary plan
    nne_shard_group *group = nullptr;
    int route = 0;                    // 0 = peer stores, 1 = NCCL all-gather
    std::vector<float *> y_full;      // [m, n_total[i]] in this rank's window
    std::vector<size_t> n_total, row_begin;
    nne::PushSeg *segs_dev = nullptr; // the slices to copy out when the forward kernels do not do it themselves
    int seg_count = 0;
    std::vector<char> stores_itself;  // per layer: its forward kernel stores into every window
    size_t push_floats = 0;
    float *staging = nullptr;         // NCCL route, m > 1: [world][m][width] of the widest layer
};
