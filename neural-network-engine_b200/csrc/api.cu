// extern "C" entry points of the nne_cuda library (declared in include/nne_cuda.h): argument
// checks, device memory ownership, host<->device staging and kernel dispatch.  The arithmetic
// lives in quantize.cu, gemv.cu and prefill.cu.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <memory>
#include <new>
#include <utility>
#include <vector>

#include "common.cuh"
#include "shard.cuh"

namespace nne {

std::atomic<uint64_t> g_launches{0};

std::string &last_error_ref() {
    thread_local std::string s;
    return s;
}

int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return status;
}

int ensure_dynamic_smem(int device, const void *func, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<int, const void *>, size_t> have;
    std::lock_guard<std::mutex> lock(mu);
    size_t &cur = have[std::make_pair(device, func)];
    if (bytes <= cur) return NNE_OK;
    NNE_CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    cur = bytes;
    return NNE_OK;
}

int GrowBuf::reserve(size_t bytes) {
    if (bytes <= cap) return NNE_OK;
    if (ptr) {
        cudaFree(ptr);
        ptr = nullptr;
        cap = 0;
    }
    size_t want = bytes + bytes / 4;  // headroom so a slowly growing m does not reallocate
    want = (want + 255) & ~(size_t)255;
    NNE_CUDA_TRY(cudaMalloc(&ptr, want));
    cap = want;
    return NNE_OK;
}

void GrowBuf::release() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    cap = 0;
}

namespace {

bool mul_overflows(size_t a, size_t b, size_t *out) { return __builtin_mul_overflow(a, b, out); }

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int check_layer(const nne_qlinear *ql) {
    if (!ql || !ql->ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null layer handle");
    return NNE_OK;
}

int alloc_layer(nne_ctx *ctx, size_t n, size_t k, bool has_bias, nne_qlinear **out) {
    size_t nk;
    if (mul_overflows(n, k, &nk)) return fail(NNE_ERR_INVALID_ARGUMENT, "n*k overflows size_t");
    nne_qlinear *ql = new (std::nothrow) nne_qlinear();
    if (!ql) return fail(NNE_ERR_OUT_OF_MEMORY, "host allocation failed");
    ql->ctx = ctx;
    ql->device = ctx->device;
    ql->n = n;
    ql->k = k;
    cudaError_t e = cudaMalloc(&ql->q, nk ? nk : 1);
    if (e == cudaSuccess) e = cudaMalloc(&ql->scales, (n ? n : 1) * sizeof(float));
    if (e == cudaSuccess && has_bias) e = cudaMalloc(&ql->bias, (n ? n : 1) * sizeof(float));
    if (e != cudaSuccess) {
        int st = fail(e == cudaErrorMemoryAllocation ? NNE_ERR_OUT_OF_MEMORY : NNE_ERR_CUDA,
                      "device allocation for a %zu x %zu layer failed: %s", n, k,
                      cudaGetErrorString(e));
        cudaGetLastError();
        nne_qlinear_destroy(ql);
        return st;
    }
    *out = ql;
    return NNE_OK;
}

// NNE_PREFILL=bf16 selects the bf16 tensor-core kernel (int8 codes dequantized in shared memory)
// instead of the integer one.
bool prefill_bf16_forced() {
    static const bool v = [] {
        const char *e = getenv("NNE_PREFILL");
        return e && e[0] == 'b';
    }();
    return v;
}

// NNE_SKINNY=0 sends 3..16-row forwards through the streaming GEMV in passes of two rows.
bool skinny_disabled() {
    static const bool v = []() {
        const char *e = getenv("NNE_SKINNY");
        return e && e[0] == '0';
    }();
    return v;
}

// Kernel choice for a forward of m rows.  1 = streaming GEMV, 2 = tensor-core, 3 = generic,
// 4 = small-batch tensor-core.
int pick_kernel(const nne_qlinear *ql, size_t m, const float *x, const float *y) {
    const bool base_ok = aligned(ql->q, 16) && (x == nullptr || aligned(x, 16)) &&
                         (y == nullptr || aligned(y, 4));
    if (base_ok && skinny_supports(ql, m) && !skinny_disabled()) return 4;
    // The bf16 tensor-core kernel rounds x to bf16 (worst case above the path's tolerance), so it
    // runs only when asked for; a shape the integer kernel declines goes to the fp32 kernels.
    if (m > 16 && base_ok &&
        (prefill_bf16_forced() ? prefill_supports(ql, m) : prefill_i8_supports(ql, m)))
        return 2;
    if (base_ok && gemv_supports(ql->n, ql->k, m)) return 1;
    return 3;
}

// Copy kernels pay off for latency-bound transfers (decode-sized activations); bulk transfers stay
// with the copy engines, which move a megabyte in less time than 64 CTAs pull it over PCIe.
constexpr size_t HOST_COPY_KERNEL_MAX_BYTES = (size_t)1 << 20;

// The device alias of [p, p + bytes) if that is pinned host memory (first and last byte asked), else
// null.  NNE_HOST_COPY=engine makes it null always.
void *pinned_alias(const void *p, size_t bytes) {
    static const bool engine_only = [] {
        const char *e = getenv("NNE_HOST_COPY");
        return e && e[0] == 'e';
    }();
    if (engine_only || !p || bytes == 0) return nullptr;
    cudaPointerAttributes a0, a1;
    if (cudaPointerGetAttributes(&a0, p) != cudaSuccess ||
        cudaPointerGetAttributes(&a1, static_cast<const char *>(p) + bytes - 1) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (a0.type != cudaMemoryTypeHost || a1.type != cudaMemoryTypeHost || !a0.devicePointer) return nullptr;
    return a0.devicePointer;
}

// Does a forward of m rows on this layer take a kernel that can store into the peers' windows itself?
bool forward_stores_to_peers(const nne_qlinear *ql, size_t m, const float *x, const float *y) {
    return ql->k != 0 && pick_kernel(ql, m, x, y) == 2 && !prefill_bf16_forced();
}

int forward_dev(nne_qlinear *ql, const float *x, size_t m, size_t k, float *y, size_t ldy,
                cudaStream_t s, const PeerSet *peers = nullptr) {
    NNE_TRY(check_layer(ql));
    if (k != ql->k)
        return fail(NNE_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%zu], got [%zu]", ql->k, k);
    if (ldy < ql->n) return fail(NNE_ERR_INVALID_ARGUMENT, "ldy %zu < out_features %zu", ldy, ql->n);
    size_t t;
    if (mul_overflows(m, ql->k, &t) || mul_overflows(m, ldy, &t))
        return fail(NNE_ERR_INVALID_ARGUMENT, "m*k or m*ldy overflows size_t");
    if (m == 0 || ql->n == 0) return NNE_OK;
    if (!x || !y) return fail(NNE_ERR_INVALID_ARGUMENT, "null activation or output pointer");
    NNE_TRY(use_ctx(ql->ctx));
    if (ql->k == 0) {
        // Empty contraction: dot = 0, y = 0*scale (+bias), as the reference's loops produce.
        return launch_generic(ql->ctx, ql->q, ql->scales, ql->bias, x, y, ql->n, 0, m, ldy, s);
    }
    switch (pick_kernel(ql, m, x, y)) {
        case 2:
            if (!prefill_bf16_forced()) return launch_prefill_i8(ql, x, y, m, ldy, s, peers);
            return launch_prefill(ql, x, y, m, ldy, s);
        case 4:
            return launch_skinny(ql, x, y, m, ldy, s);
        case 1:
            return launch_gemv(ql->ctx, ql->q, ql->scales, ql->bias, x, y, ql->n, ql->k, m, ldy, s);
        default:
            return launch_generic(ql->ctx, ql->q, ql->scales, ql->bias, x, y, ql->n, ql->k, m, ldy,
                                  s);
    }
}

}  // namespace
}  // namespace nne

using namespace nne;

extern "C" {

const char *nne_status_string(int status) {
    switch (status) {
        case NNE_OK: return "ok";
        case NNE_ERR_INVALID_ARGUMENT: return "invalid argument";
        case NNE_ERR_SHAPE_MISMATCH: return "shape mismatch";
        case NNE_ERR_CUDA: return "CUDA error";
        case NNE_ERR_NCCL: return "NCCL error";
        case NNE_ERR_TIMEOUT: return "timeout";
        case NNE_ERR_OUT_OF_MEMORY: return "out of memory";
        case NNE_ERR_UNSUPPORTED: return "unsupported";
        default: return "unknown status";
    }
}

int nne_last_error(char *buf, size_t n) {
    if (!buf || n == 0) return NNE_ERR_INVALID_ARGUMENT;
    const std::string &s = last_error_ref();
    size_t c = s.size() < n - 1 ? s.size() : n - 1;
    memcpy(buf, s.data(), c);
    buf[c] = 0;
    return NNE_OK;
}

uint64_t nne_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int nne_cuda_ctx_create(int device, nne_ctx **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(NNE_ERR_CUDA, "no usable CUDA device: %s", cudaGetErrorString(e));
    }
    if (device < 0 || device >= count)
        return fail(NNE_ERR_INVALID_ARGUMENT, "device %d out of range (have %d)", device, count);
    NNE_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    NNE_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(NNE_ERR_UNSUPPORTED,
                    "device %d is sm_%d%d; this library holds sm_100a code only and has no fallback",
                    device, prop.major, prop.minor);
    nne_ctx *ctx = new nne_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->total_mem = prop.totalGlobalMem;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->absmax_word, 256);
    if (e == cudaSuccess) e = cudaMemset(ctx->absmax_word, 0, 256);
    if (e == cudaSuccess) {
        void *hp = nullptr;
        e = cudaHostAlloc(&hp, 64, cudaHostAllocMapped);
        if (e == cudaSuccess) {
            ctx->err_host = static_cast<volatile int *>(hp);
            *ctx->err_host = 0;
            void *dp = nullptr;
            e = cudaHostGetDevicePointer(&dp, hp, 0);
            ctx->err_word = static_cast<int *>(dp);
        }
    }
    if (e == cudaSuccess) {
        // Keep freed stream-ordered workspaces cached in the pool instead of returning them to
        // the driver at every synchronisation.
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
            uint64_t keep = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        }
        cudaGetLastError();
    }
    if (e != cudaSuccess) {
        int st = fail(NNE_ERR_CUDA, "context set-up failed: %s", cudaGetErrorString(e));
        nne_cuda_ctx_destroy(ctx);
        return st;
    }
    *out = ctx;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_cuda_ctx_destroy(nne_ctx *ctx) {
    NNE_GUARD_BEGIN
    if (!ctx) return NNE_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    ctx->stage_a.release();
    ctx->stage_b.release();
    ctx->stage_c.release();
    if (ctx->absmax_word) cudaFree(ctx->absmax_word);
    if (ctx->err_host) cudaFreeHost(const_cast<int *>(ctx->err_host));
    delete ctx;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_cuda_ctx_check(nne_ctx *ctx) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    NNE_CUDA_TRY(cudaDeviceSynchronize());
    const int word = *ctx->err_host;
    if (word != 0) {
        *ctx->err_host = 0;
        return fail(NNE_ERR_TIMEOUT, "a kernel's bounded wait ran out (code 0x%x)", word);
    }
    return NNE_OK;
    NNE_GUARD_END
}

int nne_cuda_ctx_reserve_sms(nne_ctx *ctx, int count) {
    NNE_GUARD_BEGIN
    if (!ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null context");
    if (count < 0 || count >= ctx->sm_count)
        return fail(NNE_ERR_INVALID_ARGUMENT, "reserved SM count %d outside [0, %d)", count, ctx->sm_count);
    ctx->reserved_sms = count;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_cuda_ctx_info(const nne_ctx *ctx, int *device, int *sm_count, int *cc_major, int *cc_minor,
                      size_t *total_mem_bytes) {
    if (!ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null context");
    if (device) *device = ctx->device;
    if (sm_count) *sm_count = ctx->sm_count;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    if (total_mem_bytes) *total_mem_bytes = ctx->total_mem;
    return NNE_OK;
}

// ---- device buffers for a host-side tensor type ------------------------------------------------

int nne_device_alloc(nne_ctx *ctx, size_t bytes, void **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    NNE_CUDA_TRY(cudaMalloc(out, bytes ? bytes : 1));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_device_free(nne_ctx *ctx, void *ptr) {
    NNE_GUARD_BEGIN
    if (!ptr) return NNE_OK;
    NNE_TRY(use_ctx(ctx));
    NNE_CUDA_TRY(cudaFree(ptr));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_device_upload(nne_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (bytes == 0) return NNE_OK;
    if (!dst_dev || !src_host) return fail(NNE_ERR_INVALID_ARGUMENT, "null pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    NNE_CUDA_TRY(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    NNE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_device_download(nne_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (bytes == 0) return NNE_OK;
    if (!dst_host || !src_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    // everything issued on the device so far (any stream) is complete before the copy reads
    NNE_CUDA_TRY(cudaDeviceSynchronize());
    NNE_CUDA_TRY(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    NNE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    const int word = *ctx->err_host;
    if (word != 0) {
        *ctx->err_host = 0;
        return fail(NNE_ERR_TIMEOUT, "a kernel's bounded wait ran out (code 0x%x)", word);
    }
    return NNE_OK;
    NNE_GUARD_END
}

void *nne_cuda_ctx_stream(nne_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

// ---- quantize ---------------------------------------------------------------------------------

int nne_quantize_rows_dev(nne_ctx *ctx, const float *w_dev, size_t rows, size_t cols, int8_t *q_dev,
                          float *scales_dev, void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t t;
    if (mul_overflows(rows, cols, &t) || mul_overflows(t, sizeof(float), &t))
        return fail(NNE_ERR_INVALID_ARGUMENT, "rows*cols overflows size_t");
    if (rows == 0) return NNE_OK;
    if (!scales_dev || (cols && (!w_dev || !q_dev)))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_quantize_rows(ctx, w_dev, rows, cols, q_dev, scales_dev, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_quantize_rows(nne_ctx *ctx, const float *w_host, size_t rows, size_t cols, int8_t *q_host,
                      float *scales_host) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t nk, bytes;
    if (mul_overflows(rows, cols, &nk) || mul_overflows(nk, sizeof(float), &bytes))
        return fail(NNE_ERR_INVALID_ARGUMENT, "rows*cols overflows size_t");
    if (rows == 0) return NNE_OK;
    if (!scales_host || (nk && (!w_host || !q_host)))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null host pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    NNE_TRY(ctx->stage_a.reserve(bytes ? bytes : 4));
    NNE_TRY(ctx->stage_b.reserve(nk ? nk : 4));
    NNE_TRY(ctx->stage_c.reserve(rows * sizeof(float)));
    cudaStream_t s = ctx->stream;
    if (bytes) NNE_CUDA_TRY(cudaMemcpyAsync(ctx->stage_a.ptr, w_host, bytes, cudaMemcpyHostToDevice, s));
    NNE_TRY(launch_quantize_rows(ctx, (const float *)ctx->stage_a.ptr, rows, cols,
                                 (int8_t *)ctx->stage_b.ptr, (float *)ctx->stage_c.ptr, s));
    if (nk) NNE_CUDA_TRY(cudaMemcpyAsync(q_host, ctx->stage_b.ptr, nk, cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaMemcpyAsync(scales_host, ctx->stage_c.ptr, rows * sizeof(float),
                                 cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_quantize_tensor_dev(nne_ctx *ctx, const float *v_dev, size_t n, int8_t *q_dev,
                            float *scale_dev, void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (!scale_dev || (n && (!v_dev || !q_dev)))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_quantize_tensor(ctx, v_dev, n, q_dev, scale_dev, ctx->absmax_word,
                                  (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_quantize_tensor(nne_ctx *ctx, const float *v_host, size_t n, int8_t *q_host,
                        float *scale_out) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t bytes;
    if (mul_overflows(n, sizeof(float), &bytes))
        return fail(NNE_ERR_INVALID_ARGUMENT, "n overflows size_t");
    if (!scale_out || (n && (!v_host || !q_host)))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null host pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    NNE_TRY(ctx->stage_a.reserve(bytes ? bytes : 4));
    NNE_TRY(ctx->stage_b.reserve(n ? n : 4));
    NNE_TRY(ctx->stage_c.reserve(sizeof(float)));
    cudaStream_t s = ctx->stream;
    if (n) NNE_CUDA_TRY(cudaMemcpyAsync(ctx->stage_a.ptr, v_host, bytes, cudaMemcpyHostToDevice, s));
    NNE_TRY(launch_quantize_tensor(ctx, (const float *)ctx->stage_a.ptr, n,
                                   (int8_t *)ctx->stage_b.ptr, (float *)ctx->stage_c.ptr,
                                   ctx->absmax_word, s));
    if (n) NNE_CUDA_TRY(cudaMemcpyAsync(q_host, ctx->stage_b.ptr, n, cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaMemcpyAsync(scale_out, ctx->stage_c.ptr, sizeof(float), cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_dequantize_rows_dev(nne_ctx *ctx, const int8_t *q_dev, const float *scales_dev, size_t rows,
                            size_t cols, float *out_dev, void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t t;
    if (mul_overflows(rows, cols, &t) || mul_overflows(t, sizeof(float), &t))
        return fail(NNE_ERR_INVALID_ARGUMENT, "rows*cols overflows size_t");
    if (rows == 0 || cols == 0) return NNE_OK;
    if (!q_dev || !scales_dev || !out_dev)
        return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_dequantize_rows(ctx, q_dev, scales_dev, rows, cols, out_dev, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_dequantize_rows(nne_ctx *ctx, const int8_t *q_host, const float *scales_host, size_t rows,
                        size_t cols, float *out_host) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t nk, bytes;
    if (mul_overflows(rows, cols, &nk) || mul_overflows(nk, sizeof(float), &bytes))
        return fail(NNE_ERR_INVALID_ARGUMENT, "rows*cols overflows size_t");
    if (nk == 0) return NNE_OK;
    if (!q_host || !scales_host || !out_host)
        return fail(NNE_ERR_INVALID_ARGUMENT, "null host pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    NNE_TRY(ctx->stage_a.reserve(bytes));
    NNE_TRY(ctx->stage_b.reserve(nk));
    NNE_TRY(ctx->stage_c.reserve(rows * sizeof(float)));
    cudaStream_t s = ctx->stream;
    NNE_CUDA_TRY(cudaMemcpyAsync(ctx->stage_b.ptr, q_host, nk, cudaMemcpyHostToDevice, s));
    NNE_CUDA_TRY(cudaMemcpyAsync(ctx->stage_c.ptr, scales_host, rows * sizeof(float),
                                 cudaMemcpyHostToDevice, s));
    NNE_TRY(launch_dequantize_rows(ctx, (const int8_t *)ctx->stage_b.ptr,
                                   (const float *)ctx->stage_c.ptr, rows, cols,
                                   (float *)ctx->stage_a.ptr, s));
    NNE_CUDA_TRY(cudaMemcpyAsync(out_host, ctx->stage_a.ptr, bytes, cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    return NNE_OK;
    NNE_GUARD_END
}

// ---- layer ------------------------------------------------------------------------------------

int nne_qlinear_create_from_f32_dev(nne_ctx *ctx, const float *w_dev, const float *bias_dev_or_null,
                                    size_t n, size_t k, void *stream, nne_qlinear **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    if (n && k && !w_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null weight pointer");
    nne_qlinear *ql = nullptr;
    NNE_TRY(alloc_layer(ctx, n, k, bias_dev_or_null != nullptr, &ql));
    cudaStream_t s = (cudaStream_t)stream;
    int st = launch_quantize_rows(ctx, w_dev, n, k, ql->q, ql->scales, s);
    if (st == NNE_OK && bias_dev_or_null && n) {
        cudaError_t e = cudaMemcpyAsync(ql->bias, bias_dev_or_null, n * sizeof(float),
                                        cudaMemcpyDeviceToDevice, s);
        if (e != cudaSuccess) st = fail(NNE_ERR_CUDA, "bias copy failed: %s", cudaGetErrorString(e));
    }
    // The layer is handed out only once its codes are complete: forwards may read the weights
    // ahead of the stream's earlier work (programmatic dependent launch).
    if (st == NNE_OK) {
        cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) st = fail(NNE_ERR_CUDA, "quantize failed: %s", cudaGetErrorString(e));
    }
    if (st == NNE_OK) st = prefill_prepare_layer(ql);
    if (st == NNE_OK) st = prefill_i8_prepare_layer(ql);
    if (st == NNE_OK) st = skinny_prepare_layer(ql);
    if (st != NNE_OK) {
        nne_qlinear_destroy(ql);
        return st;
    }
    *out = ql;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_create_from_f32(nne_ctx *ctx, const float *w_host, const float *bias_host_or_null,
                                size_t n, size_t k, nne_qlinear **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    size_t nk, bytes;
    if (mul_overflows(n, k, &nk) || mul_overflows(nk, sizeof(float), &bytes))
        return fail(NNE_ERR_INVALID_ARGUMENT, "n*k overflows size_t");
    if (nk && !w_host) return fail(NNE_ERR_INVALID_ARGUMENT, "null weight pointer");
    nne_qlinear *ql = nullptr;
    NNE_TRY(alloc_layer(ctx, n, k, bias_host_or_null != nullptr, &ql));
    int st = NNE_OK;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        cudaStream_t s = ctx->stream;
        st = ctx->stage_a.reserve(bytes ? bytes : 4);
        cudaError_t e = cudaSuccess;
        if (st == NNE_OK && bytes)
            e = cudaMemcpyAsync(ctx->stage_a.ptr, w_host, bytes, cudaMemcpyHostToDevice, s);
        if (st == NNE_OK && e == cudaSuccess)
            st = launch_quantize_rows(ctx, (const float *)ctx->stage_a.ptr, n, k, ql->q, ql->scales, s);
        if (st == NNE_OK && e == cudaSuccess && bias_host_or_null && n)
            e = cudaMemcpyAsync(ql->bias, bias_host_or_null, n * sizeof(float),
                                cudaMemcpyHostToDevice, s);
        if (st == NNE_OK && e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (st == NNE_OK && e != cudaSuccess)
            st = fail(NNE_ERR_CUDA, "layer upload failed: %s", cudaGetErrorString(e));
    }
    if (st == NNE_OK) st = prefill_prepare_layer(ql);
    if (st == NNE_OK) st = prefill_i8_prepare_layer(ql);
    if (st == NNE_OK) st = skinny_prepare_layer(ql);
    if (st != NNE_OK) {
        nne_qlinear_destroy(ql);
        return st;
    }
    *out = ql;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_create_from_i8(nne_ctx *ctx, const int8_t *q_host, const float *scales_host,
                               const float *bias_host_or_null, size_t n, size_t k,
                               nne_qlinear **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    size_t nk;
    if (mul_overflows(n, k, &nk)) return fail(NNE_ERR_INVALID_ARGUMENT, "n*k overflows size_t");
    if ((nk && !q_host) || (n && !scales_host))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null codes or scales pointer");
    nne_qlinear *ql = nullptr;
    NNE_TRY(alloc_layer(ctx, n, k, bias_host_or_null != nullptr, &ql));
    cudaError_t e = cudaSuccess;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        cudaStream_t s = ctx->stream;
        if (nk) e = cudaMemcpyAsync(ql->q, q_host, nk, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess && n)
            e = cudaMemcpyAsync(ql->scales, scales_host, n * sizeof(float), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess && n && bias_host_or_null)
            e = cudaMemcpyAsync(ql->bias, bias_host_or_null, n * sizeof(float),
                                cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    }
    int st = NNE_OK;
    if (e != cudaSuccess) st = fail(NNE_ERR_CUDA, "layer upload failed: %s", cudaGetErrorString(e));
    if (st == NNE_OK) st = prefill_prepare_layer(ql);
    if (st == NNE_OK) st = prefill_i8_prepare_layer(ql);
    if (st == NNE_OK) st = skinny_prepare_layer(ql);
    if (st != NNE_OK) {
        nne_qlinear_destroy(ql);
        return st;
    }
    *out = ql;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_destroy(nne_qlinear *ql) {
    NNE_GUARD_BEGIN
    if (!ql) return NNE_OK;
    cudaSetDevice(ql->device);
    prefill_release_layer(ql);
    prefill_i8_release_layer(ql);
    skinny_release_layer(ql);
    if (ql->own) {
        if (ql->q) cudaFree(ql->q);
        if (ql->scales) cudaFree(ql->scales);
        if (ql->bias) cudaFree(ql->bias);
    }
    delete ql;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_download(const nne_qlinear *ql, int8_t *q_host, float *scales_host) {
    NNE_GUARD_BEGIN
    NNE_TRY(check_layer(ql));
    NNE_TRY(use_ctx(ql->ctx));
    std::lock_guard<std::mutex> lock(ql->ctx->mu);
    cudaStream_t s = ql->ctx->stream;
    if (q_host && ql->n && ql->k)
        NNE_CUDA_TRY(cudaMemcpyAsync(q_host, ql->q, ql->n * ql->k, cudaMemcpyDeviceToHost, s));
    if (scales_host && ql->n)
        NNE_CUDA_TRY(cudaMemcpyAsync(scales_host, ql->scales, ql->n * sizeof(float),
                                     cudaMemcpyDeviceToHost, s));
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_info(const nne_qlinear *ql, size_t *n, size_t *k, int *has_bias,
                     const int8_t **q_dev, const float **scales_dev, const float **bias_dev) {
    NNE_TRY(check_layer(ql));
    if (n) *n = ql->n;
    if (k) *k = ql->k;
    if (has_bias) *has_bias = ql->bias != nullptr;
    if (q_dev) *q_dev = ql->q;
    if (scales_dev) *scales_dev = ql->scales;
    if (bias_dev) *bias_dev = ql->bias;
    return NNE_OK;
}

size_t nne_qlinear_memory_bytes(const nne_qlinear *ql) {
    if (!ql) return 0;
    return ql->n * ql->k + ql->n * sizeof(float) + (ql->bias ? ql->n * sizeof(float) : 0);
}

int nne_qlinear_kernel_for(const nne_qlinear *ql, size_t m) {
    if (!ql || !ql->ctx) return 0;
    return pick_kernel(ql, m, nullptr, nullptr);
}

int nne_qlinear_forward_dev(nne_qlinear *ql, const float *x_dev, size_t m, size_t k, float *y_dev,
                            void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(check_layer(ql));
    return forward_dev(ql, x_dev, m, k, y_dev, ql->n, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_qlinear_forward_dev_strided(nne_qlinear *ql, const float *x_dev, size_t m, size_t k,
                                    float *y_dev, size_t ldy, void *stream) {
    NNE_GUARD_BEGIN
    return forward_dev(ql, x_dev, m, k, y_dev, ldy, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_qlinear_forward_host(nne_qlinear *ql, const float *x_host, size_t m, size_t k,
                             float *y_host) {
    NNE_GUARD_BEGIN
    NNE_TRY(check_layer(ql));
    if (k != ql->k)
        return fail(NNE_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%zu], got [%zu]", ql->k, k);
    size_t xb, yb;
    if (mul_overflows(m, ql->k, &xb) || mul_overflows(xb, sizeof(float), &xb) ||
        mul_overflows(m, ql->n, &yb) || mul_overflows(yb, sizeof(float), &yb))
        return fail(NNE_ERR_INVALID_ARGUMENT, "m*k or m*n overflows size_t");
    if (m == 0 || ql->n == 0) return NNE_OK;
    if ((xb && !x_host) || !y_host) return fail(NNE_ERR_INVALID_ARGUMENT, "null host pointer");
    nne_ctx *ctx = ql->ctx;
    NNE_TRY(use_ctx(ctx));
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaStream_t s = ctx->stream;
    NNE_TRY(ctx->stage_a.reserve(xb ? xb : 4));
    NNE_TRY(ctx->stage_b.reserve(yb));
    // Pinned x and y (16-byte aligned, whole float4s): copy kernels chained to the forward by
    // programmatic dependent launch instead of copy-engine transfers (see nne_qlinear_plan_run_host).
    const float *x_alias = nullptr;
    float *y_alias = nullptr;
    if (xb && xb + yb <= HOST_COPY_KERNEL_MAX_BYTES && xb % 16 == 0 && yb % 16 == 0 && aligned(x_host, 16) &&
        aligned(y_host, 16)) {
        x_alias = static_cast<const float *>(pinned_alias(x_host, xb));
        y_alias = x_alias ? static_cast<float *>(pinned_alias(y_host, yb)) : nullptr;
    }
    if (x_alias && y_alias) {
        HostCopySegs in = {}, out = {};
        in.count = out.count = 1;
        in.seg[0].src = x_alias;
        in.seg[0].dst = (float *)ctx->stage_a.ptr;
        in.seg[0].n4 = xb / 16;
        out.seg[0].src = (const float *)ctx->stage_b.ptr;
        out.seg[0].dst = y_alias;
        out.seg[0].n4 = yb / 16;
        NNE_TRY(launch_host_copy(ctx, in, false, s));
        NNE_TRY(forward_dev(ql, (const float *)ctx->stage_a.ptr, m, k, (float *)ctx->stage_b.ptr, ql->n, s));
        NNE_TRY(launch_host_copy(ctx, out, true, s));
    } else {
        if (xb) NNE_CUDA_TRY(cudaMemcpyAsync(ctx->stage_a.ptr, x_host, xb, cudaMemcpyHostToDevice, s));
        NNE_TRY(forward_dev(ql, (const float *)ctx->stage_a.ptr, m, k, (float *)ctx->stage_b.ptr, ql->n, s));
        NNE_CUDA_TRY(cudaMemcpyAsync(y_host, ctx->stage_b.ptr, yb, cudaMemcpyDeviceToHost, s));
    }
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    const int word = *ctx->err_host;
    if (word != 0) {
        *ctx->err_host = 0;
        return fail(NNE_ERR_TIMEOUT, "a kernel's bounded wait ran out (code 0x%x)", word);
    }
    return NNE_OK;
    NNE_GUARD_END
}

}  // extern "C"

// ---- plan ---------------------------------------------------------------------------------------

namespace nne {
namespace {

// Which items of a list have to wait for the items before them: sync[i] = 1 when item i reads
// something an earlier item (since the last such point) writes, or writes something an earlier one
// reads or writes.  Byte intervals; a strided output counts from its first to its last element.
// An item whose own output overlaps its own input is refused (every CTA reads all of x while others
// already store y), except a residual that IS the output (read and written by the same thread).
struct ByteRange {
    uintptr_t lo, hi;
    bool meets(const ByteRange &o) const { return lo < o.hi && o.lo < hi; }
};
ByteRange range_of(const void *p, size_t floats) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    return {a, p ? a + floats * sizeof(float) : a};
}
int plan_hazards(size_t count, nne_qlinear *const *layers, const float *const *x, float *const *y, size_t m,
                 const nne_plan_item *items, std::vector<char> &sync) {
    sync.assign(count, 0);
    std::vector<ByteRange> reads, writes;
    for (size_t i = 0; i < count; ++i) {
        NNE_TRY(check_layer(layers[i]));
        const size_t n = layers[i]->n, k = layers[i]->k;
        if (m == 0 || n == 0) continue;
        const ByteRange w = range_of(y[i], m * n);
        ByteRange r[4] = {range_of(x[i], m * k), {0, 0}, {0, 0}, {0, 0}};
        if (items) {
            if (items[i].input_op == NNE_INPUT_RMSNORM) r[1] = range_of(items[i].gamma, k);
            if (items[i].input_op == NNE_INPUT_SILU_MUL) r[1] = range_of(items[i].x2, m * k);
            if (items[i].residual && items[i].residual != y[i]) r[2] = range_of(items[i].residual, m * n);
        }
        for (const ByteRange &q : r)
            if (q.meets(w))
                return fail(NNE_ERR_INVALID_ARGUMENT, "item %zu: its output overlaps one of its inputs", i);
        bool wait = false;
        for (const ByteRange &q : writes) {
            wait = wait || q.meets(w);
            for (const ByteRange &mine : r) wait = wait || q.meets(mine);
        }
        for (const ByteRange &q : reads) wait = wait || q.meets(w);
        if (wait) {
            sync[i] = 1;
            reads.clear();
            writes.clear();
        }
        writes.push_back(w);
        for (const ByteRange &mine : r)
            if (mine.hi > mine.lo) reads.push_back(mine);
        if (items && items[i].residual == y[i]) reads.push_back(w);
    }
    return NNE_OK;
}

// Fills the plan's layer lists and decides how it runs (one streaming launch, one small-batch
// launch, or layer by layer).  y[i] / ldy[i] are where this plan's kernels write.  `sync` (or null)
// marks the items that wait for the ones before them (plan_hazards): a streaming launch lets its
// grid meet there; any other list is cut into sub-plans that run one after another.
int plan_build(nne_plan *plan, nne_ctx *ctx, size_t count, nne_qlinear *const *layers,
               const float *const *x_dev_in, float *const *y_dev, const size_t *ldy_or_null, size_t m,
               const nne_plan_item *items = nullptr, const char *sync = nullptr) {
    plan->ctx = ctx;
    plan->m = m;
    bool any_sync = false;
    for (size_t i = 0; sync && i < count; ++i) any_sync = any_sync || sync[i];
    bool fused = (m >= 1 && m <= 2);
    // Can the whole list run as one streaming launch?  Then that kernel applies the items' input
    // transforms and residuals itself.  Otherwise they become standalone launches around the
    // forwards, and the forwards read the transformed activations from a buffer of the plan.
    for (size_t i = 0; i < count && fused; ++i) {
        nne_qlinear *ql = layers[i];
        NNE_TRY(check_layer(ql));
        fused = aligned(ql->q, 16) && aligned(x_dev_in[i], 16) && aligned(y_dev[i], 4) &&
                gemv_tma_supports(ql->n, ql->k, m) &&
                !(m >= 2 && !skinny_disabled() && ql->tmap_wsk) &&
                // the decode kernel reads gamma and x2 sixteen bytes at a time
                (!items || (aligned(items[i].gamma, 16) && aligned(items[i].x2, 16)));
    }
    if (any_sync && !fused) {
        for (size_t i = 0; i < count; ++i) {
            plan->layers.push_back(layers[i]);
            plan->x.push_back(x_dev_in[i]);
            plan->y.push_back(y_dev[i]);
            plan->ldy.push_back(ldy_or_null ? ldy_or_null[i] : layers[i]->n);
        }
        size_t b = 0;
        for (size_t i = 1; i <= count; ++i) {
            if (i < count && !sync[i]) continue;
            nne_plan *sub = new nne_plan();
            plan->phases.push_back(sub);
            NNE_TRY(plan_build(sub, ctx, i - b, layers + b, x_dev_in + b, y_dev + b,
                               ldy_or_null ? ldy_or_null + b : nullptr, m, items ? items + b : nullptr));
            b = i;
        }
        return NNE_OK;
    }
    std::vector<const float *> x_eff(x_dev_in, x_dev_in + count);
    if (items && !fused) {
        size_t floats = 0;
        for (size_t i = 0; i < count; ++i) {
            if (items[i].input_op == NNE_INPUT_PLAIN) continue;
            bool seen = false;
            for (size_t j = 0; j < i && !seen; ++j)
                seen = items[j].input_op == items[i].input_op && items[j].x == items[i].x &&
                       items[j].gamma == items[i].gamma && items[j].x2 == items[i].x2 &&
                       items[j].eps == items[i].eps && layers[j]->k == layers[i]->k;
            if (!seen) floats += ((m * layers[i]->k + 63) / 64) * 64;
        }
        if (floats) NNE_CUDA_TRY(cudaMalloc(&plan->xform_buf, floats * sizeof(float)));
        size_t off = 0;
        for (size_t i = 0; i < count; ++i) {
            if (items[i].input_op == NNE_INPUT_PLAIN) continue;
            const float *aux = items[i].input_op == NNE_INPUT_RMSNORM ? items[i].gamma : items[i].x2;
            float *dst = nullptr;
            for (const nne_plan::PreOp &op : plan->pre_ops)
                if (op.kind == items[i].input_op && op.x == items[i].x && op.aux == aux &&
                    op.eps == items[i].eps && op.cols == layers[i]->k)
                    dst = op.dst;
            if (!dst) {
                dst = plan->xform_buf + off;
                off += ((m * layers[i]->k + 63) / 64) * 64;
                plan->pre_ops.push_back({items[i].input_op, items[i].x, aux, items[i].eps, dst, m, layers[i]->k});
            }
            x_eff[i] = dst;
        }
        for (size_t i = 0; i < count; ++i) {
            if (!items[i].residual) continue;
            const size_t ldy = ldy_or_null ? ldy_or_null[i] : layers[i]->n;
            if (m > 1 && ldy != layers[i]->n)
                return fail(NNE_ERR_UNSUPPORTED, "layer %zu: a residual on strided rows needs the streaming kernel", i);
            plan->post_ops.push_back({y_dev[i], items[i].residual, m * layers[i]->n});
        }
    }
    const float *const *x_dev = x_eff.data();
    fused = (m >= 1 && m <= 2);
    for (size_t i = 0; i < count; ++i) {
        nne_qlinear *ql = layers[i];
        NNE_TRY(check_layer(ql));
        if (ql->ctx != ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "layer %zu lives on another context", i);
        if (m && ql->n && (!x_dev[i] || !y_dev[i]))
            return fail(NNE_ERR_INVALID_ARGUMENT, "null x or y pointer for layer %zu", i);
        const size_t ldy = ldy_or_null ? ldy_or_null[i] : ql->n;
        if (ldy < ql->n) return fail(NNE_ERR_INVALID_ARGUMENT, "row stride of layer %zu below its width", i);
        plan->layers.push_back(ql);
        plan->x.push_back(x_dev[i]);
        plan->y.push_back(y_dev[i]);
        plan->ldy.push_back(ldy);
        StreamLayer L;
        L.q = ql->q;
        L.scales = ql->scales;
        L.bias = ql->bias;
        L.x = x_dev[i];
        L.y = y_dev[i];
        L.ldy = ldy;
        L.n = (int)ql->n;
        L.k = (int)ql->k;
        L.rw = stream_rows_per_stage(ql->k);
        if (items && plan->pre_ops.empty() && plan->post_ops.empty()) {
            L.eps = items[i].eps;
            L.gamma = items[i].input_op == NNE_INPUT_RMSNORM ? items[i].gamma : nullptr;
            L.x2 = items[i].input_op == NNE_INPUT_SILU_MUL ? items[i].x2 : nullptr;
            L.residual = items[i].residual;
        }
        L.sync = (sync && sync[i]) ? 1 : 0;
        if (i > 0 && !L.sync && ldy_or_null == nullptr) {
            // (not for column shards: their launches do not take this flag)
            const StreamLayer &P = plan->descs.back();
            L.same_input = P.x == L.x && P.k == L.k && P.gamma == L.gamma && P.x2 == L.x2 &&
                           (L.gamma == nullptr || P.eps == L.eps);
        }
        plan->descs.push_back(L);
        fused = fused && aligned(ql->q, 16) && aligned(x_dev[i], 16) && aligned(y_dev[i], 4) &&
                gemv_tma_supports(ql->n, ql->k, m);
    }
    plan->fused = fused && count > 0;
    if (m >= 2 && !skinny_disabled() && skinny_plan_supports(layers, x_dev, y_dev, count, m)) {
        NNE_TRY(skinny_plan_create(ctx, layers, x_dev, y_dev, ldy_or_null, count, m, &plan->skinny));
        plan->fused = false;
    }
    if (any_sync && !plan->fused)
        return fail(NNE_ERR_UNSUPPORTED, "a list with dependent items did not come out as one streaming launch");
#ifdef NNE_TRACE
    if (plan->fused) {
        const size_t gsync_bytes = 16 * 1024;  // + the debug build's time stamps
#else
    if (any_sync) {
        const size_t gsync_bytes = sizeof(unsigned long long);
#endif
        NNE_CUDA_TRY(cudaMalloc(&plan->gsync_dev, gsync_bytes));
        NNE_CUDA_TRY(cudaMemset(plan->gsync_dev, 0, gsync_bytes));
    }
    if (plan->fused && count > (size_t)STREAM_INLINE_LAYERS) {
        NNE_CUDA_TRY(cudaMalloc(&plan->descs_dev, count * sizeof(StreamLayer)));
        NNE_CUDA_TRY(cudaMemcpy(plan->descs_dev, plan->descs.data(), count * sizeof(StreamLayer),
                                cudaMemcpyHostToDevice));
    }
    return NNE_OK;
}

void plan_free(nne_plan *plan) {
    if (!plan) return;
    if (plan->ctx) cudaSetDevice(plan->ctx->device);
    for (nne_plan *sub : plan->phases) plan_free(sub);
    if (plan->gsync_dev) cudaFree(plan->gsync_dev);
    if (plan->descs_dev) cudaFree(plan->descs_dev);
    if (plan->xform_buf) cudaFree(plan->xform_buf);
    if (plan->segs_dev) cudaFree(plan->segs_dev);
    if (plan->staging) cudaFree(plan->staging);
    skinny_plan_destroy(plan->skinny);
    delete plan;
}

// The plan's forward kernels on `s`, each layer writing y[i] at row stride ldy[i].
int plan_compute(nne_plan *plan, const PeerSet *peers, cudaStream_t s) {
    if (!plan->phases.empty()) {
        for (nne_plan *sub : plan->phases) NNE_TRY(plan_compute(sub, nullptr, s));
        return NNE_OK;
    }
    if (plan->fused)
        return launch_stream_batch(plan->ctx, plan->descs.data(), plan->descs_dev, (int)plan->descs.size(),
                                   plan->m, false, s, peers, plan->gsync_dev);
    for (const nne_plan::PreOp &op : plan->pre_ops) {
        if (op.kind == NNE_INPUT_RMSNORM)
            NNE_TRY(launch_rmsnorm(plan->ctx, op.x, op.aux, op.eps, op.rows, op.cols, op.dst, s));
        else
            NNE_TRY(launch_silu_mul(plan->ctx, op.x, op.aux, op.rows * op.cols, op.dst, s));
    }
    if (plan->skinny) {
        NNE_TRY(skinny_plan_run(plan->skinny, s));
    } else {
        for (size_t i = 0; i < plan->layers.size(); ++i)
            NNE_TRY(forward_dev(plan->layers[i], plan->x[i], plan->m, plan->layers[i]->k, plan->y[i],
                                plan->ldy[i], s,
                                (peers && !plan->stores_itself.empty() && plan->stores_itself[i]) ? peers : nullptr));
    }
    for (const nne_plan::PostOp &op : plan->post_ops)
        NNE_TRY(launch_add(plan->ctx, op.y, op.residual, op.count, op.y, s));
    return NNE_OK;
}

// One run of a plan: the forwards and, for column shards, the exchange of the output slices.
int plan_issue(nne_plan *plan, cudaStream_t s) {
    nne_shard_group *g = plan->group;
    if (!g || g->world == 1) return plan_compute(plan, nullptr, s);
    if (!g->connected) return fail(NNE_ERR_INVALID_ARGUMENT, "the shard group is not connected to its peers");
    if (plan->route == 0) {
        const unsigned long long epoch = g->epoch.fetch_add(1) + 1;
        if (plan->fused) {
            // the streaming kernel stores into every window itself
            const PeerSet ps = shard_peerset(g, epoch);
            return plan_compute(plan, &ps, s);
        }
        // tensor-core forwards store their tiles into every window themselves; what is left (small
        // batches, odd shapes) is copied out by the push kernel
        const PeerSet ps = shard_peerset(g, epoch);
        NNE_TRY(plan_compute(plan, &ps, s));
        if (plan->seg_count == 0) return NNE_OK;
        return shard_push(g, plan->segs_dev, plan->seg_count, plan->push_floats, epoch, s);
    }
    // NCCL route.  One row (or a world of one column block each): the slices already sit where an
    // in-place all-gather of y_full wants them.  More rows: gather [m, width] blocks into a staging
    // area and interleave them into row-major y_full.
    const size_t count = plan->layers.size();
    if (plan->m == 1) {
        NNE_TRY(plan_compute(plan, nullptr, s));
        NNE_TRY(shard_nccl_group_start());
        int st = NNE_OK;
        for (size_t i = 0; i < count && st == NNE_OK; ++i)
            st = shard_nccl_all_gather(g, plan->y[i], plan->y_full[i], plan->layers[i]->n, s);
        const int st2 = shard_nccl_group_end();
        return st != NNE_OK ? st : st2;
    }
    for (size_t i = 0; i < count; ++i) {
        nne_qlinear *ql = plan->layers[i];
        const size_t w = ql->n;
        float *mine = plan->staging + (size_t)g->rank * plan->m * w;
        NNE_TRY(forward_dev(ql, plan->x[i], plan->m, ql->k, mine, w, s));
        NNE_TRY(shard_nccl_all_gather(g, mine, plan->staging, plan->m * w, s));
        NNE_TRY(shard_interleave(plan->ctx, plan->staging, plan->y_full[i], g->world, plan->m, w,
                                 plan->n_total[i], s));
    }
    return NNE_OK;
}

}  // namespace
}  // namespace nne

extern "C" {

int nne_qlinear_plan_create(nne_ctx *ctx, size_t count, nne_qlinear *const *layers,
                            const float *const *x_dev, float *const *y_dev, size_t m,
                            nne_plan **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    if (count && (!layers || !x_dev || !y_dev))
        return fail(NNE_ERR_INVALID_ARGUMENT, "null layer / x / y array");
    if (count > 0x7fffffffu) return fail(NNE_ERR_INVALID_ARGUMENT, "too many layers");
    std::vector<char> sync;
    NNE_TRY(plan_hazards(count, layers, x_dev, y_dev, m, nullptr, sync));
    nne_plan *plan = new nne_plan();
    int st = plan_build(plan, ctx, count, layers, x_dev, y_dev, nullptr, m, nullptr, sync.data());
    if (st != NNE_OK) {
        cudaGetLastError();
        plan_free(plan);
        return st;
    }
    *out = plan;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_plan_create_fused(nne_ctx *ctx, size_t count, const nne_plan_item *items, size_t m,
                                  nne_plan **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    NNE_TRY(use_ctx(ctx));
    if (count == 0 || count > 0x7fffffffu || !items) return fail(NNE_ERR_INVALID_ARGUMENT, "empty or null item list");
    std::vector<nne_qlinear *> layers(count);
    std::vector<const float *> xs(count);
    std::vector<float *> ys(count);
    for (size_t i = 0; i < count; ++i) {
        const nne_plan_item &it = items[i];
        if (it.input_op != NNE_INPUT_PLAIN && it.input_op != NNE_INPUT_RMSNORM && it.input_op != NNE_INPUT_SILU_MUL)
            return fail(NNE_ERR_INVALID_ARGUMENT, "item %zu: unknown input_op %d", i, it.input_op);
        if (it.input_op == NNE_INPUT_RMSNORM && !it.gamma)
            return fail(NNE_ERR_INVALID_ARGUMENT, "item %zu: RMSNorm input needs gamma", i);
        if (it.input_op == NNE_INPUT_SILU_MUL && !it.x2)
            return fail(NNE_ERR_INVALID_ARGUMENT, "item %zu: silu(x) * x2 input needs x2", i);
        NNE_TRY(check_layer(it.layer));
        if (it.input_op == NNE_INPUT_RMSNORM && it.layer->k == 0)
            return fail(NNE_ERR_INVALID_ARGUMENT, "item %zu: RMSNorm over an empty dimension", i);
        layers[i] = it.layer;
        xs[i] = it.x;
        ys[i] = it.y;
    }
    std::vector<char> sync;
    NNE_TRY(plan_hazards(count, layers.data(), xs.data(), ys.data(), m, items, sync));
    nne_plan *plan = new nne_plan();
    int st = plan_build(plan, ctx, count, layers.data(), xs.data(), ys.data(), nullptr, m, items, sync.data());
    if (st != NNE_OK) {
        cudaGetLastError();
        plan_free(plan);
        return st;
    }
    *out = plan;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_plan_create_sharded(nne_shard_group *group, size_t count, nne_qlinear *const *shards,
                                    const size_t *row_begin, const size_t *n_total,
                                    const float *const *x_dev, float *const *y_full_dev, size_t m,
                                    int route, nne_plan **out) {
    NNE_GUARD_BEGIN
    if (!out) return fail(NNE_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    if (!group) return fail(NNE_ERR_INVALID_ARGUMENT, "null shard group");
    nne_ctx *ctx = group->ctx;
    NNE_TRY(use_ctx(ctx));
    if (count == 0 || count > 0x7fffffffu || !shards || !row_begin || !n_total || !x_dev || !y_full_dev)
        return fail(NNE_ERR_INVALID_ARGUMENT, "empty list or null array");
    if (route != 0 && route != 1) return fail(NNE_ERR_INVALID_ARGUMENT, "route must be 0 (peer stores) or 1 (NCCL)");
    if (m == 0) return fail(NNE_ERR_INVALID_ARGUMENT, "m must be at least 1");
    const uint8_t *wbeg = group->base, *wend = group->base + group->flag_off;
    std::vector<float *> y_slice(count);
    std::vector<size_t> ldy(count);
    size_t widest = 0;
    for (size_t i = 0; i < count; ++i) {
        NNE_TRY(check_layer(shards[i]));
        const size_t w = shards[i]->n;
        size_t t;
        if (row_begin[i] > n_total[i] || w > n_total[i] - row_begin[i])
            return fail(NNE_ERR_INVALID_ARGUMENT, "layer %zu: rows [%zu, +%zu) outside %zu output channels", i,
                        row_begin[i], w, n_total[i]);
        if (!y_full_dev[i] || mul_overflows(m, n_total[i], &t) || mul_overflows(t, sizeof(float), &t))
            return fail(NNE_ERR_INVALID_ARGUMENT, "layer %zu: null or oversized output", i);
        const uint8_t *yb = reinterpret_cast<const uint8_t *>(y_full_dev[i]);
        if (group->world > 1 && (yb < wbeg || yb + t > wend))
            return fail(NNE_ERR_INVALID_ARGUMENT,
                        "layer %zu: the output [m, n_total] must lie inside the group's window", i);
        if (route == 1 && group->world > 1 &&
            (w * (size_t)group->world != n_total[i] || row_begin[i] != w * (size_t)group->rank))
            return fail(NNE_ERR_UNSUPPORTED,
                        "layer %zu: the NCCL route needs equal slices in rank order (n_total %% world == 0)", i);
        y_slice[i] = y_full_dev[i] + row_begin[i];
        ldy[i] = n_total[i];
        widest = widest > w ? widest : w;
    }
    nne_plan *plan = new nne_plan();
    plan->group = group;
    plan->route = route;
    int st = plan_build(plan, ctx, count, shards, x_dev, y_slice.data(), ldy.data(), m);
    if (st == NNE_OK && group->world > 1) {
        plan->y_full.assign(y_full_dev, y_full_dev + count);
        plan->n_total.assign(n_total, n_total + count);
        plan->row_begin.assign(row_begin, row_begin + count);
        if (route == 0 && !plan->fused) {
            std::vector<PushSeg> segs;
            plan->stores_itself.assign(count, 0);
            // A tensor-core forward's epilogue stores every tile world-1 times more.  Up to about
            // 128 MB leaving the rank per forward that hides under the MMAs (2 ranks, 117 MB: +20 %;
            // 8 ranks, 59 MB: +60 %); with 205 MB to seven peers the epilogue warps became the
            // bottleneck (12 times the forward's own time, measured): such layers store locally and
            // the push kernel copies the slice out afterwards.  NNE_SHARD_EPILOGUE_MAX_MB overrides.
            static const size_t epilogue_max = [] {
                const char *e = getenv("NNE_SHARD_EPILOGUE_MAX_MB");
                return (size_t)(e ? atol(e) : 128) << 20;
            }();
            for (size_t i = 0; i < count; ++i) {
                const size_t leaving = m * shards[i]->n * sizeof(float) * (size_t)(group->world - 1);
                if (!plan->skinny && plan->pre_ops.empty() && plan->post_ops.empty() && leaving <= epilogue_max &&
                    forward_stores_to_peers(shards[i], m, plan->x[i], y_slice[i])) {
                    plan->stores_itself[i] = 1;
                    continue;
                }
                PushSeg sg;
                sg.y = y_slice[i];
                sg.ldy = ldy[i];
                sg.rows = (unsigned)m;
                sg.width = (unsigned)shards[i]->n;
                sg.vec = aligned(y_slice[i], 16) && ldy[i] % 4 == 0 && shards[i]->n % 4 == 0;
                segs.push_back(sg);
                plan->push_floats += m * shards[i]->n;
            }
            plan->seg_count = (int)segs.size();
            if (!segs.empty()) {
                cudaError_t e = cudaMalloc(&plan->segs_dev, segs.size() * sizeof(PushSeg));
                if (e == cudaSuccess)
                    e = cudaMemcpy(plan->segs_dev, segs.data(), segs.size() * sizeof(PushSeg), cudaMemcpyHostToDevice);
                if (e != cudaSuccess) st = fail(NNE_ERR_CUDA, "plan upload failed: %s", cudaGetErrorString(e));
            }
        }
        if (route == 1 && m > 1) {
            cudaError_t e = cudaMalloc(&plan->staging, (size_t)group->world * m * widest * sizeof(float));
            if (e != cudaSuccess)
                st = fail(e == cudaErrorMemoryAllocation ? NNE_ERR_OUT_OF_MEMORY : NNE_ERR_CUDA,
                          "staging allocation failed: %s", cudaGetErrorString(e));
        }
    } else if (st == NNE_OK) {
        plan->y_full.assign(y_full_dev, y_full_dev + count);
        plan->n_total.assign(n_total, n_total + count);
        plan->row_begin.assign(row_begin, row_begin + count);
    }
    if (st != NNE_OK) {
        cudaGetLastError();
        plan_free(plan);
        return st;
    }
    *out = plan;
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_plan_run(nne_plan *plan, void *stream) {
    NNE_GUARD_BEGIN
    if (!plan || !plan->ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null plan");
    if (plan->layers.empty() || plan->m == 0) return NNE_OK;
    NNE_TRY(use_ctx(plan->ctx));
    return plan_issue(plan, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_qlinear_plan_run_host(nne_plan *plan, const float *x_all_host, float *y_all_host) {
    NNE_GUARD_BEGIN
    if (!plan || !plan->ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null plan");
    if (plan->layers.empty() || plan->m == 0) return NNE_OK;
    if (!x_all_host || !y_all_host) return fail(NNE_ERR_INVALID_ARGUMENT, "null host pointer");
    nne_ctx *ctx = plan->ctx;
    NNE_TRY(use_ctx(ctx));
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaStream_t s = ctx->stream;
    const size_t count = plan->layers.size();
    // Neighbouring device buffers that continue one another are moved with one copy; an x
    // several layers share (same pointer, q/k/v) appears once in x_all_host per layer all the same.
    const bool sharded = plan->group != nullptr;
    struct Run {
        float *dev;
        size_t off, len;  // floats
    };
    std::vector<Run> xr, yr;
    size_t i = 0, off = 0;
    while (i < count) {
        size_t j = i, len = 0;
        const float *base = plan->x[i];
        while (j < count && plan->x[j] == base + len) len += plan->m * plan->layers[j++]->k;
        if (len) xr.push_back({const_cast<float *>(base), off, len});
        off += len;
        i = j;
    }
    // What comes back: y_i [m, n_i], or for column shards the gathered y_full_i [m, n_total_i].
    i = 0;
    off = 0;
    while (i < count) {
        size_t j = i, len = 0;
        float *base = sharded ? plan->y_full[i] : plan->y[i];
        while (j < count && (sharded ? plan->y_full[j] : plan->y[j]) == base + len) {
            len += plan->m * (sharded ? plan->n_total[j] : plan->layers[j]->n);
            ++j;
        }
        if (len) yr.push_back({base, off, len});
        off += len;
        i = j;
    }
    // Pinned host memory has a device alias: a kernel can do the copies.  That is worth it because
    // kernels chain with programmatic dependent launch where a copy engine's transfer does not:
    // the forward kernel starts streaming its weights while x is still crossing PCIe, and y leaves
    // in the tail of the forward kernel's grid.  Taken when both slabs are pinned (first and last
    // byte checked), the runs are few and everything is 16-byte aligned; NNE_HOST_COPY=engine
    // switches it off.
    const float *x_alias = nullptr;
    float *y_alias = nullptr;
    if (!sharded && xr.size() <= (size_t)HOST_COPY_SEGS && yr.size() <= (size_t)HOST_COPY_SEGS) {
        // (asked on every call: a cached answer would outlive the allocation it was given for)
        const size_t xb = (xr.empty() ? 0 : xr.back().off + xr.back().len) * sizeof(float);
        const size_t yb = (yr.empty() ? 0 : yr.back().off + yr.back().len) * sizeof(float);
        if (xb + yb <= HOST_COPY_KERNEL_MAX_BYTES) {
            x_alias = xb ? static_cast<const float *>(pinned_alias(x_all_host, xb)) : nullptr;
            y_alias = yb ? static_cast<float *>(pinned_alias(y_all_host, yb)) : nullptr;
        }
        bool ok16 = x_alias && y_alias && aligned(x_alias, 16) && aligned(y_alias, 16);
        for (const Run &r : xr) ok16 = ok16 && aligned(r.dev, 16) && r.off % 4 == 0 && r.len % 4 == 0;
        for (const Run &r : yr) ok16 = ok16 && aligned(r.dev, 16) && r.off % 4 == 0 && r.len % 4 == 0;
        if (!ok16) x_alias = nullptr;
    }
    if (x_alias) {
        HostCopySegs in = {}, out = {};
        for (const Run &r : xr) {
            in.seg[in.count].src = x_alias + r.off;
            in.seg[in.count].dst = r.dev;
            in.seg[in.count++].n4 = r.len / 4;
        }
        for (const Run &r : yr) {
            out.seg[out.count].src = r.dev;
            out.seg[out.count].dst = y_alias + r.off;
            out.seg[out.count++].n4 = r.len / 4;
        }
        NNE_TRY(launch_host_copy(ctx, in, false, s));
        NNE_TRY(plan_issue(plan, s));
        NNE_TRY(launch_host_copy(ctx, out, true, s));
    } else {
        for (const Run &r : xr)
            NNE_CUDA_TRY(cudaMemcpyAsync(r.dev, x_all_host + r.off, r.len * sizeof(float), cudaMemcpyHostToDevice, s));
        NNE_TRY(plan_issue(plan, s));
        if (sharded && plan->route == 0) NNE_TRY(shard_wait(plan->group, plan->group->epoch.load(), s));
        for (const Run &r : yr)
            NNE_CUDA_TRY(cudaMemcpyAsync(y_all_host + r.off, r.dev, r.len * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    NNE_CUDA_TRY(cudaStreamSynchronize(s));
    const int word = *ctx->err_host;
    if (word != 0) {
        *ctx->err_host = 0;
        return fail(NNE_ERR_TIMEOUT, "a kernel's bounded wait ran out (code 0x%x)", word);
    }
    return NNE_OK;
    NNE_GUARD_END
}

int nne_qlinear_plan_launches(const nne_plan *plan) {
    if (!plan) return 0;
    if (!plan->phases.empty()) {
        int total = 0;
        for (const nne_plan *sub : plan->phases) total += nne_qlinear_plan_launches(sub);
        return total;
    }
    if (plan->fused) return 1;
    const int extra = (int)(plan->pre_ops.size() + plan->post_ops.size());
    const int push = extra + ((plan->group && plan->group->world > 1 && plan->route == 0 && plan->seg_count) ? 1 : 0);  // + slice push kernel
    if (plan->skinny) return 2 + push;  // pre-pass + kernel
    return (int)plan->layers.size() + push;
}

#ifdef NNE_TRACE
NNE_API void *nne_debug_plan_trace(nne_plan *plan) { return plan ? plan->gsync_dev : nullptr; }
#endif

int nne_qlinear_plan_destroy(nne_plan *plan) {
    NNE_GUARD_BEGIN
    plan_free(plan);
    return NNE_OK;
    NNE_GUARD_END
}

}  // extern "C"
