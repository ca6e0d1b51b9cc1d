// The element-wise steps either side of a QLinear in a LLaMA decoder block, as device kernels:
//   RMSNorm      y = (x * rrms) * gamma, rrms = 1 / sqrt(mean(x^2) + eps)   (reference
//                src/nn/norm.rs:141-165 with the row function :517-577; WGSL form
//                src/gpu/shaders/layernorm.wgsl:23-36)
//   SiLU * up    h = (g / (1 + exp(-g))) * u                                (src/models/llama.rs:343-346,
//                src/tensor/ops.rs:177-179; WGSL form src/gpu/shaders/elementwise.wgsl:54-58)
//   residual     y = a + b                                                   (src/models/llama.rs:377-392)
// All three are HBM bound (8 to 12 bytes per element).  The forward kernels can take the first two
// as input transforms and the third as an output step, so that a chain of QLinears never leaves
// the device between layers and these standalone launches are only needed where a forward kernel
// does not fuse them.  fp32 throughout, IEEE division and square root, no fast-math.
#include "common.cuh"

namespace nne {
namespace {

__device__ __forceinline__ float silu_mul_one(float g, float u) {
    // x / (1 + exp(-x)), then the product, as separate fp32 operations
    const float s = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(s, u);
}

// One CTA per row at a time (256 threads); the row is read twice (the second time from L1/L2).
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float *__restrict__ x, const float *__restrict__ gamma, float eps, size_t rows,
                    size_t cols, float *__restrict__ y) {
    __shared__ float wsum[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float *xr = x + r * cols;
        float acc = 0.0f;
        for (size_t c = tid; c < cols; c += 256) acc = fmaf(xr[c], xr[c], acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        __syncthreads();  // wsum of the previous row has been read by everybody
        if (lane == 0) wsum[warp] = acc;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += wsum[w];
        const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)cols), eps)));
        float *yr = y + r * cols;
        for (size_t c = tid; c < cols; c += 256) yr[c] = __fmul_rn(__fmul_rn(xr[c], rrms), gamma[c]);
    }
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const float *__restrict__ gate, const float *__restrict__ up, size_t n, float *__restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
        out[i] = silu_mul_one(gate[i], up[i]);
}

__global__ void __launch_bounds__(256)
add_kernel(const float *__restrict__ a, const float *__restrict__ b, size_t n, float *__restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
        out[i] = __fadd_rn(a[i], b[i]);
}

// Up to HOST_COPY_SEGS runs of float4 moved between pinned host memory (through its device alias)
// and device buffers by the SMs instead of a copy engine.  wait_first: the sources are results of
// the previous kernel of the stream, which this kernel - launched with programmatic stream
// serialization - may otherwise overtake.
__global__ void __launch_bounds__(256)
host_copy_kernel(const HostCopySegs segs, int wait_first) {
    if (wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
    // the kernel after this one may start its prologue (its weight stream) while the copy runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int g = 0; g < segs.count; ++g) {
        const float4 *src = reinterpret_cast<const float4 *>(segs.seg[g].src);
        float4 *dst = reinterpret_cast<float4 *>(segs.seg[g].dst);
        const size_t n4 = segs.seg[g].n4;
        for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) dst[i] = src[i];
    }
}

unsigned grid_for(const nne_ctx *ctx, size_t work_items) {
    size_t blocks = (work_items + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    return (unsigned)(blocks ? blocks : 1);
}

}  // namespace

int launch_host_copy(nne_ctx *ctx, const HostCopySegs &segs, bool results_of_previous_kernel, cudaStream_t s) {
    size_t n4 = 0;
    for (int g = 0; g < segs.count; ++g) n4 = n4 > segs.seg[g].n4 ? n4 : segs.seg[g].n4;
    if (n4 == 0) return NNE_OK;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > 64) blocks = 64;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (results_of_previous_kernel && pdl_enabled()) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, host_copy_kernel, segs, results_of_previous_kernel ? 1 : 0);
    count_launch();
    if (e != cudaSuccess) return fail(NNE_ERR_CUDA, "host copy kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

int launch_rmsnorm(nne_ctx *ctx, const float *x, const float *gamma, float eps, size_t rows, size_t cols,
                   float *y, cudaStream_t s) {
    if (rows == 0 || cols == 0) return NNE_OK;
    size_t blocks = rows < (size_t)ctx->sm_count * 8 ? rows : (size_t)ctx->sm_count * 8;
    rmsnorm_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, gamma, eps, rows, cols, y);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

int launch_silu_mul(nne_ctx *ctx, const float *gate, const float *up, size_t n, float *out, cudaStream_t s) {
    if (n == 0) return NNE_OK;
    silu_mul_kernel<<<grid_for(ctx, n), 256, 0, s>>>(gate, up, n, out);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

int launch_add(nne_ctx *ctx, const float *a, const float *b, size_t n, float *out, cudaStream_t s) {
    if (n == 0) return NNE_OK;
    add_kernel<<<grid_for(ctx, n), 256, 0, s>>>(a, b, n, out);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

}  // namespace nne

using namespace nne;

extern "C" {

int nne_rmsnorm_dev(nne_ctx *ctx, const float *x_dev, const float *gamma_dev, float eps, size_t rows,
                    size_t cols, float *y_dev, void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    size_t t;
    if (__builtin_mul_overflow(rows, cols, &t) || __builtin_mul_overflow(t, sizeof(float), &t))
        return fail(NNE_ERR_INVALID_ARGUMENT, "rows*cols overflows size_t");
    if (rows == 0) return NNE_OK;
    if (cols == 0) return fail(NNE_ERR_INVALID_ARGUMENT, "RMSNorm over an empty dimension");
    if (!x_dev || !gamma_dev || !y_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_rmsnorm(ctx, x_dev, gamma_dev, eps, rows, cols, y_dev, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_silu_mul_dev(nne_ctx *ctx, const float *gate_dev, const float *up_dev, size_t n, float *out_dev,
                     void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (n == 0) return NNE_OK;
    if (!gate_dev || !up_dev || !out_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_silu_mul(ctx, gate_dev, up_dev, n, out_dev, (cudaStream_t)stream);
    NNE_GUARD_END
}

int nne_add_dev(nne_ctx *ctx, const float *a_dev, const float *b_dev, size_t n, float *out_dev, void *stream) {
    NNE_GUARD_BEGIN
    NNE_TRY(use_ctx(ctx));
    if (n == 0) return NNE_OK;
    if (!a_dev || !b_dev || !out_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null device pointer");
    return launch_add(ctx, a_dev, b_dev, n, out_dev, (cudaStream_t)stream);
    NNE_GUARD_END
}

}  // extern "C"
