// Quantize / dequantize kernels: the device form of the row loop in QLinear::from_linear
// (reference src/nn/quantized.rs:107-127), of Int8Tensor::from_raw (:32-57) and of the
// q * scale loops in Int8Tensor::dequantize (:60-67) and QLinear::to_linear (:200-209).
//
// Bit-exactness rules (codes and scales must equal the reference's byte for byte):
//   scale = max>0 ? max/127 : 1      IEEE f32 divide          -> __fdiv_rn
//   inv   = 1/scale                  IEEE f32 divide          -> __fdiv_rn
//   t     = v*inv                    one rounding, never fused -> __fmul_rn
//   q     = round half AWAY from zero, clamp [-128,127], NaN -> 0
// The absmax is a max of |v| that skips NaN, which is order independent, so a shuffle/atomic
// reduction gives the same bits as the reference's serial `if a > max_abs` loop.
// The file must be built without --use_fast_math, -ftz=true or -prec-div=false.
//
// HBM traffic per row-quantize launch: 4*rows*cols read + rows*cols + 4*rows written.
#include "common.cuh"
#include "ptx.cuh"

namespace nne {
namespace {

__device__ __forceinline__ float absmax_acc(float m, float v) {
    // fmaxf returns the non-NaN operand, so a NaN element never wins (reference :113-116).
    return fmaxf(m, fabsf(v));
}

__device__ __forceinline__ float scale_from_max(float max_abs) {
    return (max_abs > 0.0f) ? __fdiv_rn(max_abs, 127.0f) : 1.0f;
}

// round-half-away-from-zero, clamp to the int8 range, NaN -> 0 (Rust `as i8` semantics), without
// the conversion unit and with as few ALU-pipe instructions (min/max, compare, select, logic) as
// could be found - the kernel is bound by that pipe, not by HBM.  Clamping first gives the same code
// as clamping after the rounding and puts the value in the range of the magic-number rounding:
// u = c + 1.5 * 2^23 holds rint(c), half to even, in its low mantissa bits and u - 1.5 * 2^23 is
// that integer as a float.  d = c - rint(c) is exact and equals copysign(0.5, c) exactly when c is
// a tie that half-to-even sent TOWARD zero; the code then steps one away (in float, where the step
// is 2 d).  The last magic add turns the integer-valued float back into an int.
__device__ __forceinline__ int quant_code(float v, float inv_scale) {
    float t = __fmul_rn(v, inv_scale);
    t = (t == t) ? t : 0.0f;
    const float c = fminf(fmaxf(t, -128.0f), 127.0f);
    const float rf = __fsub_rn(__fadd_rn(c, 12582912.0f), 12582912.0f);
    const float d = __fsub_rn(c, rf);
    const float half = copysignf(0.5f, c);
    const float r = (d == half) ? __fadd_rn(rf, __fadd_rn(half, half)) : rf;
    return __float_as_int(__fadd_rn(r, 12582912.0f)) - 0x4B400000;
}

// Four codes -> one word, low byte first.
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return __byte_perm(__byte_perm((uint32_t)a, (uint32_t)b, 0x0040), __byte_perm((uint32_t)c, (uint32_t)d, 0x0040),
                       0x5410);
}

__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    return m;
}

// One CTA per row (grid-stride over rows).  The row is read from HBM once: pass 1 keeps it in
// shared memory while taking the absmax, pass 2 quantizes from shared memory.  Rows longer than
// the shared buffer re-read the overflow part from global memory (it is L2 resident).
// VEC: cols % 4 == 0 and both bases 16-/4-byte aligned, so float4 loads and 32-bit stores.
template <bool VEC>
__global__ void __launch_bounds__(256)
quantize_rows_cta_kernel(const float *__restrict__ w, size_t rows, size_t cols,
                         int8_t *__restrict__ q, float *__restrict__ scales, size_t cache_floats) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float warp_part[8];
    __shared__ float row_max;
    const int tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;

    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *src = w + row * cols;
        int8_t *dst = q + row * cols;
        float m = 0.0f;
        if (VEC) {
            const size_t n4 = cols >> 2, c4 = cache_floats >> 2;
            const float4 *src4 = reinterpret_cast<const float4 *>(src);
            float4 *cache4 = reinterpret_cast<float4 *>(row_cache);
            for (size_t i = tid; i < n4; i += blockDim.x) {
                float4 v = __ldcs(src4 + i);
                if (i < c4) cache4[i] = v;
                m = absmax_acc(absmax_acc(absmax_acc(absmax_acc(m, v.x), v.y), v.z), v.w);
            }
        } else {
            for (size_t i = tid; i < cols; i += blockDim.x) {
                float v = src[i];
                if (i < cache_floats) row_cache[i] = v;
                m = absmax_acc(m, v);
            }
        }
        m = warp_max(m);
        if (lane == 0) warp_part[wid] = m;
        __syncthreads();
        if (wid == 0) {
            float t = (lane < (int)(blockDim.x >> 5)) ? warp_part[lane] : 0.0f;
            t = warp_max(t);
            if (lane == 0) {
                row_max = t;
                scales[row] = scale_from_max(t);
            }
        }
        __syncthreads();
        const float inv = __fdiv_rn(1.0f, scale_from_max(row_max));
        if (VEC) {
            const size_t n4 = cols >> 2, c4 = cache_floats >> 2;
            const float4 *src4 = reinterpret_cast<const float4 *>(src);
            const float4 *cache4 = reinterpret_cast<const float4 *>(row_cache);
            uint32_t *dst4 = reinterpret_cast<uint32_t *>(dst);
            for (size_t i = tid; i < n4; i += blockDim.x) {
                float4 v = (i < c4) ? cache4[i] : __ldg(src4 + i);
                dst4[i] = pack4(quant_code(v.x, inv), quant_code(v.y, inv), quant_code(v.z, inv),
                                quant_code(v.w, inv));
            }
        } else {
            for (size_t i = tid; i < cols; i += blockDim.x) {
                float v = (i < cache_floats) ? row_cache[i] : src[i];
                dst[i] = (int8_t)quant_code(v, inv);
            }
        }
        __syncthreads();  // row_cache / row_max are reused by the next row
    }
}

// The same row loop with the row brought into shared memory by a 1-D bulk copy, two rows per CTA
// in flight: while a row is reduced and coded out of one buffer the next one is already on its
// way into the other, so the CTA always has loads outstanding (the kernel above has none while it
// computes).  Needs cols % 4 == 0, a 16-byte aligned base and a row of at most 64 KB.
__global__ void __launch_bounds__(256)
quantize_rows_bulk_kernel(const float *__restrict__ w, size_t rows, size_t cols,
                          int8_t *__restrict__ q, float *__restrict__ scales, int *err) {
    extern __shared__ __align__(128) uint8_t qsmem[];
    __shared__ uint64_t full[2];
    __shared__ float warp_part[8];
    __shared__ float row_max;
    __shared__ int abort_word;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const uint32_t row_bytes = (uint32_t)(cols * sizeof(float));
    const size_t n4 = cols >> 2;
    volatile int *abort_flag = &abort_word;
    if (tid == 0) {
        mbar_init(smem_u32(&full[0]), 1);
        mbar_init(smem_u32(&full[1]), 1);
        abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint64_t pol = l2_policy_evict_first();
        for (int b = 0; b < 2; ++b) {
            const size_t row = (size_t)blockIdx.x + (size_t)b * gridDim.x;
            if (row < rows) {
                mbar_arrive_expect_tx(smem_u32(&full[b]), row_bytes);
                bulk_load_1d_hint(smem_u32(qsmem + (size_t)b * row_bytes), w + row * cols, row_bytes,
                                  smem_u32(&full[b]), pol);
            }
        }
    }
    __syncthreads();
    size_t it = 0;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
        const int b = (int)(it & 1);
        if (!mbar_wait(smem_u32(&full[b]), (uint32_t)((it >> 1) & 1), abort_flag, err, 0x41)) break;
        const float4 *cache4 = reinterpret_cast<const float4 *>(qsmem + (size_t)b * row_bytes);
        float m = 0.0f;
        for (size_t i = tid; i < n4; i += 256) {
            const float4 v = cache4[i];
            m = absmax_acc(absmax_acc(absmax_acc(absmax_acc(m, v.x), v.y), v.z), v.w);
        }
        m = warp_max(m);
        if (lane == 0) warp_part[wid] = m;
        __syncthreads();
        if (wid == 0) {
            float t = (lane < 8) ? warp_part[lane] : 0.0f;
            t = warp_max(t);
            if (lane == 0) {
                row_max = t;
                scales[row] = scale_from_max(t);
            }
        }
        __syncthreads();
        const float inv = __fdiv_rn(1.0f, scale_from_max(row_max));
        uint32_t *dst4 = reinterpret_cast<uint32_t *>(q + row * cols);
        for (size_t i = tid; i < n4; i += 256) {
            const float4 v = cache4[i];
            dst4[i] = pack4(quant_code(v.x, inv), quant_code(v.y, inv), quant_code(v.z, inv),
                            quant_code(v.w, inv));
        }
        __syncthreads();  // every thread is done with buffer b, warp_part and row_max
        if (tid == 0) {
            const size_t next = row + 2 * (size_t)gridDim.x;
            if (next < rows) {
                fence_proxy_async();  // the generic-proxy reads above come before the async write
                mbar_arrive_expect_tx(smem_u32(&full[b]), row_bytes);
                bulk_load_1d_hint(smem_u32(qsmem + (size_t)b * row_bytes), w + next * cols, row_bytes,
                                  smem_u32(&full[b]), l2_policy_evict_first());
            }
        }
    }
    // A wait that ran out leaves copies in flight: let them land before the CTA exits.
    if (*abort_flag && tid == 0) {
        for (int b = 0; b < 2; ++b) {
            const unsigned long long t0 = globaltimer_ns();
            while (!mbar_try_wait(smem_u32(&full[b]), 0) && !mbar_try_wait(smem_u32(&full[b]), 1) &&
                   globaltimer_ns() - t0 < 100000000ull) {
            }
        }
    }
}

// One warp per row, for short rows (cols <= 1024): the second pass re-reads the row, which is
// at most 4 KB and still in L1.  Many short rows (e.g. 64 -> 128 layers) stay efficient.
__global__ void __launch_bounds__(256)
quantize_rows_warp_kernel(const float *__restrict__ w, size_t rows, size_t cols,
                          int8_t *__restrict__ q, float *__restrict__ scales) {
    const int lane = threadIdx.x & 31;
    const size_t warps_per_grid = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
         row += warps_per_grid) {
        const float *src = w + row * cols;
        int8_t *dst = q + row * cols;
        float m = 0.0f;
        for (size_t i = lane; i < cols; i += 32) m = absmax_acc(m, src[i]);
        m = warp_max(m);
        const float scale = scale_from_max(m);
        if (lane == 0) scales[row] = scale;
        const float inv = __fdiv_rn(1.0f, scale);
        for (size_t i = lane; i < cols; i += 32) dst[i] = (int8_t)quant_code(src[i], inv);
    }
}

// ---- per-tensor (Int8Tensor::from_raw) ------------------------------------------------------
// Pass 1: grid-wide absmax into one 32-bit word.  For non-negative, non-NaN floats the bit
// pattern orders like the value, so atomicMax on the bits is an exact float max.
__global__ void __launch_bounds__(256)
absmax_kernel(const float *__restrict__ v, size_t n, unsigned int *__restrict__ max_bits) {
    __shared__ float warp_part[8];
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    float m = 0.0f;
    const bool vec = ((reinterpret_cast<uintptr_t>(v) & 15u) == 0);
    size_t body = vec ? (n & ~(size_t)3) : 0;
    const float4 *v4 = reinterpret_cast<const float4 *>(v);
    for (size_t i = tid; i < (body >> 2); i += nthreads) {
        float4 t = __ldcs(v4 + i);
        m = absmax_acc(absmax_acc(absmax_acc(absmax_acc(m, t.x), t.y), t.z), t.w);
    }
    for (size_t i = body + tid; i < n; i += nthreads) m = absmax_acc(m, v[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x >> 5)) ? warp_part[threadIdx.x] : 0.0f;
        t = warp_max(t);
        if (threadIdx.x == 0) atomicMax(max_bits, __float_as_uint(t));
    }
}

// Pass 2: every thread derives the same scale from the reduced max; thread 0 publishes it.
__global__ void __launch_bounds__(256)
quantize_with_max_kernel(const float *__restrict__ v, size_t n,
                         const unsigned int *__restrict__ max_bits, int8_t *__restrict__ q,
                         float *__restrict__ scale_out) {
    const float scale = scale_from_max(__uint_as_float(*max_bits));
    const float inv = __fdiv_rn(1.0f, scale);
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    if (tid == 0) *scale_out = scale;
    const bool vec = ((reinterpret_cast<uintptr_t>(v) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 3u) == 0);
    size_t body = vec ? (n & ~(size_t)3) : 0;
    const float4 *v4 = reinterpret_cast<const float4 *>(v);
    uint32_t *q4 = reinterpret_cast<uint32_t *>(q);
    for (size_t i = tid; i < (body >> 2); i += nthreads) {
        float4 t = __ldcs(v4 + i);
        q4[i] = pack4(quant_code(t.x, inv), quant_code(t.y, inv), quant_code(t.z, inv),
                      quant_code(t.w, inv));
    }
    for (size_t i = body + tid; i < n; i += nthreads) q[i] = (int8_t)quant_code(v[i], inv);
}

// out[r, c] = (f32)q[r, c] * scales[r]   (exact int8 -> f32, one rounding in the multiply)
__global__ void __launch_bounds__(256)
dequantize_rows_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                       size_t rows, size_t cols, float *__restrict__ out) {
    for (size_t row = blockIdx.y; row < rows; row += gridDim.y) {
        const float s = scales[row];
        const int8_t *src = q + row * cols;
        float *dst = out + row * cols;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < cols;
             i += (size_t)gridDim.x * blockDim.x)
            dst[i] = __fmul_rn((float)src[i], s);
    }
}

}  // namespace

// NNE_QUANT_BULK=0 keeps the register-staged row kernel.
static bool quantize_bulk_disabled() {
    static const bool v = []() {
        const char *e = getenv("NNE_QUANT_BULK");
        return e && e[0] == '0';
    }();
    return v;
}

int launch_quantize_rows(nne_ctx *ctx, const float *w, size_t rows, size_t cols, int8_t *q,
                         float *scales, cudaStream_t s) {
    if (rows == 0) return NNE_OK;
    if (cols == 0) {
        // Empty rows: absmax 0 -> scale 1.0, no codes.  Done with a 1-column view of nothing.
        quantize_rows_warp_kernel<<<(unsigned)((rows + 7) / 8 > 65535 ? 65535 : (rows + 7) / 8),
                                    256, 0, s>>>(w, rows, 0, q, scales);
        NNE_LAUNCH_CHECK();
        return NNE_OK;
    }
    if (cols <= 1024) {
        size_t blocks = (rows + 7) / 8;
        size_t cap = (size_t)ctx->sm_count * 8;
        if (blocks > cap) blocks = cap;
        quantize_rows_warp_kernel<<<(unsigned)blocks, 256, 0, s>>>(w, rows, cols, q, scales);
        NNE_LAUNCH_CHECK();
        return NNE_OK;
    }
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(q) & 3u) == 0);
    if (vec && cols * sizeof(float) <= 64 * 1024 && !quantize_bulk_disabled()) {
        // two row buffers per CTA; as many CTAs per SM as 200 KB of shared memory hold (at most 6)
        const size_t smem2 = 2 * cols * sizeof(float);
        size_t per = (200 * 1024) / smem2;
        if (per > 6) per = 6;
        if (per < 1) per = 1;
        size_t nblocks = rows;
        if (nblocks > (size_t)ctx->sm_count * per) nblocks = (size_t)ctx->sm_count * per;
        NNE_TRY(ensure_dynamic_smem(ctx->device, quantize_rows_bulk_kernel, smem2));
        quantize_rows_bulk_kernel<<<(unsigned)nblocks, 256, smem2, s>>>(w, rows, cols, q, scales,
                                                                       ctx->err_word);
        NNE_LAUNCH_CHECK();
        return NNE_OK;
    }
    // Shared row cache: the whole row when it fits in 64 KB (3 CTAs/SM), else the first 64 KB.
    size_t cache_floats = cols < 16384 ? cols : 16384;
    cache_floats &= ~(size_t)3;
    size_t smem = cache_floats * sizeof(float);
    size_t blocks = rows;
    size_t per_sm = smem ? (200 * 1024) / smem : 8;
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    size_t cap = (size_t)ctx->sm_count * per_sm;
    if (blocks > cap) blocks = cap;
    if (vec) {
        NNE_TRY(ensure_dynamic_smem(ctx->device, quantize_rows_cta_kernel<true>, smem));
        quantize_rows_cta_kernel<true><<<(unsigned)blocks, 256, smem, s>>>(w, rows, cols, q, scales,
                                                                         cache_floats);
    } else {
        NNE_TRY(ensure_dynamic_smem(ctx->device, quantize_rows_cta_kernel<false>, smem));
        quantize_rows_cta_kernel<false><<<(unsigned)blocks, 256, smem, s>>>(w, rows, cols, q,
                                                                          scales, cache_floats);
    }
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

int launch_quantize_tensor(nne_ctx *ctx, const float *v, size_t n, int8_t *q, float *scale_dev,
                           unsigned int *absmax_word, cudaStream_t s) {
    NNE_CUDA_TRY(cudaMemsetAsync(absmax_word, 0, sizeof(unsigned int), s));
    size_t blocks = (n / 4 + 255) / 256;
    size_t cap = (size_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    absmax_kernel<<<(unsigned)blocks, 256, 0, s>>>(v, n, absmax_word);
    NNE_LAUNCH_CHECK();
    quantize_with_max_kernel<<<(unsigned)blocks, 256, 0, s>>>(v, n, absmax_word, q, scale_dev);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

int launch_dequantize_rows(nne_ctx *ctx, const int8_t *q, const float *scales, size_t rows,
                           size_t cols, float *out, cudaStream_t s) {
    if (rows == 0 || cols == 0) return NNE_OK;
    size_t bx = (cols + 255) / 256;
    size_t capx = (size_t)ctx->sm_count * 8;
    if (bx > capx) bx = capx;
    size_t by = rows > 65535 ? 65535 : rows;
    while (bx * by > capx * 4 && by > 1) by = (by + 1) / 2;
    dim3 grid((unsigned)bx, (unsigned)by);
    dequantize_rows_kernel<<<grid, 256, 0, s>>>(q, scales, rows, cols, out);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

}  // namespace nne
