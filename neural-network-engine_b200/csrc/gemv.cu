// Decode-shape forward (small m): y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j]),
// the device form of the j-loop in QLinear::forward_quantized (reference
// src/nn/quantized.rs:184-192) with its dot product (:253-324).
//
// The kernel is HBM bound: the int8 weight matrix [N,K] is streamed exactly once with 128-bit
// loads that bypass L1, activations are held in registers for the whole kernel, and every
// partial sum is reduced with warp shuffles.  Algorithmic bytes per launch:
//   N*K (codes) + 4N (scales) + 4N*[bias] + 4*m*K (x) + 4*m*N (y).
//
// Work split: a CTA of T threads owns groups of R consecutive output rows.  Thread t owns the
// 16-byte chunks c = t + i*T (i < I) of every row, so its slice of x never changes and stays in
// registers (I*16 floats per activation row).  int8 -> f32 is exact, accumulation is fp32 FMA,
// scale and bias are applied as a separate multiply and add like the reference (:187-190).
#include <stdlib.h>

#include "common.cuh"

namespace nne {
namespace {

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Four int8 packed in a word -> four f32, exactly.  Flipping the sign bits turns each byte into
// b+128 in [0,255]; placing it in the low mantissa byte of 2^23 gives the float 2^23 + b + 128,
// and one subtraction of 2^23 + 128 recovers b.
__device__ __forceinline__ void cvt_i8x4(uint32_t w, float *f) {
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Compile-time shape of one instantiation.  MT: activation rows (1..4).  I: 16-byte chunks per
// thread per weight row.  XREG: the thread's slice of x (MT*I*16 floats) lives in registers;
// otherwise it is re-read through L1 for every row group (weights bypass L1, so x stays there).
// R: weight rows per group.  MAXT: largest CTA the register budget allows.
template <int MT, int I>
struct GemvShape {
    static constexpr bool XREG = (MT * I <= 4);
    static constexpr int R = XREG ? (MT * I <= 2 ? 4 : 2) : 2;
    static constexpr int MAXT = (!XREG || MT * I <= 2) ? 512 : 448;
};

__device__ __forceinline__ void load_x16(const float *__restrict__ p, float *dst) {
    const float4 *p4 = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        float4 t = __ldg(p4 + v);
        dst[4 * v + 0] = t.x;
        dst[4 * v + 1] = t.y;
        dst[4 * v + 2] = t.z;
        dst[4 * v + 3] = t.w;
    }
}

template <int MT, int I>
__global__ void __launch_bounds__(GemvShape<MT, I>::MAXT)
qgemv_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
             const float *__restrict__ bias, const float *__restrict__ x, float *__restrict__ y,
             int n, int k, size_t ldy) {
    constexpr bool XREG = GemvShape<MT, I>::XREG;
    constexpr int R = GemvShape<MT, I>::R;
    __shared__ float part[16][R * MT];  // one slot per warp
    const int tid = threadIdx.x;
    const int T = blockDim.x;
    const int lane = tid & 31, wid = tid >> 5, nwarps = T >> 5;
    const int chunks = k >> 4;

    // This thread's slice of the activations, loaded once (XREG only).
    float xr[XREG ? MT : 1][XREG ? I : 1][16];
    if (XREG) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int i = 0; i < I; ++i) {
                const int c = tid + i * T;
                if (c < chunks) {
                    load_x16(x + (size_t)m * k + (size_t)c * 16, xr[XREG ? m : 0][XREG ? i : 0]);
                } else {
#pragma unroll
                    for (int v = 0; v < 16; ++v) xr[XREG ? m : 0][XREG ? i : 0][v] = 0.0f;
                }
            }
    }

    const int groups = (n + R - 1) / R;
    for (int g = blockIdx.x; g < groups; g += gridDim.x) {
        const int j0 = g * R;
        uint4 wv[R][I];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int j = min(j0 + r, n - 1);
            const uint4 *prow = reinterpret_cast<const uint4 *>(q + (size_t)j * k);
#pragma unroll
            for (int i = 0; i < I; ++i) {
                const int c = tid + i * T;
                wv[r][i] = (c < chunks) ? ldg_stream(prow + c) : make_uint4(0x0, 0x0, 0x0, 0x0);
            }
        }
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

        if (XREG) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int i = 0; i < I; ++i) {
                    float wf[16];
                    cvt_i8x4(wv[r][i].x, wf + 0);
                    cvt_i8x4(wv[r][i].y, wf + 4);
                    cvt_i8x4(wv[r][i].z, wf + 8);
                    cvt_i8x4(wv[r][i].w, wf + 12);
#pragma unroll
                    for (int m = 0; m < MT; ++m)
#pragma unroll
                        for (int v = 0; v < 16; ++v)
                            acc[r][m] = fmaf(xr[XREG ? m : 0][XREG ? i : 0][v], wf[v], acc[r][m]);
                }
        } else {
#pragma unroll
            for (int i = 0; i < I; ++i) {
                const int c = tid + i * T;
                float wf[R][16];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    cvt_i8x4(wv[r][i].x, wf[r] + 0);
                    cvt_i8x4(wv[r][i].y, wf[r] + 4);
                    cvt_i8x4(wv[r][i].z, wf[r] + 8);
                    cvt_i8x4(wv[r][i].w, wf[r] + 12);
                }
                if (c < chunks) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float xm[16];
                        load_x16(x + (size_t)m * k + (size_t)c * 16, xm);
#pragma unroll
                        for (int r = 0; r < R; ++r)
#pragma unroll
                            for (int v = 0; v < 16; ++v)
                                acc[r][m] = fmaf(xm[v], wf[r][v], acc[r][m]);
                    }
                }
            }
        }

#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float s = warp_sum(acc[r][m]);
                if (lane == 0) part[wid][r * MT + m] = s;
            }
        __syncthreads();
        if (tid < R * MT) {
            float s = 0.0f;
            for (int w = 0; w < nwarps; ++w) s += part[w][tid];
            const int r = tid / MT, m = tid % MT;
            const int j = j0 + r;
            if (j < n) {
                float val = __fmul_rn(s, scales[j]);
                if (bias) val = __fadd_rn(val, bias[j]);
                y[(size_t)m * ldy + j] = val;
            }
        }
        __syncthreads();
    }
}

// Any shape: one warp per output row, scalar byte loads, activation rows in blocks of 4.
// Takes the shapes the streaming kernel does not (k not a multiple of 16, unaligned bases).
__global__ void __launch_bounds__(256)
qlinear_generic_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                       const float *__restrict__ bias, const float *__restrict__ x,
                       float *__restrict__ y, size_t n, size_t k, size_t m, size_t ldy) {
    const int lane = threadIdx.x & 31;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t j = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); j < n;
         j += warps) {
        const int8_t *wrow = q + j * k;
        for (size_t r0 = (size_t)blockIdx.y * 4; r0 < m; r0 += (size_t)gridDim.y * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (size_t i = lane; i < k; i += 32) {
                const float wf = (float)wrow[i];
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (r0 + r < m) acc[r] = fmaf(x[(r0 + r) * k + i], wf, acc[r]);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float s = warp_sum(acc[r]);
                if (lane == 0 && r0 + r < m) {
                    float val = __fmul_rn(s, scales[j]);
                    if (bias) val = __fadd_rn(val, bias[j]);
                    y[(r0 + r) * ldy + j] = val;
                }
            }
        }
    }
}

struct GemvPlan {
    int threads;
    int chunks_per_thread;
};

template <int MT>
constexpr int max_threads_for(int I) {
    return I == 1 ? GemvShape<MT, 1>::MAXT
         : I == 2 ? GemvShape<MT, 2>::MAXT
         : I == 3 ? GemvShape<MT, 3>::MAXT
                  : GemvShape<MT, 4>::MAXT;
}

// Picks T (a multiple of 32) and I (<= 4) with T*I >= k/16 and the least idle lanes.
template <int MT>
GemvPlan plan_for(size_t k) {
    const int chunks = (int)(k >> 4);
    GemvPlan best{0, 0};
    double best_cost = 1e30;
    for (int I = 1; I <= 4; ++I) {
        int T = (chunks + I - 1) / I;
        T = (T + 31) / 32 * 32;
        if (T > max_threads_for<MT>(I)) continue;
        if (T < 64) T = 64;
        // idle fraction, with a mild preference for smaller CTAs (more of them per SM)
        double waste = (double)(T * I - chunks) / (double)(T * I);
        double cost = waste + (T > 384 ? 0.02 : 0.0) + (I > 2 ? 0.01 * (I - 2) : 0.0);
        if (cost < best_cost) {
            best_cost = cost;
            best = GemvPlan{T, I};
        }
    }
    return best;
}

template <int MT, int I>
int launch_one(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
               const float *x, float *y, size_t n, size_t k, size_t ldy, int threads,
               cudaStream_t s) {
    constexpr int R = GemvShape<MT, I>::R;
    static int per_sm_cache[17] = {0};  // indexed by threads / 32
    int per_sm = per_sm_cache[threads >> 5];
    if (per_sm == 0) {
        NNE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qgemv_kernel<MT, I>,
                                                                   threads, 0));
        if (per_sm < 1) per_sm = 1;
        per_sm_cache[threads >> 5] = per_sm;
    }
    const int groups = (int)((n + R - 1) / R);
    int grid = ctx->sm_count * per_sm;
    if (grid > groups) grid = groups;
    qgemv_kernel<MT, I><<<grid, threads, 0, s>>>(q, scales, bias, x, y, (int)n, (int)k, ldy);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

template <int MT>
int launch_mt(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
              const float *x, float *y, size_t n, size_t k, size_t ldy, cudaStream_t s) {
    const GemvPlan p = plan_for<MT>(k);
    switch (p.chunks_per_thread) {
        case 1: return launch_one<MT, 1>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
        case 2: return launch_one<MT, 2>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
        case 3: return launch_one<MT, 3>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
        case 4: return launch_one<MT, 4>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
        default: return fail(NNE_ERR_UNSUPPORTED, "no streaming plan for k=%zu", k);
    }
}

}  // namespace

bool gemv_supports(size_t n, size_t k, size_t m) {
    (void)m;
    if (n == 0 || k == 0) return false;
    if (k % 16 != 0) return false;
    if (n > 0x7fffffffu || k > 0x7fffffffu) return false;
    return plan_for<4>(k).threads != 0 && plan_for<1>(k).threads != 0;
}

int launch_gemv(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                cudaStream_t s) {
    // Activation rows go through in blocks of at most 4; each block streams the weights once.
    // A block goes to the TMA-staged kernel when its slice of x fits in registers there,
    // otherwise to the register-staged kernel in this file.
    static const bool no_tma = [] {
        const char *e = getenv("NNE_NO_TMA_GEMV");
        return e && e[0] == '1';
    }();
    if (!no_tma && m > 2 && m <= 2 * (size_t)STREAM_INLINE_LAYERS && gemv_tma_supports(n, k, 2))
        return launch_gemv_tma_passes(ctx, q, scales, bias, x, y, n, k, m, ldy, s);
    size_t r = 0;
    while (r < m) {
        const size_t left = m - r;
        size_t mt = left >= 4 ? 4 : left;
        const float *xb = x + r * k;
        float *yb = y + r * ldy;
        if (!no_tma) {
            // prefer the largest block the TMA kernel takes, down to 1
            size_t t = mt;
            while (t >= 1 && !gemv_tma_supports(n, k, t)) --t;
            if (t >= 1 && (t == mt || t >= 2 || mt == 1)) {
                NNE_TRY(launch_gemv_tma(ctx, q, scales, bias, xb, yb, n, k, t, ldy, s));
                r += t;
                continue;
            }
        }
        if (mt == 4) {
            NNE_TRY(launch_mt<4>(ctx, q, scales, bias, xb, yb, n, k, ldy, s));
        } else if (mt == 3) {
            NNE_TRY(launch_mt<3>(ctx, q, scales, bias, xb, yb, n, k, ldy, s));
        } else if (mt == 2) {
            NNE_TRY(launch_mt<2>(ctx, q, scales, bias, xb, yb, n, k, ldy, s));
        } else {
            NNE_TRY(launch_mt<1>(ctx, q, scales, bias, xb, yb, n, k, ldy, s));
        }
        r += mt;
    }
    return NNE_OK;
}

int launch_generic(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                   const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                   cudaStream_t s) {
    if (n == 0 || m == 0) return NNE_OK;
    size_t bx = (n + 7) / 8;
    const size_t cap = (size_t)ctx->sm_count * 8;
    if (bx > cap) bx = cap;
    size_t by = (m + 3) / 4;
    if (by > 64) by = 64;
    dim3 grid((unsigned)bx, (unsigned)by);
    qlinear_generic_kernel<<<grid, 256, 0, s>>>(q, scales, bias, x, y, n, k, m, ldy);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
}

}  // namespace nne
