// Decode-shape forward (m <= 4), TMA-staged: the main streaming kernel.
//   y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j])   (reference
//   src/nn/quantized.rs:184-192 with the dot product of :253-324), fp32 throughout.
//
// HBM bound.  Every CTA owns a contiguous range of output rows, which is a contiguous byte range
// of the [N,K] int8 matrix.  One producer thread streams it through a shared-memory ring with
// 1-D bulk copies (cp.async.bulk, R rows = up to 32 KB per copy, several copies in flight), so
// the amount of data in flight does not depend on registers or on how fast the math warps go.
// The consumer warps split K across the whole CTA: thread t owns the 16-byte chunks t + i*T of
// every row, so its slice of x is loaded once and stays in registers; partial sums are reduced
// with warp shuffles and one named barrier per stage.  Weights are read from HBM exactly once:
// algorithmic bytes per launch = N*K + 4N (scales) + 4N*[bias] + 4*m*K + 4*m*N.
//
// The kernel is launched with programmatic stream serialization: its producer starts filling
// the ring with WEIGHTS while the previous kernel in the stream is still draining, and only
// the consumers wait for that kernel (griddepcontrol.wait) before they touch x or y.  Weights
// are immutable once a layer exists, which is what makes that early read safe.
//
// Every mbarrier wait is bounded (~2 s): on expiry the context's device error word is set and
// the CTA drains and returns.
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"

namespace nne {
namespace {

// Four int8 packed in a word -> four f32, exactly (see gemv.cu for the derivation).
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

constexpr int MAX_STAGES = 8;
constexpr int MAX_WARPS = 16;

// MT activation rows, I chunks per thread per weight row; rows per stage follow from I so that a
// stage never exceeds 32 KB (I = 1: k <= 8192, I = 2: k <= 16384, I >= 3: k <= 32768).
template <int I>
struct StageRows {
    static constexpr int R = (I == 1) ? 4 : (I == 2) ? 2 : 1;
};

struct RingBars {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    int abort_flag;
};

template <int MT, int I>
__global__ void __launch_bounds__(544, 1)
qgemv_tma_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                 const float *__restrict__ bias, const float *__restrict__ x,
                 float *__restrict__ y, int n, int k, size_t ldy, int num_stages,
                 int stage_stride, int *err) {
    constexpr int R = StageRows<I>::R;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: ring [num_stages][stage_stride] | RingBars | part[2][MAX_WARPS][R*MT]
    uint8_t *ring = smem;
    RingBars *bars = reinterpret_cast<RingBars *>(smem + (size_t)num_stages * stage_stride);
    float *part = reinterpret_cast<float *>(bars + 1);

    const int T = blockDim.x - 32;  // consumer threads; the last warp is the producer
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int nwarps = T >> 5;
    const int chunks = k >> 4;
    volatile int *abort_flag = &bars->abort_flag;

    // contiguous row range of this CTA: as equal as rows allow
    const int per = n / gridDim.x, rem = n % gridDim.x;
    const int row0 = blockIdx.x * per + min((int)blockIdx.x, rem);
    const int cnt = per + ((int)blockIdx.x < rem ? 1 : 0);
    const int nst = (cnt + R - 1) / R;

    if (tid == 0) {
        for (int s = 0; s < num_stages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), nwarps);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream begin its own weight prefetch as soon as SMs free up.
    grid_launch_dependents();

    if (warp == nwarps) {
        // ---------------- producer: weights only, may run ahead of the previous kernel ----------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int s = 0; s < nst; ++s) {
                ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, err, 0x11);
                if (!ok) break;
                const int rows = min(R, cnt - s * R);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)k;
                const uint32_t full = smem_u32(&bars->full[stage]);
                mbar_arrive_expect_tx(full, bytes);
                bulk_load_1d(smem_u32(ring + (size_t)stage * stage_stride),
                             q + (size_t)(row0 + s * R) * k, bytes, full);
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                for (int s = 0; s < num_stages; ++s) {
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&bars->full[s]), 0) &&
                           !mbar_try_wait(smem_u32(&bars->full[s]), 1) &&
                           globaltimer_ns() - t0 < 100000000ull) {
                    }
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        grid_dependency_wait();  // x may be the previous kernel's output
        float xr[MT][I][16];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int i = 0; i < I; ++i) {
                const int c = tid + i * T;
                if (c < chunks) {
                    const float4 *p4 =
                        reinterpret_cast<const float4 *>(x + (size_t)m * k + (size_t)c * 16);
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const float4 t4 = __ldg(p4 + v);
                        xr[m][i][4 * v + 0] = t4.x;
                        xr[m][i][4 * v + 1] = t4.y;
                        xr[m][i][4 * v + 2] = t4.z;
                        xr[m][i][4 * v + 3] = t4.w;
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < 16; ++v) xr[m][i][v] = 0.0f;
                }
            }

        int stage = 0;
        uint32_t phase = 0;
        for (int s = 0; s < nst; ++s) {
            // If the wait runs out the error word is set and every later wait returns at once;
            // the warp still walks all stages so that no other warp is left alone at a barrier.
            (void)mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 0x12);
            const int rows = min(R, cnt - s * R);
            const uint8_t *st = ring + (size_t)stage * stage_stride;
            uint4 wv[R][I];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int i = 0; i < I; ++i) {
                    const int c = tid + i * T;
                    wv[r][i] = (r < rows && c < chunks)
                                   ? *reinterpret_cast<const uint4 *>(st + (size_t)r * k + (size_t)c * 16)
                                   : make_uint4(0u, 0u, 0u, 0u);
                }
            // the stage's bytes are in registers: hand the buffer back to the producer
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->empty[stage]));

            float acc[R][MT][2];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[r][m][0] = acc[r][m][1] = 0.0f;
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
                            acc[r][m][v & 1] = fmaf(xr[m][i][v], wf[v], acc[r][m][v & 1]);
                }
            float *pbuf = part + (size_t)(s & 1) * MAX_WARPS * (R * MT);
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float sum = warp_sum(acc[r][m][0] + acc[r][m][1]);
                    if (lane == 0) pbuf[warp * (R * MT) + r * MT + m] = sum;
                }
            named_bar_sync(1, T);
            if (tid < rows * MT) {
                float sum = 0.0f;
                for (int w = 0; w < nwarps; ++w) sum += pbuf[w * (R * MT) + tid];
                const int r = tid / MT, m = tid % MT;
                const int j = row0 + s * R + r;
                float val = __fmul_rn(sum, scales[j]);
                if (bias) val = __fadd_rn(val, bias[j]);
                y[(size_t)m * ldy + j] = val;
            }
            if (++stage == num_stages) { stage = 0; phase ^= 1; }
        }
    }
}

struct TmaPlan {
    int threads;  // consumer threads
    int I;
};

// T (multiple of 32, 64..512) and I (1..4) with T*I >= k/16, the fewest idle lanes, and the
// register-resident slice of x (MT*I*16 floats) at most 64 floats.
TmaPlan tma_plan(size_t k, int mt) {
    const int chunks = (int)(k >> 4);
    TmaPlan best{0, 0};
    double best_cost = 1e30;
    for (int I = 1; I <= 4; ++I) {
        if (mt * I > 4) continue;
        int T = (chunks + I - 1) / I;
        T = (T + 31) / 32 * 32;
        if (T > 512) continue;
        if (T < 64) T = 64;
        const double waste = (double)(T * I - chunks) / (double)(T * I);
        const double cost = waste + 0.01 * (I - 1);
        if (cost < best_cost) {
            best_cost = cost;
            best = TmaPlan{T, I};
        }
    }
    return best;
}

bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNE_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <int MT, int I>
int launch_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
               const float *x, float *y, size_t n, size_t k, size_t ldy, int threads,
               cudaStream_t s) {
    constexpr int R = StageRows<I>::R;
    const int stage_stride = (int)(((size_t)R * k + 127) & ~(size_t)127);
    // two CTAs per SM, each with about 100 KB of ring
    const size_t tail = sizeof(RingBars) + 2 * MAX_WARPS * R * MT * sizeof(float) + 128;
    int stages = (int)((100 * 1024 - tail) / (size_t)stage_stride);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * stage_stride + tail;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        NNE_CUDA_TRY(cudaFuncSetAttribute(qgemv_tma_kernel<MT, I>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    static int occ_cache[18] = {0};  // CTAs per SM, indexed by consumer threads / 32
    int occ = occ_cache[threads >> 5];
    if (occ == 0) {
        NNE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, qgemv_tma_kernel<MT, I>,
                                                                   threads + 32, smem));
        if (occ < 1) occ = 1;
        if (occ > 2) occ = 2;
        occ_cache[threads >> 5] = occ;
    }
    int grid = ctx->sm_count * occ;  // all CTAs resident at once: one wave, equal row ranges
    const int max_useful = (int)((n + R - 1) / R);
    if (grid > max_useful) grid = max_useful;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)(threads + 32));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, qgemv_tma_kernel<MT, I>, q, scales, bias, x, y, (int)n,
                                       (int)k, ldy, stages, stage_stride, ctx->err_word);
    count_launch();
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "streaming kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace

// m is the number of activation rows of ONE launch (1..4).
bool gemv_tma_supports(size_t n, size_t k, size_t m) {
    if (m < 1 || m > 4 || n == 0) return false;
    if (k % 16 != 0 || k < 512 || k > 32768) return false;
    if (n > 0x7fffffffu) return false;
    return tma_plan(k, (int)m).threads != 0;
}

int launch_gemv_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                    const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                    cudaStream_t s) {
    const TmaPlan p = tma_plan(k, (int)m);
#define NNE_TMA_CASE(MT_, I_)                                                                     \
    if (m == MT_ && p.I == I_)                                                                    \
        return launch_tma<MT_, I_>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
    NNE_TMA_CASE(1, 1)
    NNE_TMA_CASE(1, 2)
    NNE_TMA_CASE(1, 3)
    NNE_TMA_CASE(1, 4)
    NNE_TMA_CASE(2, 1)
    NNE_TMA_CASE(2, 2)
    NNE_TMA_CASE(3, 1)
    NNE_TMA_CASE(4, 1)
#undef NNE_TMA_CASE
    return fail(NNE_ERR_UNSUPPORTED, "no TMA streaming plan for k=%zu m=%zu", k, m);
}

}  // namespace nne
