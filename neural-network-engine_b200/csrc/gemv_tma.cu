// Decode-shape forward (m <= 2 per launch), TMA-staged: the main streaming kernel.
//   y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j])   (reference
//   src/nn/quantized.rs:184-192 with the dot product of :253-324).
//
// HBM bound.  Every CTA owns a contiguous range of output rows, i.e. a contiguous byte range of
// the [N,K] int8 matrix.  One producer thread streams it through a shared-memory ring with 1-D
// bulk copies (cp.async.bulk, up to 32 KB per copy, several in flight), so the bytes in flight
// do not depend on registers or on how fast the math warps go.  Weights are read from HBM
// exactly once: algorithmic bytes per launch = N*K + 4N (scales) + 4N*[bias] + 4*m*K + 4*m*N.
//
// Arithmetic.  Converting int8 weights to f32 costs more issue slots than the SM has at HBM
// speed, so the contraction runs on the integer dot-product unit instead.  Each activation row
// is put on a power-of-two fixed-point grid, v_i = rint(x_i * 2^e) with |v_i| <= 2^20 (e from
// the row's largest |x|), and v_i is split into three balanced base-128 digits held as int8.
// Then sum_i v_i*q_ji = D0 + 128*D1 + 16384*D2 with every D an EXACT int32 dp4a sum, and
// dot = that * 2^-e.  The only approximation is the rounding of x to the grid: at most
// 2^-21 * 2^ceil(log2 max|x|) per element, i.e. a result error below 1e-6 of the a-priori bound
// ||x||inf * scale_j * sum|q_jk| the path's tolerance is written against (tolerance: 1e-3 of it),
// the same size as fp32 summation error.  Scale and bias are applied as a separate fp32 multiply
// and add like the reference (:187-190).  Rows of x that hold Inf or NaN take an fp32 FMA loop
// in the same kernel, so those propagate as IEEE prescribes.
//
// Work split: consumer thread t owns the 16-byte chunks t + i*T of every weight row, so its slice
// of x (as digits) is prepared once and stays in registers; per stage the per-thread sums are
// reduced with a transposing warp-shuffle reduction and one named barrier.
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

__device__ __forceinline__ float pow2f(int p) {  // 2^p for p in [-126, 127]
    return __int_as_float((127 + p) << 23);
}

constexpr int MAX_STAGES = 8;
constexpr int MAX_WARPS = 16;
template <int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template <> struct Log2<1> { static constexpr int value = 0; };

// Reduces V per-lane values across the warp with V-1 + (5 - log2 V) shuffles: at every step a
// lane keeps half of its values and hands the other half to its partner.  On return lane l holds
// the warp total of value number l >> (5 - log2 V).
template <int V>
__device__ __forceinline__ float transposing_warp_sum(float (&v)[V], int lane) {
    int o = 16;
#pragma unroll
    for (int half = V / 2; half >= 1; half >>= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float keep = upper ? v[i + half] : v[i];
            const float send = upper ? v[i] : v[i + half];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
        o >>= 1;
    }
#pragma unroll
    for (int oo = 16 >> Log2<V>::value; oo >= 1; oo >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], oo);
    return v[0];
}

#ifdef NNE_TRACE
// Debug builds only: per-CTA timestamps (globaltimer ns) of the kernel's phases.
__device__ unsigned long long g_trace[1024 * 16];
#define NNE_TRACE_MARK(slot)                                                  \
    do {                                                                      \
        if (blockIdx.x < 1024) g_trace[blockIdx.x * 16 + (slot)] = globaltimer_ns(); \
    } while (0)
#else
#define NNE_TRACE_MARK(slot) \
    do {                     \
    } while (0)
#endif

struct RingBars {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    int abort_flag;
    int bad[MAX_WARPS];        // per consumer warp: its slice of x holds Inf/NaN
    float xmax[MAX_WARPS][2];  // per consumer warp and activation row: max |x|
};

// MT activation rows (1..2), I chunks per thread per weight row, R weight rows per stage.
template <int MT, int I, int R>
__global__ void __launch_bounds__(544, 1)
qgemv_tma_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                 const float *__restrict__ bias, const float *__restrict__ x,
                 float *__restrict__ y, int n, int k, size_t ldy, int num_stages,
                 int stage_stride, int sb_rows, int l2_prefetch, int *err) {
    constexpr int V = R * MT;  // sums per stage
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: ring [num_stages][stage_stride] | RingBars | part[2][MAX_WARPS][V] |
    //         scale_s[sb_rows] | bias_s[sb_rows]   (this CTA's rows; sb_rows = 0: read from global)
    uint8_t *ring = smem;
    RingBars *bars = reinterpret_cast<RingBars *>(smem + (size_t)num_stages * stage_stride);
    float *part = reinterpret_cast<float *>(bars + 1);
    float *scale_s = part + 2 * MAX_WARPS * V;
    float *bias_s = scale_s + sb_rows;

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
            NNE_TRACE_MARK(8);
            // Pull this CTA's whole byte range towards L2 right away: the DRAM stream then runs at
            // full depth from the first cycle (and, under programmatic dependent launch, already
            // while the previous kernel drains), independent of how small the shared ring is.
            const uint64_t pol_stream = l2_policy_evict_first();
            if (l2_prefetch) {
                const uint8_t *base = reinterpret_cast<const uint8_t *>(q) + (size_t)row0 * k;
                const size_t total = (size_t)cnt * k;
                for (size_t off = 0; off < total; off += 32768) {
                    const size_t left = total - off;
                    bulk_prefetch_l2(base + off, (uint32_t)(left < 32768 ? left : 32768), pol_stream);
                }
            }
            for (int s = 0; s < nst && ok; ++s) {
                ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, err, 0x11);
                if (!ok) break;
                if (s == num_stages) NNE_TRACE_MARK(9);
                const int rows = min(R, cnt - s * R);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)k;
                const uint32_t full = smem_u32(&bars->full[stage]);
                mbar_arrive_expect_tx(full, bytes);
                bulk_load_1d_hint(smem_u32(ring + (size_t)stage * stage_stride),
                                  q + (size_t)(row0 + s * R) * k, bytes, full, pol_stream);
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
            NNE_TRACE_MARK(10);
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
        return;
    }

    // ---------------- consumers ----------------
    if (tid == 0) NNE_TRACE_MARK(0);
    // Scales and bias are layer constants: fetch this CTA's rows before waiting for the previous
    // kernel.  Loads are unconditional from clamped addresses and masked afterwards, so no
    // predicated register write has to wait for a load that is still in flight.
    const uint64_t pol_keep = l2_policy_evict_last();  // activations and scales stay in L2
    float sc_pre[4], bs_pre[4];  // rows tid, tid+T, ... of this CTA (at most 4 per thread)
    if (sb_rows) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = min(tid + u * T, cnt - 1);
            sc_pre[u] = ldg_f1_hint(scales + row0 + i, pol_keep);
            bs_pre[u] = bias ? ldg_f1_hint(bias + row0 + i, pol_keep) : 0.0f;
        }
    }
    grid_dependency_wait();  // x may be the previous kernel's output
    if (tid == 0) NNE_TRACE_MARK(1);
    float xf[MT][I][16];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int i = 0; i < I; ++i) {
            const int c = min(tid + i * T, chunks - 1);
            const float4 *p4 = reinterpret_cast<const float4 *>(x + (size_t)m * k + (size_t)c * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const float4 t4 = ldg_f4_hint(p4 + v, pol_keep);
                xf[m][i][4 * v + 0] = t4.x;
                xf[m][i][4 * v + 1] = t4.y;
                xf[m][i][4 * v + 2] = t4.z;
                xf[m][i][4 * v + 3] = t4.w;
            }
        }
    float mx[MT];
    int bad = 0;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        mx[m] = 0.0f;
#pragma unroll
        for (int i = 0; i < I; ++i) {
            const bool live = (tid + i * T) < chunks;
#pragma unroll
            for (int v = 0; v < 16; ++v) {
                if (!live) xf[m][i][v] = 0.0f;
                const float a = fabsf(xf[m][i][v]);
                bad |= !(a <= 3.402823466e38f);  // Inf or NaN
                mx[m] = fmaxf(mx[m], a);
            }
        }
    }
    // CTA-wide max |x| per activation row and the Inf/NaN flag (consumer warps only)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xffffffffu, mx[m], o));
        if (lane == 0) bars->xmax[warp][m] = mx[m];
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) bars->bad[warp] = bad;
    if (sb_rows) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = tid + u * T;
            if (i < cnt) {
                scale_s[i] = sc_pre[u];
                bias_s[i] = bs_pre[u];
            }
        }
    }
    named_bar_sync(1, T);
    if (tid == 0) NNE_TRACE_MARK(2);
    bad = 0;
    for (int w = 0; w < nwarps; ++w) bad |= bars->bad[w];
    float unscale1[MT], unscale2[MT];  // dot = integer sum * unscale1 * unscale2  (= 2^-e)

    if (!bad) {
        // ---- integer path: digits of rint(x * 2^e) in registers, dp4a against the raw int8 codes
        int xs[MT][I][3][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float big = 0.0f;
            for (int w = 0; w < nwarps; ++w) big = fmaxf(big, bars->xmax[w][m]);
            const int e = 19 - ((big > 0.0f) ? ilogbf(big) : 0);  // max|x| * 2^e in [2^19, 2^20)
            const int e1 = e >> 1, e2 = e - e1;                     // 2^e = 2^e1 * 2^e2, both finite
            const float f1 = pow2f(e1), f2 = pow2f(e2);
            unscale1[m] = pow2f(-e1);
            unscale2[m] = pow2f(-e2);
#pragma unroll
            for (int i = 0; i < I; ++i)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t d[3] = {0u, 0u, 0u};
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        const int v = __float2int_rn(xf[m][i][4 * w + b] * f1 * f2);
                        const int d0 = ((v + 64) & 127) - 64;
                        const int v1 = (v - d0) >> 7;
                        const int d1 = ((v1 + 64) & 127) - 64;
                        const int d2 = (v1 - d1) >> 7;
                        d[0] |= (uint32_t)(d0 & 0xff) << (8 * b);
                        d[1] |= (uint32_t)(d1 & 0xff) << (8 * b);
                        d[2] |= (uint32_t)(d2 & 0xff) << (8 * b);
                    }
                    xs[m][i][0][w] = (int)d[0];
                    xs[m][i][1][w] = (int)d[1];
                    xs[m][i][2][w] = (int)d[2];
                }
        }

        int stage = 0;
        uint32_t phase = 0;
        if (tid == 0) NNE_TRACE_MARK(3);
        for (int s = 0; s < nst; ++s) {
            const int rows = min(R, cnt - s * R);
            float sc = 0.0f, bs = 0.0f;
            if (tid < rows * MT) {
                const int jl = s * R + tid / MT;
                if (sb_rows) {
                    sc = scale_s[jl];
                    bs = bias_s[jl];
                } else {
                    sc = __ldg(scales + row0 + jl);
                    if (bias) bs = __ldg(bias + row0 + jl);
                }
            }
            // If the wait runs out the error word is set and every later wait returns at once;
            // the warp still walks all stages so that no other warp is left alone at a barrier.
            (void)mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 0x12);
            if (tid == 0 && s == 0) NNE_TRACE_MARK(4);
            if (tid == 0 && s == 1) NNE_TRACE_MARK(5);
            if (tid == 0 && s == nst - 1) NNE_TRACE_MARK(6);
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

            float f[V];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
                    for (int i = 0; i < I; ++i) {
                        const int w4[4] = {(int)wv[r][i].x, (int)wv[r][i].y, (int)wv[r][i].z,
                                           (int)wv[r][i].w};
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            a0 = __dp4a(w4[w], xs[m][i][0][w], a0);
                            a1 = __dp4a(w4[w], xs[m][i][1][w], a1);
                            a2 = __dp4a(w4[w], xs[m][i][2][w], a2);
                        }
                    }
                    // |a| < 2^24, so the conversions are exact; the two FMAs round at 2^-24
                    f[r * MT + m] = fmaf(16384.0f, (float)a2, fmaf(128.0f, (float)a1, (float)a0));
                }
            const float total = transposing_warp_sum<V>(f, lane);
            float *pbuf = part + (size_t)(s & 1) * MAX_WARPS * V;
            if ((lane & ((32 >> Log2<V>::value) - 1)) == 0) pbuf[warp * V + (lane >> (5 - Log2<V>::value))] = total;
            named_bar_sync(1, T);
            if (tid < rows * MT) {
                float sum = 0.0f;
                for (int w = 0; w < nwarps; ++w) sum += pbuf[w * V + tid];
                const int r = tid / MT, m = tid % MT;
                const float dot = sum * unscale1[m] * unscale2[m];
                float val = __fmul_rn(dot, sc);
                if (bias) val = __fadd_rn(val, bs);
                y[(size_t)m * ldy + row0 + s * R + r] = val;
            }
            if (++stage == num_stages) { stage = 0; phase ^= 1; }
        }
        if (tid == 0) NNE_TRACE_MARK(7);
    } else {
        // ---- fp32 path for activations holding Inf/NaN: exact int8 -> f32, FMA accumulation
        int stage = 0;
        uint32_t phase = 0;
        for (int s = 0; s < nst; ++s) {
            const int rows = min(R, cnt - s * R);
            (void)mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 0x13);
            const uint8_t *st = ring + (size_t)stage * stage_stride;
            float f[V];
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int m = 0; m < MT; ++m) f[r * MT + m] = 0.0f;
#pragma unroll
                for (int i = 0; i < I; ++i) {
                    const int c = tid + i * T;
                    if (r < rows && c < chunks) {
                        const uint4 wq = *reinterpret_cast<const uint4 *>(st + (size_t)r * k + (size_t)c * 16);
                        float wf[16];
                        cvt_i8x4(wq.x, wf + 0);
                        cvt_i8x4(wq.y, wf + 4);
                        cvt_i8x4(wq.z, wf + 8);
                        cvt_i8x4(wq.w, wf + 12);
#pragma unroll
                        for (int m = 0; m < MT; ++m)
#pragma unroll
                            for (int v = 0; v < 16; ++v)
                                f[r * MT + m] = fmaf(xf[m][i][v], wf[v], f[r * MT + m]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->empty[stage]));
            const float total = transposing_warp_sum<V>(f, lane);
            float *pbuf = part + (size_t)(s & 1) * MAX_WARPS * V;
            if ((lane & ((32 >> Log2<V>::value) - 1)) == 0) pbuf[warp * V + (lane >> (5 - Log2<V>::value))] = total;
            named_bar_sync(1, T);
            if (tid < rows * MT) {
                float sum = 0.0f;
                for (int w = 0; w < nwarps; ++w) sum += pbuf[w * V + tid];
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
    int R;
};

// T (multiple of 32, 64..512) and I (1..4) with T*I >= k/16 and the fewest idle lanes, with the
// register-resident slice of x bounded (mt*I <= 4); R = rows per stage, at most 32 KB per stage.
TmaPlan tma_plan(size_t k, int mt) {
    const int chunks = (int)(k >> 4);
    TmaPlan best{0, 0, 0};
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
            best.threads = T;
            best.I = I;
        }
    }
    if (best.threads) {
        // instantiated (I, R) pairs: I=1 {8,4}, I=2 {4,2}, I=3 {2,1}, I=4 {2,1}
        const int hi = best.I == 1 ? 8 : best.I == 2 ? 4 : 2;
        best.R = ((size_t)hi * k <= 24576) ? hi : hi / 2;
        if ((size_t)best.R * k > 40960) best.threads = 0;
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

bool l2_prefetch_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNE_GEMV_L2PF");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Residency plan.  Default (1): one CTA per SM with a ring of about 100 KB, so that a CTA of the
// NEXT kernel in the stream fits on the same SM and prefetches its weights while this one runs.
// NNE_GEMV_CTAS=2: two CTAs of the same kernel per SM.  NNE_GEMV_CTAS=0: one CTA with a 200 KB ring.
int residency_mode() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("NNE_GEMV_CTAS");
        v = (e && e[0] == '2') ? 2 : (e && e[0] == '0') ? 0 : 1;
    }
    return v;
}

template <int MT, int I, int R>
int launch_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
               const float *x, float *y, size_t n, size_t k, size_t ldy, int threads,
               cudaStream_t s) {
    const int stage_stride = (int)(((size_t)R * k + 127) & ~(size_t)127);
    const int mode = residency_mode();
    const int want = mode == 2 ? 2 : 1;
    // rows per CTA (upper bound) -> shared scale/bias staging, unless that would eat the ring
    const int grid_guess = ctx->sm_count * want;
    int sb_rows = (int)((n + grid_guess - 1) / grid_guess) + 1;
    if (sb_rows > 4 * threads) sb_rows = 0;  // the prologue stages at most 4 rows per thread
    const size_t tail = sizeof(RingBars) + 2 * MAX_WARPS * R * MT * sizeof(float) +
                        2 * (size_t)sb_rows * sizeof(float) + 128;
    const size_t budget = (mode == 0 ? 200 : 100) * 1024;
    int stages = (int)((budget - tail) / (size_t)stage_stride);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    const size_t smem = (size_t)stages * stage_stride + tail;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        NNE_CUDA_TRY(cudaFuncSetAttribute(qgemv_tma_kernel<MT, I, R>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    static int occ_cache[18] = {0};  // CTAs per SM, indexed by consumer threads / 32
    int occ = occ_cache[threads >> 5];
    if (occ == 0) {
        NNE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &occ, qgemv_tma_kernel<MT, I, R>, threads + 32, smem));
        if (occ < 1) occ = 1;
        if (occ > want) occ = want;
        occ_cache[threads >> 5] = occ;
    }
    int grid = ctx->sm_count * occ;  // all CTAs resident at once: one wave, equal row ranges
    const int max_useful = (int)((n + R - 1) / R);
    if (grid > max_useful) grid = max_useful;
    if (sb_rows && (int)((n + grid - 1) / grid) > sb_rows) sb_rows = 0;  // fewer CTAs than guessed

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
    cudaError_t e = cudaLaunchKernelEx(&cfg, qgemv_tma_kernel<MT, I, R>, q, scales, bias, x, y,
                                       (int)n, (int)k, ldy, stages, stage_stride, sb_rows, l2_prefetch_enabled() ? 1 : 0,
                                       ctx->err_word);
    count_launch();
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "streaming kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace

#ifdef NNE_TRACE
extern "C" __attribute__((visibility("default"))) int nne_debug_read_trace(unsigned long long *out,
                                                                           size_t n) {
    return (int)cudaMemcpyFromSymbol(out, g_trace, n * sizeof(unsigned long long));
}
#endif

// m is the number of activation rows of ONE launch (1..2).
bool gemv_tma_supports(size_t n, size_t k, size_t m) {
    if (m < 1 || m > 2 || n == 0) return false;
    if (k % 16 != 0 || k < 512 || k > 32768) return false;
    if (n > 0x7fffffffu) return false;
    return tma_plan(k, (int)m).threads != 0;
}

int launch_gemv_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                    const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                    cudaStream_t s) {
    const TmaPlan p = tma_plan(k, (int)m);
#define NNE_TMA_CASE(MT_, I_, R_)                                                                 \
    if (m == MT_ && p.I == I_ && p.R == R_)                                                       \
        return launch_tma<MT_, I_, R_>(ctx, q, scales, bias, x, y, n, k, ldy, p.threads, s);
    NNE_TMA_CASE(1, 1, 8)
    NNE_TMA_CASE(1, 1, 4)
    NNE_TMA_CASE(1, 2, 4)
    NNE_TMA_CASE(1, 2, 2)
    NNE_TMA_CASE(1, 3, 2)
    NNE_TMA_CASE(1, 3, 1)
    NNE_TMA_CASE(1, 4, 2)
    NNE_TMA_CASE(1, 4, 1)
    NNE_TMA_CASE(2, 1, 8)
    NNE_TMA_CASE(2, 1, 4)
    NNE_TMA_CASE(2, 2, 4)
    NNE_TMA_CASE(2, 2, 2)
#undef NNE_TMA_CASE
    return fail(NNE_ERR_UNSUPPORTED, "no TMA streaming plan for k=%zu m=%zu", k, m);
}

}  // namespace nne
