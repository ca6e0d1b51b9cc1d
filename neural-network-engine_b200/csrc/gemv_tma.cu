// Decode-shape forward (m <= 2 activation rows per launch), TMA-staged: the main streaming kernel.
//   y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j])   (reference
//   src/nn/quantized.rs:184-192 with the dot product of :253-324).
//
// HBM bound.  One launch serves a LIST of layers (a single forward is a list of one; a layer
// marked `sync` consumes what earlier layers of the list wrote, and the grid meets before its
// activations are prepared): every CTA owns a contiguous range of output rows of each layer, i.e. a contiguous byte
// range of that layer's [N,K] int8 matrix, and one producer thread streams those ranges, layer
// after layer, through a shared-memory ring with 1-D bulk copies (cp.async.bulk, 8-24 KB each,
// several in flight).  The bytes in flight therefore do not depend on registers or on how fast
// the math warps go, and the stream does not stop at a layer boundary: while the consumer warps
// prepare the next layer's activations the ring keeps filling with that layer's weights.
// Weights are read from HBM exactly once: algorithmic bytes per layer =
// N*K + 4N (scales) + 4N*[bias] + 4*m*K + 4*m*N.
// What bounds the stream is the bytes one SM can have on their way: ring bytes / (time a slot is in
// flight + time its warp works on it).  Shared memory limits the ring to 100-130 KB, so the producer
// also asks for the stages 64-192 KB AHEAD of the ring to be brought into L2 (cp.async.bulk.prefetch):
// the ring's own copy then comes from L2 in well under a microsecond, which is worth 8 % on a
// 12-layer launch and 20 % on 28672-wide layers.
//
// Arithmetic.  Converting int8 weights to f32 costs several instructions per byte, so the
// contraction runs on the integer dot-product unit instead.  Each activation row is put on a
// power-of-two fixed-point grid, v_i = rint(x_i * 2^e) with |v_i| < 2^15 (e from the row's
// largest |x|), and v_i is split into two balanced base-256 digits held as int8.  Then
// sum_i v_i*q_ji = D0 + 256*D1 with every D an EXACT int32 dp4a sum, and
// dot = that * 2^-e, rounded to f32 once.  The only approximation is the rounding of x to the
// grid: at most 2^-15 of the row's largest |x| per element, i.e. a result error of at most 3 % of
// the path's tolerance (1e-3 * ||x||inf * scale_j * sum|q_jk|) and about 0.1 % of it on random
// data (the errors of the elements do not add up in one direction).  Three base-128 digits
// (|v| <= 2^20) were the first form: a third more dot products, digit bytes and shared memory for
// an error the tolerance does not ask for; measured, the two-digit kernel streams 5-9 % faster.
// Scale and bias are applied as a
// separate fp32 multiply and add like the reference (:187-190).  Rows of x that hold Inf or NaN
// take an fp32 FMA loop in the same kernel, so those propagate as IEEE prescribes.
//
// Work split: math warp w is bound to ring slot w and takes the stages that land there (a stage =
// 1-4 weight rows).  Its 32 lanes split K in 16-byte chunks; the integer sums are reduced with
// redux.sync.  Seven more warps prepare the digit planes of the NEXT layer's activations (and stage
// its scales and bias) into the second of two shared buffers meanwhile, so at a layer boundary
// neither the math warps nor the weight stream wait for activations.  No CTA-wide barrier: every
// warp free-runs between mbarriers.  Sixteen warps in all, four per SM sub-partition, which is what
// lets every thread have 128 registers (a seventeenth warp would cap them at 96 and spill).
//
// The kernel is launched with programmatic stream serialization: its producer starts filling
// the ring with WEIGHTS while the previous kernel in the stream is still draining, and only
// the consumers wait for that kernel (griddepcontrol.wait) before they touch x or y.  Weights
// are immutable once a layer exists, which is what makes that early read safe.
//
// Every mbarrier wait is bounded (~2 s): on expiry the context's device error word is set and
// the CTA drains and returns.  The only hardware barrier is the one among the prep warps,
// each of which executes it the same fixed number of times per layer.
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"
#include "shard.cuh"

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

constexpr int NP = ACT_PLANES, DIGIT_BITS = ACT_DIGIT_BITS;
constexpr int MAX_SLOTS = 8;   // ring slots = math warps
constexpr int MATH_WARPS = 8;  // warps 0..7: one ring slot each
constexpr int PREP_WARPS = 7;  // warps 8..14: prepare the next layer's activations
constexpr int PREP_THREADS = PREP_WARPS * 32;
constexpr int THREADS = (MATH_WARPS + PREP_WARPS + 1) * 32;  // + the producer warp (last)

// Per activation buffer: what a math warp needs when it finishes an output.  Kept in shared memory
// and read at that point, not carried in registers through the dot-product loop (one more live
// pointer there costs the kernel a tenth of its speed).
struct LayerConsts {
    float unscale[2][2];    // per activation row: dot = integer sum * [0] * [1]
    const float *residual;  // added to the result (laid out like y), or null
};

struct RingBars {
    uint64_t full[MAX_SLOTS];    // slot's bytes have landed
    uint64_t empty[MAX_SLOTS];   // slot's bytes have been consumed
    uint64_t xs_full[2];         // activation buffer b is prepared (count: prep warps)
    uint64_t xs_empty[2];        // every math warp is done with activation buffer b (count: math warps)
    uint64_t gsync;              // every math warp has stored its results of the layers before a chained one
    int abort_flag;
    uint32_t gsync_parity;       // phase of `gsync` the next rendezvous waits for (one thread's variable)
#ifdef NNE_TRACE
    int tr_j, tr_jm;
#endif
    int bad_warp[PREP_WARPS];    // per prep warp: its part of x holds Inf/NaN
    float xmax[PREP_WARPS][2];   // per prep warp and activation row: max |x|
    int bad[2];                  // per buffer: the layer's x holds Inf/NaN
    LayerConsts lc[2];           // per buffer
    float sumsq[2][PREP_WARPS][2];  // RMSNorm input: per layer parity, prep warp and row, sum of x^2
    float rrms[2][2];            // per buffer and activation row: 1 / sqrt(mean(x^2) + eps)
};

// Element `col` of row m of the layer's effective input x' (see StreamLayer), from the raw x value.
__device__ __forceinline__ float input_value(const StreamLayer &L, float xv, int m, size_t col, float rrms) {
    if (L.gamma) return __fmul_rn(__fmul_rn(xv, rrms), __ldg(L.gamma + col));
    if (L.x2) {
        const float s = __fdiv_rn(xv, __fadd_rn(1.0f, expf(-xv)));
        return __fmul_rn(s, L.x2[(size_t)m * L.k + col]);
    }
    return xv;
}

// Row range of CTA `b` of `g` for a layer of n rows: contiguous, as equal as rows allow.
__host__ __device__ inline void cta_rows(int n, int b, int g, int &row0, int &cnt) {
    const int per = n / g, rem = n % g;
    row0 = b * per + (b < rem ? b : rem);
    cnt = per + (b < rem ? 1 : 0);
}

// Digits of one 16-element chunk of x on the grid 2^-e: v = rint(x * f1 * f2), |v| < 2^ACT_GRID_BITS,
// v = sum_p d_p * 2^(p * DIGIT_BITS) with balanced digits that fit int8; byte b of word w holds
// element 4w+b.
__device__ __forceinline__ void chunk_digits(const float (&xv)[16], float f1, float f2, uint4 (&o)[NP]) {
    if constexpr (NP == 2) {
        // Two base-256 digits straight from the bits of x * 2^e + 1.5 * 2^23: that float's low 23
        // bits hold v in two's complement, so byte 0 of the word is the balanced low digit (the low
        // byte of v read as int8) and byte 1 of word + 128 is the high digit, floor((v + 128) / 256).
        // Four fp/int instructions per element and four byte permutes per four elements.
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t b[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                b[i] = __float_as_uint(__fadd_rn(xv[4 * w + i] * f1 * f2, 12582912.0f));
                c[i] = b[i] + 128u;
            }
            lo[w] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
            hi[w] = __byte_perm(__byte_perm(c[0], c[1], 0x0051), __byte_perm(c[2], c[3], 0x0051), 0x5410);
        }
        o[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        o[NP - 1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        return;
    }
    constexpr int HALF = 1 << (DIGIT_BITS - 1), MASK = (1 << DIGIT_BITS) - 1;
    uint32_t d[NP][4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int p = 0; p < NP; ++p) d[p][w] = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            int v = rint_small(xv[4 * w + b] * f1 * f2);
#pragma unroll
            for (int p = 0; p < NP - 1; ++p) {
                const int dp = ((v + HALF) & MASK) - HALF;
                d[p][w] |= (uint32_t)(dp & 0xff) << (8 * b);
                v = (v - dp) >> DIGIT_BITS;
            }
            d[NP - 1][w] |= (uint32_t)(v & 0xff) << (8 * b);
        }
    }
#pragma unroll
    for (int p = 0; p < NP; ++p) o[p] = make_uint4(d[p][0], d[p][1], d[p][2], d[p][3]);
}

// One stage (RW weight rows in shared memory at `st`) against the digit planes `xs`; the warp's
// lanes split K.  Writes rows [0, rows) of the stage to y.
// A result goes to y in this rank's memory and, for a column shard (PEER), to the same place in
// every other rank's window: plain stores through the peer mappings.
template <bool PEER>
__device__ __forceinline__ void store_result(float *p, float val, const PeerSet &ps) {
    *p = val;
    if (PEER) {
#pragma unroll
        for (int q = 0; q < SHARD_MAX_RANKS; ++q)
            if (q < ps.world && q != ps.rank)
                *reinterpret_cast<float *>(reinterpret_cast<char *>(p) + ps.delta[q]) = val;
    }
}

template <int MT, int RW, bool PEER>
__device__ __forceinline__ void consume_stage(const StreamLayer &L, const uint8_t *st,
                                              const uint4 *xs, int kpad, int rows, int jl0,
                                              int row0, const LayerConsts *lc, const float *scale_s,
                                              const float *bias_s, bool staged, int lane,
                                              uint32_t empty_bar, const PeerSet &ps
#ifdef NNE_TRACE
                                              , unsigned long long *tr
#endif
                                              ) {
    const int k = L.k;
    int acc[RW][MT][NP];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int d = 0; d < NP; ++d) acc[r][m][d] = 0;
#pragma unroll 2
    for (int c = lane; c < kpad; c += 32) {
        uint4 xd[MT][NP];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int d = 0; d < NP; ++d) xd[m][d] = xs[((size_t)m * NP + d) * kpad + c];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            // chunks past the row's end read the next row (or the slot's slack) and meet zero
            // digits; rows past `rows` hold stale bytes and are never written out
            const uint4 wv = *reinterpret_cast<const uint4 *>(st + (size_t)r * k + (size_t)c * 16);
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int d = 0; d < NP; ++d) {
                    int a = acc[r][m][d];
                    a = __dp4a((int)wv.x, (int)xd[m][d].x, a);
                    a = __dp4a((int)wv.y, (int)xd[m][d].y, a);
                    a = __dp4a((int)wv.z, (int)xd[m][d].z, a);
                    a = __dp4a((int)wv.w, (int)xd[m][d].w, a);
                    acc[r][m][d] = a;
                }
        }
    }
#ifdef NNE_TRACE
    if (tr && lane == 0) tr[0] = globaltimer_ns();
#endif
    // The slot's bytes have been consumed: hand it back to the producer.  Lane 31 arrives, a lane
    // that never stores results: the arrive is a release, and a release issued by a lane whose
    // earlier stores went to a peer GPU would wait for their acknowledgement over NVLink.
    __syncwarp();
    if (lane == 31) mbar_arrive(empty_bar);
    // warp totals (exact integers), then lane r*MT+m finishes output (r, m)
    double mine = 0.0;
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            double tot = 0.0;
#pragma unroll
            for (int d = NP - 1; d >= 0; --d)
                tot = tot * (double)(1 << DIGIT_BITS) + (double)__reduce_add_sync(0xffffffffu, acc[r][m][d]);
            if (lane == r * MT + m) mine = tot;
        }
    if (lane < rows * MT) {
        const int r = lane / MT, m = lane % MT;
        const int jl = jl0 + r;
        const float dot = (float)(mine * (double)lc->unscale[m][0] * (double)lc->unscale[m][1]);
        const float sc = staged ? scale_s[jl] : __ldg(L.scales + row0 + jl);
        float val = __fmul_rn(dot, sc);
        if (L.bias) val = __fadd_rn(val, staged ? bias_s[jl] : __ldg(L.bias + row0 + jl));
        const float *residual = lc->residual;  // read here: a prefetch before the loop cost the loop 1 %
        if (residual) val = __fadd_rn(val, residual[(size_t)m * L.ldy + row0 + jl]);
        store_result<PEER>(L.y + (size_t)m * L.ldy + row0 + jl, val, ps);
    }
}

// fp32 loop for activations holding Inf/NaN: exact int8 -> f32, FMA accumulation, so that Inf
// and NaN propagate as IEEE arithmetic prescribes.  Not a fast path.
template <int MT, bool PEER>
__device__ __noinline__ void consume_stage_fp32(const StreamLayer &L, const uint8_t *st, int rw,
                                                int rows, int jl0, int row0, int lane,
                                                uint32_t empty_bar, const PeerSet &ps, const float *rrms) {
    const int k = L.k, chunks = k >> 4;
    for (int r = 0; r < rw; ++r) {
        float facc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) facc[m] = 0.0f;
        if (r < rows) {
            for (int c = lane; c < chunks; c += 32) {
                const uint4 wq = *reinterpret_cast<const uint4 *>(st + (size_t)r * k + (size_t)c * 16);
                float wf[16];
                cvt_i8x4(wq.x, wf + 0);
                cvt_i8x4(wq.y, wf + 4);
                cvt_i8x4(wq.z, wf + 8);
                cvt_i8x4(wq.w, wf + 12);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float *xr = L.x + (size_t)m * k + (size_t)c * 16;
#pragma unroll
                    for (int v = 0; v < 16; ++v)
                        facc[m] = fmaf(input_value(L, xr[v], m, (size_t)c * 16 + v, rrms[m]), wf[v], facc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float t = facc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0 && r < rows) {
                const int j = row0 + jl0 + r;
                float val = __fmul_rn(t, L.scales[j]);
                if (L.bias) val = __fadd_rn(val, L.bias[j]);
                if (L.residual) val = __fadd_rn(val, L.residual[(size_t)m * L.ldy + j]);
                store_result<PEER>(L.y + (size_t)m * L.ldy + j, val, ps);
            }
        }
    }
    __syncwarp();
    if (lane == 31) mbar_arrive(empty_bar);
}

// Four consecutive elements of row m of x', starting at column col (a multiple of 4), from the raw
// x values: the auxiliary operand (gamma or x2) comes in one 16-byte load.  Both are 16-byte aligned
// (checked when the plan is built).
__device__ __forceinline__ float4 input_value4(const StreamLayer &L, float4 t, int m, size_t col, float rrms) {
    if (L.gamma) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(L.gamma + col));
        t.x = __fmul_rn(__fmul_rn(t.x, rrms), g.x);
        t.y = __fmul_rn(__fmul_rn(t.y, rrms), g.y);
        t.z = __fmul_rn(__fmul_rn(t.z, rrms), g.z);
        t.w = __fmul_rn(__fmul_rn(t.w, rrms), g.w);
    } else if (L.x2) {
        const float4 u = *reinterpret_cast<const float4 *>(L.x2 + (size_t)m * L.k + col);
        t.x = __fmul_rn(__fdiv_rn(t.x, __fadd_rn(1.0f, expf(-t.x))), u.x);
        t.y = __fmul_rn(__fdiv_rn(t.y, __fadd_rn(1.0f, expf(-t.y))), u.y);
        t.z = __fmul_rn(__fdiv_rn(t.z, __fadd_rn(1.0f, expf(-t.z))), u.z);
        t.w = __fmul_rn(__fdiv_rn(t.w, __fadd_rn(1.0f, expf(-t.w))), u.w);
    }
    return t;
}

// Prep-warp passes over a layer's activations.  XF = the layer has an input transform; the plain
// case is kept free of it (a test per element in these loops showed up as 4 % of a 12-layer launch).
// Pass 1: max |x'| per row and the Inf/NaN flag.
template <int MT, bool XF>
__device__ __forceinline__ void prep_scan(const StreamLayer &L, int ptid, int chunks, uint64_t pol_keep,
                                          const float (&rr)[MT], float (&mx)[MT], int &bad) {
    const int k = L.k;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        mx[m] = 0.0f;
        for (int c = ptid; c < chunks; c += PREP_THREADS) {
            const float4 *p4 = reinterpret_cast<const float4 *>(L.x + (size_t)m * k + (size_t)c * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                float4 t4 = ld_f4_hint(p4 + v, pol_keep);
                if (XF) t4 = input_value4(L, t4, m, (size_t)c * 16 + 4 * v, rr[m]);
                const float a0 = fabsf(t4.x), a1 = fabsf(t4.y), a2 = fabsf(t4.z), a3 = fabsf(t4.w);
                bad |= !(a0 <= 3.402823466e38f) | !(a1 <= 3.402823466e38f) |
                       !(a2 <= 3.402823466e38f) | !(a3 <= 3.402823466e38f);
                mx[m] = fmaxf(fmaxf(mx[m], fmaxf(a0, a1)), fmaxf(a2, a3));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[m] = fmaxf(mx[m], __shfl_xor_sync(0xffffffffu, mx[m], o));
    }
}
// Pass 2, one row: digits of rint(x' * f1 * f2) into the row's digit planes (x is re-read; it is in
// L1 now).
template <bool XF>
__device__ __forceinline__ void prep_digits(const StreamLayer &L, int m, int ptid, int chunks, int kpad,
                                            float f1, float f2, float rr, uint4 *plane) {
    const int k = L.k;
    for (int c = ptid; c < kpad; c += PREP_THREADS) {
        uint4 o[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) o[p] = make_uint4(0u, 0u, 0u, 0u);
        if (c < chunks) {
            const float4 *p4 = reinterpret_cast<const float4 *>(L.x + (size_t)m * k + (size_t)c * 16);
            float xv[16];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                float4 t4 = p4[v];
                if (XF) t4 = input_value4(L, t4, m, (size_t)c * 16 + 4 * v, rr);
                xv[4 * v + 0] = t4.x;
                xv[4 * v + 1] = t4.y;
                xv[4 * v + 2] = t4.z;
                xv[4 * v + 3] = t4.w;
            }
            chunk_digits(xv, f1, f2, o);
        }
#pragma unroll
        for (int p = 0; p < NP; ++p) plane[p * kpad + c] = o[p];
    }
}

// One activation row (with or without an input transform) held in registers between the passes:
// thread ptid keeps chunks ptid, ptid + PREP_THREADS, ... (at most XF_CACHE_CHUNKS of them, i.e.
// k <= 14336; longer rows and two-row launches take the multi-pass code).  x and the auxiliary
// operand are read from global memory once, all loads of a chunk issued before anything is computed
// on them, and silu - an exp and a divide per element, in every CTA - is evaluated once instead of
// once per pass.
constexpr int XF_CACHE_CHUNKS = 4;
__device__ __forceinline__ void xf_load(const StreamLayer &L, int ptid, int chunks, uint64_t pol_keep,
                                        float (&xc)[XF_CACHE_CHUNKS][16]) {
#pragma unroll
    for (int u = 0; u < XF_CACHE_CHUNKS; ++u) {
        const int c = ptid + u * PREP_THREADS;
        float4 t[4], a[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) t[v] = a[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < chunks) {
            const float4 *p4 = reinterpret_cast<const float4 *>(L.x + (size_t)c * 16);
#pragma unroll
            for (int v = 0; v < 4; ++v) t[v] = ld_f4_hint(p4 + v, pol_keep);
            if (L.x2) {
                const float4 *q4 = reinterpret_cast<const float4 *>(L.x2 + (size_t)c * 16);
#pragma unroll
                for (int v = 0; v < 4; ++v) a[v] = ld_f4_hint(q4 + v, pol_keep);
            }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (L.x2) {
                // silu with the fast exponential and divide (each within about 2 ulp): every CTA
                // evaluates the whole row, and the result goes onto the 16-bit grid right after
                t[v].x = __fmul_rn(__fdividef(t[v].x, 1.0f + __expf(-t[v].x)), a[v].x);
                t[v].y = __fmul_rn(__fdividef(t[v].y, 1.0f + __expf(-t[v].y)), a[v].y);
                t[v].z = __fmul_rn(__fdividef(t[v].z, 1.0f + __expf(-t[v].z)), a[v].z);
                t[v].w = __fmul_rn(__fdividef(t[v].w, 1.0f + __expf(-t[v].w)), a[v].w);
            }
            xc[u][4 * v + 0] = t[v].x;
            xc[u][4 * v + 1] = t[v].y;
            xc[u][4 * v + 2] = t[v].z;
            xc[u][4 * v + 3] = t[v].w;
        }
    }
}
__device__ __forceinline__ void xf_apply_gamma(const StreamLayer &L, int ptid, int chunks, float rrms,
                                               float (&xc)[XF_CACHE_CHUNKS][16]) {
#pragma unroll
    for (int u = 0; u < XF_CACHE_CHUNKS; ++u) {
        const int c = ptid + u * PREP_THREADS;
        if (c < chunks) {
            const float4 *g4 = reinterpret_cast<const float4 *>(L.gamma + (size_t)c * 16);
            float4 g[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) g[v] = __ldg(g4 + v);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                xc[u][4 * v + 0] = __fmul_rn(__fmul_rn(xc[u][4 * v + 0], rrms), g[v].x);
                xc[u][4 * v + 1] = __fmul_rn(__fmul_rn(xc[u][4 * v + 1], rrms), g[v].y);
                xc[u][4 * v + 2] = __fmul_rn(__fmul_rn(xc[u][4 * v + 2], rrms), g[v].z);
                xc[u][4 * v + 3] = __fmul_rn(__fmul_rn(xc[u][4 * v + 3], rrms), g[v].w);
            }
        }
    }
}

#ifdef NNE_TRACE
#define NNE_TR_ARG , ((batch.trace && blockIdx.x == 0 && warp == 0 && g / active < 48) ? batch.trace + 800 + (g / active) : nullptr)
#else
#define NNE_TR_ARG
#endif
#ifdef NNE_TRACE
// Debug builds only: time stamps of the first rendezvous of CTAs 0, 73 and 147, behind the counter.
#define NNE_TR(j, e)                                                                                   \
    do {                                                                                               \
        const int c_ = blockIdx.x == 0 ? 0 : blockIdx.x == 73 ? 1 : blockIdx.x == 147 ? 2 : -1;        \
        if (batch.trace && c_ >= 0 && (j) < 16) batch.trace[8 + (c_ * 16 + (j)) * 8 + (e)] = globaltimer_ns(); \
    } while (0)
#else
#define NNE_TR(j, e) do { } while (0)
#endif

// Grid-wide rendezvous between two layers of one launch, the second of which reads (or overwrites)
// what the first wrote.  Called by ONE thread per CTA, after every math warp of the CTA has arrived
// at `gsync` behind its last store.  Arrival is an atomic add with release semantics on a 64-bit
// counter that only ever grows; the generation is read off the value the add returns (every CTA
// arrives exactly once per rendezvous, so the counter passes a multiple of the grid size exactly
// when all have arrived), which keeps a replayed launch - a CUDA graph - correct without any
// per-launch argument.  The wait is an acquire load, bounded like every other wait.  All CTAs of the
// grid are resident (cooperative launch, one CTA per SM), so a waiting CTA never keeps the ones it
// waits for off the GPU.
__device__ __forceinline__ bool grid_rendezvous(unsigned long long *counter, volatile int *abort_flag,
                                                int *err) {
    unsigned long long old;
    asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;" : "=l"(old) : "l"(counter) : "memory");
    const unsigned long long g = gridDim.x;
    const unsigned long long target = (old / g + 1ull) * g;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        unsigned long long now;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(now) : "l"(counter) : "memory");
        if (now >= target) return true;
        if ((++spins & 0x3f) == 0) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                *reinterpret_cast<volatile int *>(err) = 0x100 + 0x18;
                __threadfence_system();
                return false;
            }
        }
    }
}

// MT activation rows per layer (1..2).  `num_slots` ring slots of `slot_bytes`; `kpad_max` = 16-byte
// chunks per activation row rounded up to 32 for the widest layer; `sb_rows` = capacity of the
// per-layer scale/bias staging (0: read them from global memory).
//
// Warp roles: warps 0..7 math (warp w owns ring slot w), warps 8..14 prepare the NEXT layer's
// activations (digit planes, staged scales) into the other of `num_bufs` buffers while the math
// warps work on the current layer, the last warp is the producer.
//
// PEER (column shards): every result is also stored into the other ranks' windows.  The kernel does
// not announce its own results - a fence that waits for the NVLink acknowledgements, in every CTA,
// showed up as 8 us on a 72 us launch; it announces the PREVIOUS run of its rank instead, which is
// complete by the time this grid's dependency is released, from a lane that has nothing else to
// do.  Nor does it wait for anybody: a waiting CTA would hold its SM, and the completion of the
// grid, until the slowest rank is through.  The exchange's wait kernel (shard.cu) announces what is
// still unannounced and waits for the arrivals, on behalf of whoever consumes the gathered result.
template <int MT, bool PEER, bool CHAIN>
__device__ __forceinline__ void stream_body(const StreamBatch &batch, int num_slots, int slot_bytes,
                                            int kpad_max, int sb_rows, int num_bufs, int *err,
                                            const PeerSet &ps) {
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: ring [num_slots][slot_bytes] | xs [num_bufs][MT][3][kpad_max] uint4 | RingBars |
    //         scale_s[num_bufs][sb_rows] | bias_s[num_bufs][sb_rows]
    uint8_t *ring = smem;
    uint4 *xs_all = reinterpret_cast<uint4 *>(smem + (size_t)num_slots * slot_bytes);
    const size_t xs_buf = (size_t)MT * NP * kpad_max;
    RingBars *bars = reinterpret_cast<RingBars *>(xs_all + num_bufs * xs_buf);
    float *scale_all = reinterpret_cast<float *>(bars + 1);
    float *bias_all = scale_all + num_bufs * sb_rows;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    volatile int *abort_flag = &bars->abort_flag;
    const StreamLayer *layers = batch.dev ? batch.dev : batch.inl;

    if (tid == 0) {
        for (int s = 0; s < num_slots; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);  // exactly one warp consumes a slot
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->xs_full[b]), PREP_WARPS);
            mbar_init(smem_u32(&bars->xs_empty[b]), MATH_WARPS);
        }
        mbar_init(smem_u32(&bars->gsync), MATH_WARPS);
        bars->abort_flag = 0;
        bars->gsync_parity = 0;
#ifdef NNE_TRACE
        bars->tr_j = bars->tr_jm = 0;
#endif
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream begin its own weight prefetch as soon as SMs free up.
    grid_launch_dependents();

    if (warp == MATH_WARPS + PREP_WARPS) {
        // ---------------- producer: weights only, may run ahead of the previous kernel ----------
        if (lane == 0) {
            const uint64_t pol_stream = batch.reuse ? l2_policy_evict_normal() : l2_policy_evict_first();
            const uint64_t pol_pf = l2_policy_evict_normal();
            int slot = 0;
            uint32_t phase = 0;
            bool ok = true;
            // A second cursor runs ahead of the ring through the same sequence of stages and asks
            // for them to be brought into L2 (batch.pf_bytes beyond what the ring holds).  The
            // ring's copy of a stage then finds it there, which shortens the time a slot spends in
            // flight - and the ring, which shared memory limits to about 100-130 KB, is what bounds
            // the bytes this SM can have on their way.  No extra HBM traffic.
            // All per-stage state is kept incremental: this loop is one thread's chain of dependent
            // instructions, and its length per stage (0.3 us) is not far below the time HBM needs
            // to deliver a stage to one SM.
            int p_li = -1, p_left = 0, p_rw = 1, p_k = 0;  // look-ahead cursor: layer, rows left in it
            const int8_t *p_src = nullptr;
            int ahead = 0;  // bytes asked for and not yet copied into the ring
#ifdef NNE_TRACE
            int tr_g = 0;
#endif
            for (int li = 0; li < batch.count && ok; ++li) {
                const int8_t *src;
                int left, rw, k;
                {
                    int row0, cnt;
                    cta_rows(layers[li].n, (int)blockIdx.x, (int)gridDim.x, row0, cnt);
                    k = layers[li].k;
                    rw = layers[li].rw;
                    src = layers[li].q + (size_t)row0 * k;
                    left = cnt;
                }
                const uint32_t stage_bytes = (uint32_t)rw * (uint32_t)k;
                while (left > 0) {
                    while (ahead < batch.pf_bytes) {
                        if (p_left <= 0) {
                            if (p_li + 1 >= batch.count) break;
                            ++p_li;
                            int row0;
                            cta_rows(layers[p_li].n, (int)blockIdx.x, (int)gridDim.x, row0, p_left);
                            p_k = layers[p_li].k;
                            p_rw = layers[p_li].rw;
                            p_src = layers[p_li].q + (size_t)row0 * p_k;
                            continue;
                        }
                        const int pb = min(p_rw, p_left) * p_k;
                        bulk_prefetch_l2(p_src, (uint32_t)pb, pol_pf);
                        p_src += pb;
                        p_left -= p_rw;
                        ahead += pb;
                    }
                    ok = mbar_wait(smem_u32(&bars->empty[slot]), phase ^ 1, abort_flag, err, 0x11);
                    if (!ok) break;
                    const uint32_t bytes = left >= rw ? stage_bytes : (uint32_t)left * (uint32_t)k;
                    const uint32_t full = smem_u32(&bars->full[slot]);
                    mbar_arrive_expect_tx(full, bytes);
                    bulk_load_1d_hint(smem_u32(ring + (size_t)slot * slot_bytes), src, bytes, full, pol_stream);
                    src += bytes;
                    left -= rw;
                    ahead -= (int)bytes;
                    if (++slot == num_slots) { slot = 0; phase ^= 1; }
#ifdef NNE_TRACE
                    if (batch.trace && blockIdx.x == 0 && tr_g < 96) batch.trace[512 + tr_g] = globaltimer_ns();
                    ++tr_g;
#endif
                }
            }
            if (!ok) {
                // Gave up: let copies that are still in flight land before the CTA exits.
                for (int s = 0; s < num_slots; ++s) {
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

    if (warp >= MATH_WARPS) {
        // ---------------- prep warps: activations of layer li into buffer li & 1 ----------------
        const int ptid = tid - MATH_WARPS * 32, pwarp = warp - MATH_WARPS;
        const uint64_t pol_keep = l2_policy_evict_last();  // activations and scales stay in L2
        for (int li = 0; li < batch.count; ++li) {
            const StreamLayer L = layers[li];
            const int buf = li % num_bufs;
            const uint32_t use = (uint32_t)(li / num_bufs);
            const int k = L.k, chunks = k >> 4;
            const int kpad = (chunks + 31) & ~31;
            int row0, cnt;
            cta_rows(L.n, (int)blockIdx.x, (int)gridDim.x, row0, cnt);
            const bool staged = sb_rows >= cnt && sb_rows > 0;
            uint4 *xs = xs_all + buf * xs_buf;
            float *scale_s = scale_all + buf * sb_rows, *bias_s = bias_all + buf * sb_rows;

            if (CHAIN && L.same_input && num_bufs == 2 && li > 0) {
                // The layer multiplies the very activations the layer before it did (q/k/v, gate/up):
                // copy that layer's digit planes from the other buffer instead of reading, transforming
                // and digitising x again (0.3 us instead of 2-3: a group of such layers is otherwise
                // bound by this preparation, not by its weights).
                (void)mbar_wait(smem_u32(&bars->xs_empty[buf]), (use & 1u) ^ 1u, abort_flag, err, 0x15);
                named_bar_sync(1, PREP_THREADS);  // every prep thread has written its part of the other buffer
                const uint4 *from = xs_all + (buf ^ 1) * xs_buf;
                for (int i = ptid; i < MT * NP * kpad; i += PREP_THREADS) xs[i] = from[i];
                if (staged) {
                    for (int i = ptid; i < cnt; i += PREP_THREADS) {
                        scale_s[i] = ldg_f1_hint(L.scales + row0 + i, pol_keep);
                        bias_s[i] = L.bias ? ldg_f1_hint(L.bias + row0 + i, pol_keep) : 0.0f;
                    }
                }
                if (ptid == 0) {
                    bars->bad[buf] = bars->bad[buf ^ 1];
                    bars->lc[buf] = bars->lc[buf ^ 1];
                    bars->lc[buf].residual = L.residual;
#pragma unroll
                    for (int m = 0; m < MT; ++m) bars->rrms[buf][m] = bars->rrms[buf ^ 1][m];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->xs_full[buf]));
                continue;
            }

            // Scales and bias are layer constants: fetch this CTA's rows first.  Unconditional
            // loads from clamped addresses, masked afterwards, so that no predicated register
            // write has to wait for a load that is still in flight.
            float sc_pre[4], bs_pre[4];  // rows ptid, ptid + PREP_THREADS, ... of this CTA (at most 4 per thread)
            if (staged) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = min(ptid + u * PREP_THREADS, cnt - 1);
                    sc_pre[u] = ldg_f1_hint(L.scales + row0 + i, pol_keep);
                    bs_pre[u] = L.bias ? ldg_f1_hint(L.bias + row0 + i, pol_keep) : 0.0f;
                }
            }
            if (li == 0) grid_dependency_wait();  // x may be the previous kernel's output
            if (CHAIN && L.sync) {
                // This layer reads (or overwrites) what earlier layers of the launch wrote: the math
                // warps of every CTA must have stored those results first.  The weight stream does
                // not stop meanwhile; the ring fills with this layer's rows.
                if (L.gamma) {
                    // gamma is a constant: have it on its way while the grid meets
                    for (int c = ptid; c < chunks; c += PREP_THREADS)
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(L.gamma + (size_t)c * 16));
                }
                if (ptid == 0) {
                    const uint32_t par = bars->gsync_parity;  // kept in shared memory: registers are short here
                    bars->gsync_parity = par ^ 1u;
                    (void)mbar_wait(smem_u32(&bars->gsync), par, abort_flag, err, 0x17);
                    NNE_TR(bars->tr_j, 0);
                    (void)grid_rendezvous(batch.gsync, abort_flag, err);
                    NNE_TR(bars->tr_j, 1);
                }
                named_bar_sync(1, PREP_THREADS);
            }

            const bool xform = L.gamma != nullptr || L.x2 != nullptr;
            // one row of at most 14336 elements: x' stays in this warp group's registers between the
            // passes - one read of x, every load in flight at once (with or without a transform)
            const bool cached = MT == 1 && chunks <= XF_CACHE_CHUNKS * PREP_THREADS;
            float xc[XF_CACHE_CHUNKS][16];
            float rr[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) rr[m] = 1.0f;
            float mx[MT];
            int bad = 0;
            if (cached) {
                xf_load(L, ptid, chunks, pol_keep, xc);
                if (L.gamma) {
                    float acc = 0.0f;
#pragma unroll
                    for (int u = 0; u < XF_CACHE_CHUNKS; ++u)
#pragma unroll
                        for (int v = 0; v < 16; ++v) acc = fmaf(xc[u][v], xc[u][v], acc);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (lane == 0) bars->sumsq[li & 1][pwarp][0] = acc;
                    named_bar_sync(1, PREP_THREADS);
                    float tot = 0.0f;
                    for (int w = 0; w < PREP_WARPS; ++w) tot += bars->sumsq[li & 1][w][0];
                    rr[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)k), L.eps)));
                    xf_apply_gamma(L, ptid, chunks, rr[0], xc);
                }
                float m0 = 0.0f;
#pragma unroll
                for (int u = 0; u < XF_CACHE_CHUNKS; ++u)
#pragma unroll
                    for (int v = 0; v < 16; ++v) {
                        const float a0 = fabsf(xc[u][v]);
                        bad |= !(a0 <= 3.402823466e38f);
                        m0 = fmaxf(m0, a0);
                    }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
                mx[0] = m0;
            } else {
                // pass 0 (RMSNorm input only): sum of squares per row -> rrms
                if (L.gamma) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float acc = 0.0f;
                        for (int c = ptid; c < chunks; c += PREP_THREADS) {
                            const float4 *p4 = reinterpret_cast<const float4 *>(L.x + (size_t)m * k + (size_t)c * 16);
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const float4 t4 = ld_f4_hint(p4 + v, pol_keep);
                                acc = fmaf(t4.x, t4.x, acc);
                                acc = fmaf(t4.y, t4.y, acc);
                                acc = fmaf(t4.z, t4.z, acc);
                                acc = fmaf(t4.w, t4.w, acc);
                            }
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                        if (lane == 0) bars->sumsq[li & 1][pwarp][m] = acc;
                    }
                    // sumsq alternates by layer parity, so the previous layer's readers are not disturbed
                    named_bar_sync(1, PREP_THREADS);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float tot = 0.0f;
                        for (int w = 0; w < PREP_WARPS; ++w) tot += bars->sumsq[li & 1][w][m];
                        rr[m] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)k), L.eps)));
                    }
                }
                // pass 1: max |x'| and the Inf/NaN flag per activation row
                if (xform)
                    prep_scan<MT, true>(L, ptid, chunks, pol_keep, rr, mx, bad);
                else
                    prep_scan<MT, false>(L, ptid, chunks, pol_keep, rr, mx, bad);
            }
            bad = __any_sync(0xffffffffu, bad);
#ifdef NNE_TRACE
            if (L.sync && ptid == 0) NNE_TR(bars->tr_j, 2);
#endif
            // The buffer (digits, scales, flags) may still be read by math warps working on layer
            // li - num_bufs: wait until all of them have released it.
            (void)mbar_wait(smem_u32(&bars->xs_empty[buf]), (use & 1u) ^ 1u, abort_flag, err, 0x15);
            named_bar_sync(1, PREP_THREADS);  // nobody still reads xmax/bad_warp of the previous layer
            if (lane == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) bars->xmax[pwarp][m] = mx[m];
                bars->bad_warp[pwarp] = bad;
            }
            if (staged) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = ptid + u * PREP_THREADS;
                    if (i < cnt) {
                        scale_s[i] = sc_pre[u];
                        bias_s[i] = bs_pre[u];
                    }
                }
            }
            named_bar_sync(1, PREP_THREADS);
            bad = 0;
            for (int w = 0; w < PREP_WARPS; ++w) bad |= bars->bad_warp[w];
            if (ptid == 0) {
                bars->bad[buf] = bad;
                bars->lc[buf].residual = L.residual;
#pragma unroll
                for (int m = 0; m < MT; ++m) bars->rrms[buf][m] = rr[m];
            }

            if (!bad) {
                // pass 2: digits of rint(x * 2^e) into shared memory (x is re-read; it is in L1 now)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float big = 0.0f;
                    for (int w = 0; w < PREP_WARPS; ++w) big = fmaxf(big, bars->xmax[w][m]);
                    const int e = act_grid_exponent(big);
                    const int e1 = e >> 1, e2 = e - e1;                     // 2^e = 2^e1 * 2^e2, both finite
                    const float f1 = pow2f(e1), f2 = pow2f(e2);
                    if (ptid == 0) {
                        bars->lc[buf].unscale[m][0] = pow2f(-e1);
                        bars->lc[buf].unscale[m][1] = pow2f(-e2);
                    }
                    uint4 *plane = xs + (size_t)m * NP * kpad;
                    if (cached) {
#pragma unroll
                        for (int u = 0; u < XF_CACHE_CHUNKS; ++u) {
                            const int c = ptid + u * PREP_THREADS;
                            if (c < kpad) {  // chunks past the row's end hold zeros
                                uint4 o[NP];
                                chunk_digits(xc[u], f1, f2, o);
#pragma unroll
                                for (int p = 0; p < NP; ++p) plane[p * kpad + c] = o[p];
                            }
                        }
                    } else if (xform) {
                        prep_digits<true>(L, m, ptid, chunks, kpad, f1, f2, rr[m], plane);
                    } else {
                        prep_digits<false>(L, m, ptid, chunks, kpad, f1, f2, rr[m], plane);
                    }
                }
            }
            // publish the buffer to the math warps
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->xs_full[buf]));
#ifdef NNE_TRACE
            if (L.sync && ptid == 0) {
                NNE_TR(bars->tr_j, 3);
                bars->tr_j = bars->tr_j + 1;
            }
#endif
        }
        return;
    }

    // ---------------- math warps ----------------
    if (PEER && blockIdx.x == 0 && warp == MATH_WARPS - 1 && ps.target > 0x100000000ull) {
        // A warp that has nothing to do until the first layer's activations are prepared announces
        // this rank's PREVIOUS run to the other ranks: once the grids before this one have
        // completed, that run's stores are performed.  (This run is announced by the next one, or
        // by the exchange's wait kernel.)
        grid_dependency_wait();
        if (lane == 0) shard_publish(ps, ps.target - 0x100000000ull);
        __syncwarp();
    }
    int g_base = 0;  // global stage index of the current layer's first stage (in this CTA)
    for (int li = 0; li < batch.count; ++li) {
        const StreamLayer L = layers[li];
        const int buf = li % num_bufs;
        const int chunks = L.k >> 4;
        const int kpad = (chunks + 31) & ~31;
        int row0, cnt;
        cta_rows(L.n, (int)blockIdx.x, (int)gridDim.x, row0, cnt);
        const int nst = (cnt + L.rw - 1) / L.rw;
        const bool staged = sb_rows >= cnt && sb_rows > 0;
        const uint4 *xs = xs_all + buf * xs_buf;
        const float *scale_s = scale_all + buf * sb_rows, *bias_s = bias_all + buf * sb_rows;

        // the layer's activations are prepared
        (void)mbar_wait(smem_u32(&bars->xs_full[buf]), (uint32_t)(li / num_bufs) & 1u, abort_flag, err,
                        0x16);
        const int bad = bars->bad[buf];
        const LayerConsts *lc = &bars->lc[buf];
#ifdef NNE_TRACE
        if (L.sync && warp == 0 && lane == 0) NNE_TR(bars->tr_jm, 4);
#endif

        // Warp w takes the global stages g with g % num_slots == w.  One slot, one warp: a warp
        // never waits on a barrier that is more than one phase behind it, which is what the
        // parity wait needs to be unambiguous.
        if (warp < num_slots) {
#ifdef NNE_TRACE
            const int active = num_slots;
#endif
            const int slot = warp;
            int g = g_base + ((warp - g_base % num_slots) + num_slots) % num_slots;
            for (; g < g_base + nst; g += num_slots) {
                const int s = g - g_base;
                const uint32_t phase = (uint32_t)(g / num_slots) & 1u;
                // If the wait runs out the error word is set and every later wait returns at once.
                (void)mbar_wait(smem_u32(&bars->full[slot]), phase, abort_flag, err, 0x12);
#ifdef NNE_TRACE
                if (batch.trace && blockIdx.x == 0 && warp == 0 && lane == 0 && g / active < 48)
                    batch.trace[640 + (g / active) * 2] = globaltimer_ns();
#endif
                const int rows = min(L.rw, cnt - s * L.rw);
                const uint8_t *st = ring + (size_t)slot * slot_bytes;
                const uint32_t empty_bar = smem_u32(&bars->empty[slot]);
                if (bad) {
                    consume_stage_fp32<MT, PEER>(L, st, L.rw, rows, s * L.rw, row0, lane, empty_bar, ps,
                                                 &bars->rrms[buf][0]);
                } else if (L.rw == 4) {
                    consume_stage<MT, 4, PEER>(L, st, xs, kpad, rows, s * 4, row0, lc, scale_s, bias_s,
                                               staged, lane, empty_bar, ps NNE_TR_ARG);
                } else if (L.rw == 2) {
                    consume_stage<MT, 2, PEER>(L, st, xs, kpad, rows, s * 2, row0, lc, scale_s, bias_s,
                                               staged, lane, empty_bar, ps NNE_TR_ARG);
                } else {
                    consume_stage<MT, 1, PEER>(L, st, xs, kpad, rows, s, row0, lc, scale_s, bias_s,
                                               staged, lane, empty_bar, ps NNE_TR_ARG);
                }
#ifdef NNE_TRACE
                __syncwarp();
                if (batch.trace && blockIdx.x == 0 && warp == 0 && lane == 0 && g / active < 48)
                    batch.trace[640 + (g / active) * 2 + 1] = globaltimer_ns();
#endif
            }
        }
        g_base += nst;
        // this warp is done with the layer's activation buffer - and, where the next layer is chained
        // to the ones before it, with its stores (the arrive is a release behind the warp barrier)
        __syncwarp();
#ifdef NNE_TRACE
        if (warp == 0 && lane == 0) {
            if (L.sync) {
                NNE_TR(bars->tr_jm, 5);
                bars->tr_jm = bars->tr_jm + 1;
            }
            if (li + 1 < batch.count && layers[li + 1].sync) NNE_TR(bars->tr_jm, 6);
        }
#endif
        if (lane == 31) {
            mbar_arrive(smem_u32(&bars->xs_empty[buf]));
            if (CHAIN && li + 1 < batch.count && layers[li + 1].sync) mbar_arrive(smem_u32(&bars->gsync));
        }
    }
}

// The two entry points.  Sixteen warps of 128 registers fill an SM's register file; the column-shard
// variant is held to 120 so that a one-warp kernel of the exchange (the arrival wait, on a second
// stream) finds room beside a resident CTA instead of waiting for the grid to end.
template <int MT>
__global__ void __launch_bounds__(THREADS, 1)
qgemv_stream_kernel(const StreamBatch batch, int num_slots, int slot_bytes, int kpad_max, int sb_rows,
                    int num_bufs, int *err) {
    const PeerSet none;
    stream_body<MT, false, false>(batch, num_slots, slot_bytes, kpad_max, sb_rows, num_bufs, err, none);
}
// The instance for lists whose layers depend on or share the input of their predecessors (`sync`,
// `same_input`).  Separate, because those paths cost the plain instance three spilled registers and
// 2 % of its speed when they are compiled into it.
template <int MT>
__global__ void __launch_bounds__(THREADS, 1)
qgemv_stream_chain_kernel(const StreamBatch batch, int num_slots, int slot_bytes, int kpad_max, int sb_rows,
                          int num_bufs, int *err) {
    const PeerSet none;
    stream_body<MT, false, true>(batch, num_slots, slot_bytes, kpad_max, sb_rows, num_bufs, err, none);
}
template <int MT>
__global__ void __maxnreg__(120)
qgemv_stream_peer_kernel(const StreamBatch batch, int num_slots, int slot_bytes, int kpad_max, int sb_rows,
                         int num_bufs, int *err, const PeerSet ps) {
    stream_body<MT, true, false>(batch, num_slots, slot_bytes, kpad_max, sb_rows, num_bufs, err, ps);
}

template <int MT, bool PEER>
int launch_stream_mt(nne_ctx *ctx, const StreamBatch &batch, int slots, int slot_bytes, int kpad,
                     int sb_rows, int bufs, size_t smem, int grid, const PeerSet &ps, cudaStream_t s) {
    const bool chain = batch.chain && !PEER;  // some layer is tied to its predecessors
    if (PEER)
        NNE_TRY(ensure_dynamic_smem(ctx->device, qgemv_stream_peer_kernel<MT>, smem));
    else if (chain)
        NNE_TRY(ensure_dynamic_smem(ctx->device, qgemv_stream_chain_kernel<MT>, smem));
    else
        NNE_TRY(ensure_dynamic_smem(ctx->device, qgemv_stream_kernel<MT>, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    if (batch.gsync) {
        // chained layers rendezvous inside the launch: the whole grid has to be resident
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.numAttrs = 1;
    } else {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
    }
    cudaError_t e = PEER ? cudaLaunchKernelEx(&cfg, qgemv_stream_peer_kernel<MT>, batch, slots, slot_bytes,
                                              kpad, sb_rows, bufs, ctx->err_word, ps)
                         : chain ? cudaLaunchKernelEx(&cfg, qgemv_stream_chain_kernel<MT>, batch, slots, slot_bytes,
                                                      kpad, sb_rows, bufs, ctx->err_word)
                                 : cudaLaunchKernelEx(&cfg, qgemv_stream_kernel<MT>, batch, slots, slot_bytes, kpad,
                                                      sb_rows, bufs, ctx->err_word);
    count_launch();
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "streaming kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace

// Rows per stage for a layer: the largest of {4, 2, 1} that keeps a stage within 24 KB.  (Smaller
// stages in more slots were measured and lose: issuing a copy costs the producer 0.15-0.3 us whatever
// its size, and a math warp about 0.6 us per stage beside the 0.05 us per KB.)
// NNE_STREAM_STAGE_KB overrides the bound.
int stream_rows_per_stage(size_t k) {
    static const size_t cap = [] {
        const char *e = getenv("NNE_STREAM_STAGE_KB");
        const int kb = e ? atoi(e) : 24;
        return (size_t)(kb < 1 ? 1 : kb) * 1024;
    }();
    return (4 * k <= cap) ? 4 : (2 * k <= cap) ? 2 : 1;
}

// m = activation rows per layer (1..2); one layer's shape.
bool gemv_tma_supports(size_t n, size_t k, size_t m) {
    if (m < 1 || m > 2 || n == 0) return false;
    if (k % 16 != 0 || k < 256 || k > 32768) return false;
    if (n > 0x7fffffffu) return false;
    // one buffer of digit planes (48 bytes per 16 activations per row) + two slots must fit
    const size_t kpad = ((k >> 4) + 31) & ~(size_t)31;
    const size_t need = m * NP * kpad * 16 + 2 * ((size_t)stream_rows_per_stage(k) * k + 640) + 8192;
    return need <= 200 * 1024;
}

// Launches the streaming kernel over `count` layers (descriptors in host memory `host`; for more
// than STREAM_INLINE_LAYERS layers `dev` must hold the same descriptors in device memory).
int launch_stream_batch(nne_ctx *ctx, const StreamLayer *host, const StreamLayer *dev, int count,
                        size_t m, bool reuse, cudaStream_t s, const PeerSet *peers,
                        unsigned long long *gsync) {
    if (count <= 0) return NNE_OK;
    if (count > STREAM_INLINE_LAYERS && !dev)
        return fail(NNE_ERR_INVALID_ARGUMENT, "a batch of %d layers needs device descriptors", count);
    StreamBatch batch;
    batch.count = count;
    batch.reuse = reuse ? 1 : 0;
    batch.dev = count > STREAM_INLINE_LAYERS ? dev : nullptr;
    batch.gsync = nullptr;
    batch.pf_bytes = 0;
    batch.chain = 0;
    for (int i = 0; i < count; ++i) batch.chain |= (host[i].sync || host[i].same_input) ? 1 : 0;
#ifdef NNE_TRACE
    batch.trace = gsync;
#endif
    for (int i = 0; i < count; ++i)
        if (host[i].sync) {
            if (i == 0 || !gsync || (peers && peers->world > 1))
                return fail(NNE_ERR_INVALID_ARGUMENT, "layer %d: a chained layer needs an earlier one, a counter and no column shards", i);
            batch.gsync = gsync;
        }
    // L2 look-ahead of the weight stream per CTA: 192 KB for a list of layers, 64 KB for a single
    // layer (measured optima; beyond 256 KB per CTA the look-ahead of 148 CTAs starts to push itself
    // out of L2).  NNE_STREAM_LOOKAHEAD_KB overrides it, 0 switches it off.
    static const int lookahead_kb = [] {
        const char *e = getenv("NNE_STREAM_LOOKAHEAD_KB");
        return e ? atoi(e) : -1;
    }();
    batch.pf_bytes = lookahead_kb >= 0 ? lookahead_kb * 1024 : (count > 1 ? 192 : 64) * 1024;
    size_t kmax = 0, slot_payload = 0, nmax = 0, nmin = (size_t)-1;
    for (int i = 0; i < count; ++i) {
        if (i < STREAM_INLINE_LAYERS) batch.inl[i] = host[i];
        if (!gemv_tma_supports((size_t)host[i].n, (size_t)host[i].k, m))
            return fail(NNE_ERR_UNSUPPORTED, "layer %d (n=%d k=%d) is not a streaming shape", i,
                        host[i].n, host[i].k);
        kmax = kmax > (size_t)host[i].k ? kmax : (size_t)host[i].k;
        const size_t pay = (size_t)host[i].rw * host[i].k;
        slot_payload = slot_payload > pay ? slot_payload : pay;
        nmax = nmax > (size_t)host[i].n ? nmax : (size_t)host[i].n;
        nmin = nmin < (size_t)host[i].n ? nmin : (size_t)host[i].n;
    }
    const int kpad = (int)(((kmax >> 4) + 31) & ~(size_t)31);
    // a slot holds a stage plus slack for the padded chunk loop of its last row
    const int slot_bytes = (int)((slot_payload + 512 + 127) & ~(size_t)127);
    int grid = ctx->sm_count - ctx->reserved_sms;  // all CTAs resident at once: one wave, equal row ranges
    if (grid < 1) grid = 1;
    if ((size_t)grid > nmin) grid = (int)nmin;
    int sb_rows = (int)((nmax + grid - 1) / grid) + 1;
    if (sb_rows > 4 * PREP_THREADS) sb_rows = 0;  // the prep warps stage at most 4 rows per thread
    // two activation buffers (so the next layer is prepared while this one runs) when the batch has
    // more than one layer and they leave room for at least four ring slots, else one
    const size_t one_buf = m * NP * (size_t)kpad * 16 + 2 * (size_t)sb_rows * sizeof(float);
    const size_t budget = 220 * 1024;
    int bufs = count > 1 ? 2 : 1;
    if (bufs == 2 && 2 * one_buf + sizeof(RingBars) + 256 + 4 * (size_t)slot_bytes > budget) bufs = 1;
    const size_t fixed = bufs * one_buf + sizeof(RingBars) + 256;
    int slots = budget > fixed ? (int)((budget - fixed) / (size_t)slot_bytes) : 0;
    if (slots > MAX_SLOTS) slots = MAX_SLOTS;
    if (slots < 2) return fail(NNE_ERR_UNSUPPORTED, "k=%zu leaves no room for a ring", kmax);
    const size_t smem = (size_t)slots * slot_bytes + fixed;
    if (peers && peers->world > 1) {
        if (m == 1)
            return launch_stream_mt<1, true>(ctx, batch, slots, slot_bytes, kpad, sb_rows, bufs, smem, grid,
                                             *peers, s);
        return launch_stream_mt<2, true>(ctx, batch, slots, slot_bytes, kpad, sb_rows, bufs, smem, grid,
                                         *peers, s);
    }
    const PeerSet none;
    if (m == 1)
        return launch_stream_mt<1, false>(ctx, batch, slots, slot_bytes, kpad, sb_rows, bufs, smem, grid,
                                          none, s);
    return launch_stream_mt<2, false>(ctx, batch, slots, slot_bytes, kpad, sb_rows, bufs, smem, grid, none, s);
}

int launch_gemv_tma(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                    const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                    cudaStream_t s) {
    StreamLayer L;
    L.q = q;
    L.scales = scales;
    L.bias = bias;
    L.x = x;
    L.y = y;
    L.ldy = ldy;
    L.n = (int)n;
    L.k = (int)k;
    L.rw = stream_rows_per_stage(k);
    return launch_stream_batch(ctx, &L, nullptr, 1, m, false, s);
}

// m > 2 activation rows on one layer: passes of two rows, all in ONE launch.  The first pass
// brings the weights from HBM, the later ones find them in L2 (a 7B-shaped layer is 17-45 MB of
// the 126 MB L2), and no launch gap separates the passes.
int launch_gemv_tma_passes(nne_ctx *ctx, const int8_t *q, const float *scales, const float *bias,
                           const float *x, float *y, size_t n, size_t k, size_t m, size_t ldy,
                           cudaStream_t s) {
    const size_t pairs = m / 2;
    if (pairs > (size_t)STREAM_INLINE_LAYERS)
        return fail(NNE_ERR_UNSUPPORTED, "m=%zu needs more passes than one launch holds", m);
    StreamLayer L[STREAM_INLINE_LAYERS];
    for (size_t p = 0; p < pairs; ++p) {
        L[p].q = q;
        L[p].scales = scales;
        L[p].bias = bias;
        L[p].x = x + 2 * p * k;
        L[p].y = y + 2 * p * ldy;
        L[p].ldy = ldy;
        L[p].n = (int)n;
        L[p].k = (int)k;
        L[p].rw = stream_rows_per_stage(k);
    }
    if (pairs) NNE_TRY(launch_stream_batch(ctx, L, nullptr, (int)pairs, 2, pairs > 1 || (m & 1), s));
    if (m & 1)
        NNE_TRY(launch_gemv_tma(ctx, q, scales, bias, x + (m - 1) * k, y + (m - 1) * ldy, n, k, 1, ldy, s));
    return NNE_OK;
}

}  // namespace nne
