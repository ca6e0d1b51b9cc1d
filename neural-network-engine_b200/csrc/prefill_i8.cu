// Prefill-shape forward (m > 16) on the 5th-generation tensor cores, integer form:
//   y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j])
// (device form of QLinear::forward_quantized, reference src/nn/quantized.rs:164-193, for large m).
//
// The int8 codes are fed to tcgen05.mma.kind::i8 exactly as they lie in memory - no dequantizer,
// no extra pass over shared memory.  Each activation row is put on a power-of-two fixed-point
// grid, v = rint(x * 2^e) with |v| < 2^15 (e from the row's largest |x|), and split into two
// balanced base-256 digits d0, d1 held as int8 (a small pre-pass).  Two MMAs per k-step accumulate
// D0 = X0.W^T and D1 = X1.W^T as EXACT int32 sums in two TMEM accumulators, and the epilogue forms
// dot = (D0 + 256*D1) * 2^-e, then * scales[j] and + bias[j] as separate fp32 operations like the
// reference (:187-190).  The one approximation is the rounding of x to the grid: at most
// 2^-15 of the row's largest |x| per element, i.e. a result error below 3.1e-5 of the a-priori
// bound ||x||inf * scale_j * sum|q_jk| the tolerance is written against (tolerance: 1e-3 of it) -
// 128 times tighter than rounding x to bf16 could guarantee, and the same grid as the decode
// kernels use.  The int8 pipe runs at twice the bf16
// rate, so two digit MMAs cost what one bf16 MMA would.  A row of x holding Inf or NaN yields NaN
// for that row.
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Per 128-wide k-block and stage:
//   warp 0      TMA producer: int8 weight tile [256 x 128] and the two activation digit tiles
//               [128 x 128], all 128B-swizzled straight into the UMMA K-major layout; no multicast
//   warp 1, 10  one thread each issues 4 tcgen05.mma (128x256x32, kind::i8) per k-block for one
//               activation digit, and tcgen05.commit
//   warps 2-9   epilogue: tcgen05.ld of both accumulators, combine, transpose through shared
//               memory, scale, bias, coalesced f32 stores
// Every mbarrier wait is bounded (~2 s): on expiry the context's device error word is set and the
// CTA drains, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"
#include "shard.cuh"

namespace nne {
namespace {

constexpr int BM = 128, BKB = 128;  // BKB: bytes (= int8 elements) of K per k-block
constexpr int MAX_STAGES = 4;
constexpr int X_BYTES = BM * BKB;   // 16 KB per digit
constexpr int BAR_BYTES = 256;
constexpr int NUM_EPI_WARPS = 8;  // two per TMEM lane quarter, each takes half of the columns
constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;  // one 32x32 f32 block per epilogue warp
// Output tiles are 128 x BN with BN = 256 (3 stages of 64 KB) or, when that would leave SMs idle
// or the last round of tiles mostly empty, BN = 128 (4 stages of 48 KB).
template <int BN>
struct Cfg {
    static constexpr int STAGES = BN == 256 ? 3 : 4;
    static constexpr int W_BYTES = BN * BKB;
    static constexpr int STAGE_BYTES = W_BYTES + 2 * (BM * BKB);
    static constexpr int SMEM_BYTES =
        STAGES * STAGE_BYTES + NUM_EPI_WARPS * (32 * 32 * 4) + BAR_BYTES + 1024;
    static constexpr uint32_t TMEM_COLS = 2 * BN;  // two int32 accumulators of BN columns
    // Instruction descriptor: D = s32, A = B = signed int8, both K-major, M = 128, N = BN.
    static constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                      ((uint32_t)(BM >> 4) << 24);
};
constexpr int MMA_WARP_1 = 2 + NUM_EPI_WARPS;  // the second MMA issuer sits after the epilogue warps
constexpr int THREADS = 32 * (3 + NUM_EPI_WARPS);

__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);   // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset (ignored when swizzled)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                       // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Exponent of the activation grid: max|x| * 2^e in [2^14, 2^15), one lower where the top digit
// would not stay below 128 once the balanced low digit has been split off.
__device__ __forceinline__ int grid_exponent16(float big) {
    int e = 14 - ((big > 0.0f) ? ilogbf(big) : 0);
    if (scalbnf(big, e) > 32639.0f) --e;
    return e;
}

// D0 + 256*D1 as one correctly rounded float, without a 64-bit integer or an int->float
// conversion (both are slow-rate instructions): split the sum as top * 2^20 + lo with
// |top| < 2^19 + 2^11 and 0 <= lo < 2^21, turn each part into a float exactly by adding it to the
// bit pattern of 1.5 * 2^23, and let one fused multiply-add round once.
__device__ __forceinline__ float combine(uint32_t d0, uint32_t d1) {
    const int b = (int)d0, a = (int)d1;
    const int top = (b >> 20) + (a >> 12);
    const int lo = (b & 0xFFFFF) + ((a & 0xFFF) << 8);
    const float ft = __int_as_float(0x4B400000 + top) - 12582912.0f;
    const float fl = __int_as_float(0x4B400000 + lo) - 12582912.0f;
    return fmaf(ft, 1048576.0f, fl);
}

struct Bars {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Bars) <= BAR_BYTES, "barrier block too large");

// PEER (column shards): the epilogue stores every output tile into this rank's window and, through
// the peer mappings, into the other ranks' windows - the all-gather of the output slices happens
// tile by tile under the MMAs of the following tiles (TMEM is handed back before anything is
// stored), instead of as a copy of the whole slice after the kernel.  Plain stores only.
template <int BN, bool PEER>
__global__ void __launch_bounds__(THREADS, 1)
qlinear_prefill_i8_kernel(const __grid_constant__ CUtensorMap tmap_w,
                          const __grid_constant__ CUtensorMap tmap_x0,
                          const __grid_constant__ CUtensorMap tmap_x1,
                          const float *__restrict__ unscale, const float *__restrict__ scales,
                          const float *__restrict__ bias, float *__restrict__ y, int m, int n, int k,
                          size_t ldy, int tiles_m, int num_tiles, int *err, const PeerSet ps) {
    constexpr int STAGES = Cfg<BN>::STAGES, W_BYTES = Cfg<BN>::W_BYTES,
                  STAGE_BYTES = Cfg<BN>::STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = Cfg<BN>::TMEM_COLS, IDESC = Cfg<BN>::IDESC;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *epi_smem = smem + STAGES * STAGE_BYTES;
    Bars *bars = reinterpret_cast<Bars *>(epi_smem + NUM_EPI_WARPS * EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k + BKB - 1) / BKB;
    volatile int *abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 2);  // both MMA issuers commit
        }
        mbar_init(smem_u32(&bars->acc_full), 2);
        mbar_init(smem_u32(&bars->acc_empty), NUM_EPI_WARPS);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    grid_launch_dependents();  // the next kernel's prologue may overlap this one

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // Weights never change after the layer is created, so the first ring of weight
            // tiles is requested before waiting for the pre-pass (the previous kernel in the
            // stream under programmatic dependent launch) that writes the digit planes.
            int pre = 0;
            if ((int)blockIdx.x < num_tiles) {
                const int n_first = ((int)blockIdx.x / tiles_m) * BN;
                for (; pre < STAGES && pre < num_kb; ++pre) {
                    const uint32_t full = smem_u32(&bars->full[pre]);
                    mbar_arrive_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(smem_u32(smem + pre * STAGE_BYTES), &tmap_w, pre * BKB, n_first, full);
                }
            }
            grid_dependency_wait();
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    uint8_t *st = smem + stage * STAGE_BYTES;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    if (pre > 0) {
                        --pre;  // slot still empty from the start; its weight tile is on the way
                    } else {
                        ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, err, 0x21);
                        if (!ok) break;
                        mbar_arrive_expect_tx(full, STAGE_BYTES);
                        tma_load_2d(smem_u32(st), &tmap_w, kb * BKB, n0, full);
                    }
                    tma_load_2d(smem_u32(st + W_BYTES), &tmap_x0, kb * BKB, m0, full);
                    tma_load_2d(smem_u32(st + W_BYTES + X_BYTES), &tmap_x1, kb * BKB, m0, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // Gave up: let copies that are still in flight land before the CTA exits.
                for (int s = 0; s < STAGES; ++s) {
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&bars->full[s]), 0) &&
                           !mbar_try_wait(smem_u32(&bars->full[s]), 1) &&
                           globaltimer_ns() - t0 < 100000000ull) {
                    }
                }
            }
        }
    } else if (warp == 1 || warp == MMA_WARP_1) {
        // ---------------- MMA issuers ----------------
        // One warp per activation digit.  A single thread needs about as long to issue an MMA as
        // the tensor pipe needs to run a 128 x 256 x 32 one, so with all eight MMAs of a k-block on
        // one thread every barrier wait and descriptor update showed up as idle pipe; two issuers
        // leave each with half the instructions.  Both commit to the stage's and the tile's
        // barriers (count 2): tcgen05.commit covers the MMAs of the thread that executes it.
        if (lane == 0) {
            const int digit = warp == 1 ? 0 : 1;
            const uint32_t d_tmem = tmem_base + (uint32_t)(digit * BN);
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                // the epilogue has drained both accumulators of the previous tile
                ok = mbar_wait(smem_u32(&bars->acc_empty), acc_phase ^ 1, abort_flag, err, 0x22);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 0x23);
                    if (!ok) break;
                    tc_fence_after();
                    uint8_t *st = smem + stage * STAGE_BYTES;
                    const uint64_t w_desc = make_kmajor_sw128_desc(smem_u32(st));
                    const uint64_t x_desc = make_kmajor_sw128_desc(smem_u32(st + W_BYTES + digit * X_BYTES));
#pragma unroll
                    for (int kk = 0; kk < BKB / 32; ++kk) {
                        // +32 bytes per 32-element k step inside the 128-byte swizzle span
                        umma_i8(d_tmem, x_desc + (uint64_t)(kk * 2), w_desc + (uint64_t)(kk * 2), IDESC,
                                (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bars->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&bars->acc_full));
                acc_phase ^= 1;
            }
        }
    } else {
        // ---------------- epilogue ----------------
        // Warp (quarter, half) drains TMEM lanes [32*quarter, +32) x columns [128*half, +128) of
        // both accumulators in four 32-column chunks.  A chunk arrives with lane = output row;
        // it is combined and multiplied by the row's 2^-e there, transposed through a 4 KB
        // shared block (float4 slots XOR-swizzled by row: conflict free both ways), and leaves
        // with 8 lanes per output row, so each store instruction writes four full 128-byte lines
        // and the channel's scale and bias are loaded once per chunk.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        float4 *stg = reinterpret_cast<float4 *>(epi_smem + (warp - 2) * EPI_STAGE_BYTES);
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool vec_ok = ((ldy & 3) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
        const int c4 = lane & 7, rsub = lane >> 3;
        grid_dependency_wait();  // unscale[] is written by the pre-pass
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
            const int row0 = m0 + quarter * 32;
            const int row = row0 + lane;
            // written by the pre-pass while this kernel may already be resident: a coherent load
            const float us = (row < m) ? __ldcg(unscale + row) : 0.0f;
            ok = mbar_wait(smem_u32(&bars->acc_full), acc_phase, abort_flag, err, 0x24);
            if (!ok) break;
            tc_fence_after();
            const uint32_t lane_base =
                tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * (BN / 2));
            // Drain: this warp's 128 columns of both accumulators become 128 floats in
            // registers, and TMEM goes back to the MMA warp before anything is stored.
            float f[BN / 2];
#pragma unroll
            for (int g = 0; g < BN / 32; ++g) {
                uint32_t r0[16], r1[16];
                tmem_ld_32x16(lane_base + (uint32_t)(g * 16), r0);
                tmem_ld_32x16(lane_base + (uint32_t)(BN + g * 16), r1);
                tmem_ld_wait();
#pragma unroll
                for (int v = 0; v < 16; ++v) f[g * 16 + v] = combine(r0[v], r1[v]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty));
            acc_phase ^= 1;
#pragma unroll
            for (int ci = 0; ci < BN / 64; ++ci) {
                const int j0 = n0 + half * (BN / 2) + ci * 32;
                if (j0 >= n) continue;
                if (vec_ok && j0 + 32 <= n) {
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float4 o;
                        o.x = f[ci * 32 + 4 * v + 0] * us;
                        o.y = f[ci * 32 + 4 * v + 1] * us;
                        o.z = f[ci * 32 + 4 * v + 2] * us;
                        o.w = f[ci * 32 + 4 * v + 3] * us;
                        stg[lane * 8 + (v ^ (lane & 7))] = o;
                    }
                    __syncwarp();
                    const float4 sc = __ldg(reinterpret_cast<const float4 *>(scales + j0) + c4);
                    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (bias) bv = __ldg(reinterpret_cast<const float4 *>(bias + j0) + c4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + rsub;
                        float4 o = stg[rr * 8 + (c4 ^ (rr & 7))];
                        o.x = __fmul_rn(o.x, sc.x);
                        o.y = __fmul_rn(o.y, sc.y);
                        o.z = __fmul_rn(o.z, sc.z);
                        o.w = __fmul_rn(o.w, sc.w);
                        if (bias) {
                            o.x = __fadd_rn(o.x, bv.x);
                            o.y = __fadd_rn(o.y, bv.y);
                            o.z = __fadd_rn(o.z, bv.z);
                            o.w = __fadd_rn(o.w, bv.w);
                        }
                        if (row0 + rr < m) {
                            float4 *dst = reinterpret_cast<float4 *>(y + (size_t)(row0 + rr) * ldy + j0 + 4 * c4);
                            *dst = o;
                            if (PEER) {
#pragma unroll
                                for (int q = 0; q < SHARD_MAX_RANKS; ++q)
                                    if (q < ps.world && q != ps.rank)
                                        *reinterpret_cast<float4 *>(reinterpret_cast<char *>(dst) + ps.delta[q]) = o;
                            }
                        }
                    }
                    __syncwarp();  // the block is rewritten by the next chunk
                } else if (row < m) {
                    float *yrow = y + (size_t)row * ldy;
#pragma unroll
                    for (int v = 0; v < 32; ++v) {
                        const int j = j0 + v;
                        if (j < n) {
                            float o = __fmul_rn(f[ci * 32 + v] * us, __ldg(scales + j));
                            if (bias) o = __fadd_rn(o, __ldg(bias + j));
                            yrow[j] = o;
                            if (PEER) {
#pragma unroll
                                for (int q = 0; q < SHARD_MAX_RANKS; ++q)
                                    if (q < ps.world && q != ps.rank)
                                        *reinterpret_cast<float *>(reinterpret_cast<char *>(yrow + j) + ps.delta[q]) = o;
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
}

// Activation pre-pass: one CTA of 256 threads per row of x [m, k] (k % 16 == 0).  Row max -> e
// with max|x| * 2^e in [2^14, 2^15); v = rint(x * 2^e); d0 = balanced low digit in [-128, 127],
// d1 = (v - d0) / 256 in [-128, 127].  unscale[r] = 2^-e (NaN if the row holds Inf/NaN).  The row
// is read from memory once: each thread keeps up to 8 float4 of it in registers between the two
// passes (k <= 8192); longer rows re-read the rest.
__global__ void __launch_bounds__(256)
x_to_digits_kernel(const float *__restrict__ x, int8_t *__restrict__ x0, int8_t *__restrict__ x1,
                   float *__restrict__ unscale, int m, int k) {
    __shared__ float wmax[8];
    __shared__ int wbad[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n4 = k >> 2;
    // x may be the output of the previous kernel in the stream, and the digit planes may still
    // be read by it: nothing is touched before that kernel has finished.
    grid_dependency_wait();
    grid_launch_dependents();
    for (int row = blockIdx.x; row < m; row += gridDim.x) {
        const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)row * k);
        float4 keep[8];
        float mx = 0.0f;
        int bad = 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * 256;
            keep[u] = (i < n4) ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float a0 = fabsf(keep[u].x), a1 = fabsf(keep[u].y), a2 = fabsf(keep[u].z),
                        a3 = fabsf(keep[u].w);
            bad |= !(a0 <= 3.402823466e38f) | !(a1 <= 3.402823466e38f) | !(a2 <= 3.402823466e38f) |
                   !(a3 <= 3.402823466e38f);
            mx = fmaxf(fmaxf(mx, fmaxf(a0, a1)), fmaxf(a2, a3));
        }
        for (int i = tid + 2048; i < n4; i += 256) {
            const float4 t = __ldg(src + i);
            const float a0 = fabsf(t.x), a1 = fabsf(t.y), a2 = fabsf(t.z), a3 = fabsf(t.w);
            bad |= !(a0 <= 3.402823466e38f) | !(a1 <= 3.402823466e38f) | !(a2 <= 3.402823466e38f) |
                   !(a3 <= 3.402823466e38f);
            mx = fmaxf(fmaxf(mx, fmaxf(a0, a1)), fmaxf(a2, a3));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        bad = __any_sync(0xffffffffu, bad);
        __syncthreads();  // the previous row's readers of wmax/wbad are done
        if (lane == 0) {
            wmax[warp] = mx;
            wbad[warp] = bad;
        }
        __syncthreads();
        mx = 0.0f;
        bad = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            mx = fmaxf(mx, wmax[w]);
            bad |= wbad[w];
        }
        const int e = grid_exponent16(mx);
        const int e1 = e >> 1, e2 = e - e1;  // 2^e = 2^e1 * 2^e2, both factors finite
        const float f1 = __int_as_float((127 + e1) << 23), f2 = __int_as_float((127 + e2) << 23);
        if (tid == 0) {
            const float u = __int_as_float((127 - e1) << 23) * __int_as_float((127 - e2) << 23);
            unscale[row] = bad ? __int_as_float(0x7fc00000) : u;
        }
        uint32_t *d0p = reinterpret_cast<uint32_t *>(x0 + (size_t)row * k);
        uint32_t *d1p = reinterpret_cast<uint32_t *>(x1 + (size_t)row * k);
        auto emit = [&](int i, const float4 &t) {
            const float xv[4] = {t.x, t.y, t.z, t.w};
            uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int v = bad ? 0 : rint_small(xv[b] * f1 * f2);  // |v| < 2^15
                const int d0 = ((v + 128) & 255) - 128;
                const int d1 = (v - d0) >> 8;
                w0 |= (uint32_t)(d0 & 0xff) << (8 * b);
                w1 |= (uint32_t)(d1 & 0xff) << (8 * b);
            }
            d0p[i] = w0;
            d1p[i] = w1;
        };
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * 256;
            if (i < n4) emit(i, keep[u]);
        }
        for (int i = tid + 2048; i < n4; i += 256) emit(i, __ldg(src + i));
    }
}

// The same pre-pass with the row brought into shared memory by a 1-D bulk copy, two row buffers
// per CTA: while a row is scanned and turned into digits the next one is already on its way, so
// the CTA always has a load outstanding.  For rows of at most 64 KB (k <= 16384).
__global__ void __launch_bounds__(256)
x_to_digits_bulk_kernel(const float *__restrict__ x, int8_t *__restrict__ x0, int8_t *__restrict__ x1,
                        float *__restrict__ unscale, int m, int k, int *err) {
    extern __shared__ __align__(128) uint8_t xsmem[];
    __shared__ uint64_t full[2];
    __shared__ float wmax[8];
    __shared__ int wbad[8];
    __shared__ int abort_word;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n4 = k >> 2;
    const uint32_t row_bytes = (uint32_t)k * 4u;
    volatile int *abort_flag = &abort_word;
    if (tid == 0) {
        mbar_init(smem_u32(&full[0]), 1);
        mbar_init(smem_u32(&full[1]), 1);
        abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // x may be the output of the previous kernel in the stream, and the digit planes may still
    // be read by it: nothing is touched before that kernel has finished.
    grid_dependency_wait();
    grid_launch_dependents();
    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            const long long row = (long long)blockIdx.x + (long long)b * gridDim.x;
            if (row < m) {
                mbar_arrive_expect_tx(smem_u32(&full[b]), row_bytes);
                bulk_load_1d(smem_u32(xsmem + (size_t)b * row_bytes), x + (size_t)row * k, row_bytes,
                             smem_u32(&full[b]));
            }
        }
    }
    __syncthreads();
    int it = 0;
    for (int row = blockIdx.x; row < m; row += gridDim.x, ++it) {
        const int b = it & 1;
        if (!mbar_wait(smem_u32(&full[b]), (uint32_t)((it >> 1) & 1), abort_flag, err, 0x26)) break;
        const float4 *src = reinterpret_cast<const float4 *>(xsmem + (size_t)b * row_bytes);
        float mx = 0.0f;
        int bad = 0;
        for (int i = tid; i < n4; i += 256) {
            const float4 t = src[i];
            const float a0 = fabsf(t.x), a1 = fabsf(t.y), a2 = fabsf(t.z), a3 = fabsf(t.w);
            bad |= !(a0 <= 3.402823466e38f) | !(a1 <= 3.402823466e38f) | !(a2 <= 3.402823466e38f) |
                   !(a3 <= 3.402823466e38f);
            mx = fmaxf(fmaxf(mx, fmaxf(a0, a1)), fmaxf(a2, a3));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        bad = __any_sync(0xffffffffu, bad);
        if (lane == 0) {
            wmax[warp] = mx;
            wbad[warp] = bad;
        }
        __syncthreads();
        mx = 0.0f;
        bad = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            mx = fmaxf(mx, wmax[w]);
            bad |= wbad[w];
        }
        const int e = grid_exponent16(mx);
        const int e1 = e >> 1, e2 = e - e1;  // 2^e = 2^e1 * 2^e2, both factors finite
        const float f1 = __int_as_float((127 + e1) << 23), f2 = __int_as_float((127 + e2) << 23);
        if (tid == 0) {
            const float u = __int_as_float((127 - e1) << 23) * __int_as_float((127 - e2) << 23);
            unscale[row] = bad ? __int_as_float(0x7fc00000) : u;
        }
        uint32_t *d0p = reinterpret_cast<uint32_t *>(x0 + (size_t)row * k);
        uint32_t *d1p = reinterpret_cast<uint32_t *>(x1 + (size_t)row * k);
        for (int i = tid; i < n4; i += 256) {
            const float4 t = src[i];
            const float xv[4] = {t.x, t.y, t.z, t.w};
            uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int v = bad ? 0 : rint_small(xv[c] * f1 * f2);  // |v| < 2^15
                const int d0 = ((v + 128) & 255) - 128;
                const int d1 = (v - d0) >> 8;
                w0 |= (uint32_t)(d0 & 0xff) << (8 * c);
                w1 |= (uint32_t)(d1 & 0xff) << (8 * c);
            }
            d0p[i] = w0;
            d1p[i] = w1;
        }
        __syncthreads();  // every thread is done with buffer b, wmax and wbad
        if (tid == 0) {
            const long long next = (long long)row + 2ll * gridDim.x;
            if (next < m) {
                fence_proxy_async();  // the generic-proxy reads above come before the async write
                mbar_arrive_expect_tx(smem_u32(&full[b]), row_bytes);
                bulk_load_1d(smem_u32(xsmem + (size_t)b * row_bytes), x + (size_t)next * k, row_bytes,
                             smem_u32(&full[b]));
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

}  // namespace

// NNE_PREPASS_BULK=0 keeps the register-staged activation pre-pass.
static bool prepass_bulk_disabled() {
    static const bool v = []() {
        const char *e = getenv("NNE_PREPASS_BULK");
        return e && e[0] == '0';
    }();
    return v;
}

// NNE_PREFILL_TILE=256 / =128 fixes the tile width for every shape (0: chosen per shape).
static int prefill_tile_forced() {
    static const int v = []() {
        const char *e = getenv("NNE_PREFILL_TILE");
        return (e && e[0] == '2') ? 256 : (e && e[0] == '1') ? 128 : 0;
    }();
    return v;
}

bool prefill_i8_supports(const nne_qlinear *ql, size_t m) {
    if (!ql || !ql->tmap_w8) return false;
    return m > 0 && m <= 0x7fffff00u;
}

int prefill_i8_prepare_layer(nne_qlinear *ql) {
    ql->tmap_w8 = nullptr;
    if (ql->n == 0 || ql->k == 0 || ql->k % 16 != 0) return NNE_OK;
    // int32 accumulators in TMEM: exact only below 2^17 terms of at most 2^14 each
    if (ql->n > 0x7fffff00u || ql->k > NNE_TENSOR_INT_MAX_K) return NNE_OK;
    if ((reinterpret_cast<uintptr_t>(ql->q) & 15u) != 0) return NNE_OK;
    CUtensorMap *map = new CUtensorMap;
    int st = tma_make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ql->q, ql->k, ql->n, BKB, 256,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NNE_OK) {
        delete map;
        return NNE_OK;  // no tensor maps on this driver: the layer simply does not take this path
    }
    ql->tmap_w8 = map;
    return NNE_OK;
}

void prefill_i8_release_layer(nne_qlinear *ql) {
    if (ql->tmap_w8) delete static_cast<CUtensorMap *>(ql->tmap_w8);
    ql->tmap_w8 = nullptr;
}

namespace {
template <int BN, bool PEER>
cudaError_t launch_main(const cudaLaunchConfig_t &cfg, const CUtensorMap &map_w, const CUtensorMap &x0,
                        const CUtensorMap &x1, const float *unscale, const nne_qlinear *ql, float *y, size_t m,
                        size_t ldy, int tiles_m, int tiles, int *err, const PeerSet &ps) {
    return cudaLaunchKernelEx(&cfg, qlinear_prefill_i8_kernel<BN, PEER>, map_w, x0, x1, unscale,
                              (const float *)ql->scales, (const float *)ql->bias, y, (int)m, (int)ql->n,
                              (int)ql->k, ldy, tiles_m, tiles, err, ps);
}
}  // namespace

int launch_prefill_i8(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy,
                      cudaStream_t s, const PeerSet *peers) {
    nne_ctx *ctx = ql->ctx;
    const bool peer = peers && peers->world > 1;
    if (peer) {
        NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_i8_kernel<256, true>, Cfg<256>::SMEM_BYTES));
        NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_i8_kernel<128, true>, Cfg<128>::SMEM_BYTES));
    } else {
        NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_i8_kernel<256, false>, Cfg<256>::SMEM_BYTES));
        NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_i8_kernel<128, false>, Cfg<128>::SMEM_BYTES));
    }
    // stream-ordered workspace: two int8 digit planes [m, k] and the per-row factors [m]
    const size_t plane = m * ql->k;
    const size_t bytes = 2 * plane + ((m * sizeof(float) + 255) & ~(size_t)255) + 256;
    uint8_t *ws = nullptr;
    NNE_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void **>(&ws), bytes, s));
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    int8_t *x0 = reinterpret_cast<int8_t *>(ws);
    int8_t *x1 = x0 + plane;
    float *unscale = reinterpret_cast<float *>(ws + ((2 * plane + 255) & ~(size_t)255));
    {
        size_t blocks = m;
        const size_t cap = (size_t)ctx->sm_count * 32;
        if (blocks > cap) blocks = cap;
        cudaLaunchConfig_t cfg = {};
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
        cudaError_t e;
        const size_t smem2 = 2 * ql->k * sizeof(float);
        if (smem2 <= 128 * 1024 && !prepass_bulk_disabled()) {
            NNE_TRY(ensure_dynamic_smem(ctx->device, x_to_digits_bulk_kernel, 128 * 1024));
            size_t per = (200 * 1024) / smem2;
            if (per > 6) per = 6;
            size_t nb = m;
            if (nb > (size_t)ctx->sm_count * per) nb = (size_t)ctx->sm_count * per;
            cfg.gridDim = dim3((unsigned)nb);
            cfg.dynamicSmemBytes = smem2;
            e = cudaLaunchKernelEx(&cfg, x_to_digits_bulk_kernel, x, x0, x1, unscale, (int)m, (int)ql->k,
                                   ctx->err_word);
        } else {
            cfg.gridDim = dim3((unsigned)blocks);
            e = cudaLaunchKernelEx(&cfg, x_to_digits_kernel, x, x0, x1, unscale, (int)m, (int)ql->k);
        }
        count_launch();
        if (e != cudaSuccess) {
            cudaFreeAsync(ws, s);
            return fail(NNE_ERR_CUDA, "activation pre-pass launch failed: %s", cudaGetErrorString(e));
        }
    }
    CUtensorMap tmap_x0, tmap_x1;
    int st = tma_make_map_2d(&tmap_x0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x0, ql->k, m, BKB, BM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (st == NNE_OK)
        st = tma_make_map_2d(&tmap_x1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x1, ql->k, m, BKB, BM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NNE_OK) {
        cudaFreeAsync(ws, s);
        return st;
    }
    const int tiles_m = (int)((m + BM - 1) / BM);
    // Tile width: rounds of tiles over the SMs, a 128-wide tile counted as 0.55 of a 256-wide one
    // (half the MMAs, the same activation tiles to load).  The narrow tile wins where the wide one
    // leaves SMs idle (m = 128: 43 tiles for 11008 channels) or its last round mostly empty.
    const long long t256 = (long long)tiles_m * (long long)((ql->n + 255) / 256);
    const long long t128 = (long long)tiles_m * (long long)((ql->n + 127) / 128);
    const long long sms = ctx->sm_count;
    const double cost256 = (double)((t256 + sms - 1) / sms);
    const double cost128 = 0.55 * (double)((t128 + sms - 1) / sms);
    const int forced = prefill_tile_forced();
    const bool narrow = ql->tmap_wsk != nullptr && (forced ? forced == 128 : cost128 < cost256);
    const long long tiles = narrow ? t128 : t256;
    if (tiles > 0x7fffffff) {
        cudaFreeAsync(ws, s);
        return fail(NNE_ERR_UNSUPPORTED, "too many output tiles");
    }
    int grid = ctx->sm_count;
    if (grid > tiles) grid = (int)tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)THREADS);
    cfg.dynamicSmemBytes = narrow ? Cfg<128>::SMEM_BYTES : Cfg<256>::SMEM_BYTES;
    cfg.stream = s;
    cfg.attrs = pdl;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    const PeerSet none;
    const PeerSet &ps = peer ? *peers : none;
    // the 128-row boxes are the small-batch kernel's tensor map of q
    const CUtensorMap &map_w = *static_cast<const CUtensorMap *>(narrow ? ql->tmap_wsk : ql->tmap_w8);
    cudaError_t e;
    if (narrow)
        e = peer ? launch_main<128, true>(cfg, map_w, tmap_x0, tmap_x1, unscale, ql, y, m, ldy, tiles_m, (int)tiles,
                                          ctx->err_word, ps)
                 : launch_main<128, false>(cfg, map_w, tmap_x0, tmap_x1, unscale, ql, y, m, ldy, tiles_m, (int)tiles,
                                           ctx->err_word, ps);
    else
        e = peer ? launch_main<256, true>(cfg, map_w, tmap_x0, tmap_x1, unscale, ql, y, m, ldy, tiles_m, (int)tiles,
                                          ctx->err_word, ps)
                 : launch_main<256, false>(cfg, map_w, tmap_x0, tmap_x1, unscale, ql, y, m, ldy, tiles_m, (int)tiles,
                                           ctx->err_word, ps);
    count_launch();
    cudaFreeAsync(ws, s);
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "prefill kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace nne
