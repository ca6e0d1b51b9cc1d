// QLinear::forward for small batches, 3 <= m <= 16 (reference: src/nn/quantized.rs:176-194), as an
// integer tensor-core kernel that reads the int8 weights exactly once.
//
// The weights are the M side of the MMA (128 output channels per tile), the activations the N
// side: the m rows of x go to the same fixed-point grid as in the streaming GEMV
// (v = rint(x * 2^e), |v| < 2^15, e from the row's largest |x|; two balanced base-256 int8
// digits), stacked as 32 "rows" (digit d of activation row r = row 16 d + r).  One
// tcgen05.mma.kind::i8 of shape 128 x 32 x 32 therefore multiplies 4 KB of weights with both
// digit planes of all 16 rows, and the int32 accumulators in TMEM hold EXACT integer sums.  With
// the same grid and the same final expression, the result for an activation row is bit-identical
// to what the streaming GEMV gives for that row alone.
//
// A layer has fewer 128-channel tiles than the GPU has SMs, so the (tile, k-block) units are cut
// into one contiguous range per CTA.  A CTA that owns a whole tile writes y itself; otherwise it
// adds its exact int64 partial sums into a zeroed workspace with integer atomics (order
// independent, so the result does not depend on timing) and the last CTA to finish a tile turns
// the sums into y.
//
// Warp roles per CTA (192 threads, 1 CTA per SM):
//   warp 0      TMA producer: 16 KB weight tile + 4 KB digit tile per unit into an 8-slot ring,
//               SWIZZLE_128B, weights with an L2 evict-first hint
//   warp 1      one lane issues 4 tcgen05.mma per unit and commits to the slot's mbarrier
//   warps 2-5   epilogue: tcgen05.ld (TMEM lane = output channel), combine the digits, then either
//               finalize or atomically add
// The pre-pass kernel (digits of x, per-row 2^-e, zeroing of the workspace) runs just before and
// the two are chained with programmatic dependent launch: the weight ring fills while the
// pre-pass runs.
//
// The kernel is driven by per-layer descriptors (SkLayer).  A single forward passes one in the
// parameter block; a plan (nne_qlinear_plan_*, 2 <= m <= 16) keeps an array of them in device
// memory and runs all its layers as ONE pre-pass + ONE launch over the concatenated units, with
// layers that read the same x sharing one set of digit planes.
#include <memory>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace nne {
namespace {

constexpr int SK_BM = 128;    // output channels per tile
constexpr int SK_BKB = 128;   // bytes (= int8 elements) of K per unit
constexpr int SK_ROWS = 16;   // activation rows (padded)
constexpr int SK_N = ACT_PLANES * 16;  // MMA N: digit planes x 16 rows
constexpr int SK_W_BYTES = SK_BM * SK_BKB;  // 16 KB
constexpr int SK_X_BYTES = SK_N * SK_BKB;   // 4 KB
constexpr int SK_STAGE_BYTES = SK_W_BYTES + SK_X_BYTES;  // 20 KB, a multiple of 1024
constexpr int SK_STAGES = 8;
constexpr int SK_BAR_BYTES = 256;
constexpr int SK_SMEM_BYTES = SK_STAGES * SK_STAGE_BYTES + SK_BAR_BYTES + 1024;
constexpr int SK_THREADS = 192;
constexpr uint32_t SK_TMEM_COLS = 128;  // two accumulators of 64 columns (SK_N used)
static_assert(SK_STAGE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");

__device__ __forceinline__ uint64_t sk_desc(uint32_t smem_addr) {  // K-major, SWIZZLE_128B
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;  // 8 rows * 128 B between row groups
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D = s32, A = B = signed int8, both K-major, M = 128, N = 48.
constexpr uint32_t SK_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(SK_N >> 3) << 17) |
                              ((uint32_t)(SK_BM >> 4) << 24);

__device__ __forceinline__ void sk_umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(SK_IDESC), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy)
        : "memory");
}

struct SkBars {
    uint64_t full[SK_STAGES];
    uint64_t empty[SK_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(SkBars) <= SK_BAR_BYTES, "barrier block too large");

// Unit range of CTA b of g: contiguous, as equal as the count allows.
__host__ __device__ inline void sk_range(long long total, int b, int g, long long &u0, long long &u1) {
    const long long base = total / g, rem = total % g;
    u0 = b * base + (b < rem ? b : rem);
    u1 = u0 + base + (b < rem ? 1 : 0);
}
// The CTA whose range holds unit u.
__host__ __device__ inline int sk_cta_of(long long total, int g, long long u) {
    const long long base = total / g, rem = total % g;
    const long long split = rem * (base + 1);
    if (u < split) return (int)(u / (base + 1));
    return (int)(rem + (u - split) / base);
}

// One layer of a launch.  A single forward passes one of these in the kernel's parameter block; a
// plan keeps an array of them in device memory (written by the host before any launch).
struct alignas(64) SkLayer {
    CUtensorMap tmap_w;    // q [n][k] int8, boxes of 128 rows x 128 bytes
    CUtensorMap tmap_x;    // digit planes [SK_N][k] of this layer's activations
    const float *scales;
    const float *bias;
    float *y;
    size_t ldy;
    long long *sums;       // [tiles][m][128] exact partial sums, zeroed by the pre-pass
    int *arrivals;         // [tiles][4] partial sums delivered so far per lane quarter, zeroed too
    const float *unscale;  // [16][2]: 2^-e of each row as two factors (NaN for a row with Inf/NaN)
    long long unit0;       // index of this layer's first (tile, k-block) unit in the launch
    int n, k, num_kb, tiles;
};
// One distinct activation matrix of a launch (layers that read the same x share it).
struct SkInput {
    const float *x;
    int8_t *xd;      // [SK_N][k]
    float *unscale;  // [16][2]
    int k;
};

__device__ __forceinline__ float sk_finish(long long s, float u0, float u1, float scale) {
    const float dot = (float)((double)s * (double)u0 * (double)u1);  // exact product, one rounding
    return __fmul_rn(dot, scale);
}

// The layer a role is working in, with the scalars it needs per unit held in registers: the
// descriptor itself sits in the parameter block or in global memory and is read only when the
// unit index crosses into another layer (units are visited in increasing order).
struct SkCur {
    long long unit0 = 0, end = 0;  // units [unit0, end) belong to layer li
    int num_kb = 1, li = -1;
};
__device__ __forceinline__ void sk_seek(const SkLayer &one, const SkLayer *many, int count,
                                        long long u, SkCur &c) {
    if (u < c.end) return;
    if (!many) {  // a single forward: the parameter block is read directly, not through a pointer
        c.li = 0;
        c.unit0 = 0;
        c.num_kb = one.num_kb;
        c.end = (long long)one.tiles * one.num_kb;
        return;
    }
    int li = c.li < 0 ? 0 : c.li;
    while (li + 1 < count && u >= many[li + 1].unit0) ++li;
    c.li = li;
    c.unit0 = many[li].unit0;
    c.num_kb = many[li].num_kb;
    c.end = c.unit0 + (long long)many[li].tiles * c.num_kb;
}
// Field f of the current layer.
#define SK_FIELD(f) (many ? many[c.li].f : one.f)

__global__ void __launch_bounds__(SK_THREADS, 1)
qlinear_skinny_i8_kernel(const __grid_constant__ SkLayer one, const SkLayer *__restrict__ many,
                         int count, int m, long long total, int *err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    SkBars *bars = reinterpret_cast<SkBars *>(smem + SK_STAGES * SK_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long u0, u1;
    sk_range(total, (int)blockIdx.x, (int)gridDim.x, u0, u1);
    volatile int *abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), 4);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"(SK_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    grid_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
            // Weights never change after the layer is created: the ring's first round of weight
            // tiles is requested before waiting for the pre-pass that writes the digit planes.
            int pre = 0;
            SkCur c;
            // (tile, kb) of the current unit are carried along instead of divided out per unit: the
            // producer is one thread, and its own instruction latency is what limits the ring.
            int tile = 0, kb = 0;
            for (; pre < SK_STAGES && u0 + pre < u1; ++pre) {
                const long long u = u0 + pre;
                if (u >= c.end) {
                    sk_seek(one, many, count, u, c);
                    const int lu = (int)(u - c.unit0);
                    tile = lu / c.num_kb;
                    kb = lu % c.num_kb;
                }
                const uint32_t full = smem_u32(&bars->full[pre]);
                mbar_arrive_expect_tx(full, SK_STAGE_BYTES);
                tma_load_2d_hint(smem_u32(smem + pre * SK_STAGE_BYTES), (many ? &many[c.li].tmap_w : &one.tmap_w), kb * SK_BKB,
                                 tile * SK_BM, full, pol_w);
                if (++kb == c.num_kb) { kb = 0; ++tile; }
            }
            grid_dependency_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            c = SkCur();
            const CUtensorMap *map_w = nullptr, *map_x = nullptr;
            for (long long u = u0; u < u1; ++u) {
                if (u >= c.end) {
                    sk_seek(one, many, count, u, c);
                    map_w = many ? &many[c.li].tmap_w : &one.tmap_w;
                    map_x = many ? &many[c.li].tmap_x : &one.tmap_x;
                    const int lu = (int)(u - c.unit0);
                    tile = lu / c.num_kb;
                    kb = lu % c.num_kb;
                }
                uint8_t *st = smem + stage * SK_STAGE_BYTES;
                const uint32_t full = smem_u32(&bars->full[stage]);
                if (pre > 0) {
                    --pre;
                } else {
                    ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, err, 0x31);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full, SK_STAGE_BYTES);
                    tma_load_2d_hint(smem_u32(st), map_w, kb * SK_BKB, tile * SK_BM, full, pol_w);
                }
                tma_load_2d_hint(smem_u32(st + SK_W_BYTES), map_x, kb * SK_BKB, 0, full, pol_x);
                if (++kb == c.num_kb) { kb = 0; ++tile; }
                if (++stage == SK_STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                // Gave up: let copies that are still in flight land before the CTA exits.
                for (int s = 0; s < SK_STAGES; ++s) {
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(smem_u32(&bars->full[s]), 0) &&
                           !mbar_try_wait(smem_u32(&bars->full[s]), 1) &&
                           globaltimer_ns() - t0 < 100000000ull) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int seg = 0;
            bool ok = true;
            long long u = u0;
            SkCur c;
            while (u < u1 && ok) {
                sk_seek(one, many, count, u, c);
                const int lu = (int)(u - c.unit0);
                long long seg_end = u + (c.num_kb - lu % c.num_kb);  // end of this (layer, tile)
                if (seg_end > u1) seg_end = u1;
                const int buf = seg & 1;
                ok = mbar_wait(smem_u32(&bars->acc_empty[buf]), (uint32_t)(((seg >> 1) & 1) ^ 1),
                               abort_flag, err, 0x32);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 64);
                bool first = true;
                for (; u < seg_end; ++u) {
                    ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 0x33);
                    if (!ok) break;
                    tc_fence_after();
                    uint8_t *st = smem + stage * SK_STAGE_BYTES;
                    const uint64_t w_desc = sk_desc(smem_u32(st));
                    const uint64_t x_desc = sk_desc(smem_u32(st + SK_W_BYTES));
#pragma unroll
                    for (int kk = 0; kk < SK_BKB / 32; ++kk) {
                        sk_umma(d_tmem, w_desc + (uint64_t)(kk * 2), x_desc + (uint64_t)(kk * 2),
                                (first && kk == 0) ? 0u : 1u);
                    }
                    first = false;
                    umma_commit(smem_u32(&bars->empty[stage]));
                    if (++stage == SK_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&bars->acc_full[buf]));
                ++seg;
            }
        }
    } else {
        // ---------------- epilogue ----------------
        grid_dependency_wait();  // unscale[], sums[] and arrivals[] are written by the pre-pass
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) belong to this warp
        const int ch_in_tile = quarter * 32 + lane;
        int seg = 0;
        bool ok = true;
        long long u = u0;
        SkCur c;
        while (u < u1 && ok) {
            sk_seek(one, many, count, u, c);
            const int tile = (int)(u - c.unit0) / c.num_kb;
            const long long tile_u0 = c.unit0 + (long long)tile * c.num_kb, tile_u1 = tile_u0 + c.num_kb;
            const long long seg_end = tile_u1 < u1 ? tile_u1 : u1;
            const bool whole = (u == tile_u0) && (seg_end == tile_u1);
            const int buf = seg & 1;
            // Everything the segment needs from the descriptor and from global memory is fetched
            // before the wait, so that only the TMEM read and the reduction follow the MMAs.
            const int ch = tile * SK_BM + ch_in_tile;
            const int n = SK_FIELD(n);
            long long *dst = SK_FIELD(sums) + ((size_t)tile * m) * SK_BM + ch_in_tile;
            int *ticket_word = SK_FIELD(arrivals) + tile * 4 + quarter;
            const float *bias = SK_FIELD(bias);
            const float *unscale = SK_FIELD(unscale);
            float *y = SK_FIELD(y);
            const size_t ldy = SK_FIELD(ldy);
            const float sc = (ch < n) ? __ldg(SK_FIELD(scales) + ch) : 0.0f;
            const float bv = (bias && ch < n) ? __ldg(bias + ch) : 0.0f;
            const int parts = whole ? 1
                                    : sk_cta_of(total, (int)gridDim.x, tile_u1 - 1) -
                                          sk_cta_of(total, (int)gridDim.x, tile_u0) + 1;
            ok = mbar_wait(smem_u32(&bars->acc_full[buf]), (uint32_t)((seg >> 1) & 1), abort_flag, err,
                           0x34);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 64);
            uint32_t dg[ACT_PLANES][16];
#pragma unroll
            for (int p = 0; p < ACT_PLANES; ++p) tmem_ld_32x16(taddr + 16 * p, dg[p]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[buf]));

            long long s[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                s[r] = 0;
#pragma unroll
                for (int p = ACT_PLANES - 1; p >= 0; --p) s[r] = s[r] * (1 << ACT_DIGIT_BITS) + (long long)(int)dg[p][r];
            }

            bool finish = whole;
            if (!whole) {
#pragma unroll
                for (int r = 0; r < 16; ++r)
                    if (r < m)
                        atomicAdd(reinterpret_cast<unsigned long long *>(dst + r * SK_BM),
                                  (unsigned long long)s[r]);
                // Each warp keeps its own count per (tile, lane quarter): no rendezvous between
                // the epilogue warps.  The fence orders this warp's additions before its ticket.
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    const int ticket = atomicAdd(ticket_word, 1);
                    last = (ticket == parts - 1) ? 1 : 0;
                    __threadfence();
                }
                finish = __shfl_sync(0xffffffffu, last, 0) != 0;
                if (finish) {
#pragma unroll
                    for (int r = 0; r < 16; ++r)
                        if (r < m) s[r] = __ldcg(dst + r * SK_BM);
                }
            }
            if (finish && ch < n) {
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    if (r < m) {
                        // unscale[] is written by the pre-pass while this kernel may already be resident:
                        // coherent loads, not the read-only path
                        float v = sk_finish(s[r], __ldcg(unscale + 2 * r), __ldcg(unscale + 2 * r + 1), sc);
                        if (bias) v = __fadd_rn(v, bv);
                        y[(size_t)r * ldy + ch] = v;
                    }
                }
            }
            u = seg_end;
            ++seg;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(SK_TMEM_COLS)
                     : "memory");
    }
}

// Pre-pass.  Blocks 0 .. 16*count-1: activation row r = block % 16 of input block / 16, x [m, k]
// (k % 16 == 0) -> digit plane p at row 16 p + r of xd [SK_N, k] and the row's 2^-e as two factors
// (rows >= m: zeros).  Same grid as the streaming GEMV (act_grid_exponent).
// The blocks after those zero the partial-sum workspace and the arrival counters.
__global__ void __launch_bounds__(256)
skinny_prepass_kernel(const __grid_constant__ SkInput one, const SkInput *__restrict__ many, int count,
                      int m, uint4 *__restrict__ zero_base, size_t zero_count) {
    __shared__ float wmax[8];
    __shared__ int wbad[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // x may be the output of the previous kernel in the stream, and the workspace may still be
    // in use by it: nothing is touched before that kernel has finished.
    grid_dependency_wait();
    grid_launch_dependents();
    const int row_blocks = SK_ROWS * count;
    if ((int)blockIdx.x >= row_blocks) {
        const size_t nz = gridDim.x - row_blocks;
        for (size_t i = (size_t)(blockIdx.x - row_blocks) * 256 + tid; i < zero_count; i += nz * 256)
            zero_base[i] = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const SkInput &in = many ? many[blockIdx.x / SK_ROWS] : one;
    const int row = blockIdx.x % SK_ROWS;
    const int k = in.k;
    const float *x = in.x;
    int8_t *xd = in.xd;
    float *unscale = in.unscale;
    const int n4 = k >> 2;
    uint32_t *pl[ACT_PLANES];
#pragma unroll
    for (int p = 0; p < ACT_PLANES; ++p) pl[p] = reinterpret_cast<uint32_t *>(xd + (size_t)(p * SK_ROWS + row) * k);
    if (row >= m) {
        for (int i = tid; i < n4; i += 256)
#pragma unroll
            for (int p = 0; p < ACT_PLANES; ++p) pl[p][i] = 0u;
        if (tid == 0) unscale[2 * row] = unscale[2 * row + 1] = 0.0f;
        return;
    }
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)row * k);
    // The row is read once: each thread keeps up to 8 float4 of it in registers between the max
    // pass and the digit pass (k <= 8192); longer rows re-read the rest.
    float4 keep[8];
    float mx = 0.0f;
    int bad = 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        keep[u] = (i < n4) ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    auto scan = [&](const float4 &t) {
        const float a0 = fabsf(t.x), a1 = fabsf(t.y), a2 = fabsf(t.z), a3 = fabsf(t.w);
        bad |= !(a0 <= 3.402823466e38f) | !(a1 <= 3.402823466e38f) | !(a2 <= 3.402823466e38f) |
               !(a3 <= 3.402823466e38f);
        mx = fmaxf(fmaxf(mx, fmaxf(a0, a1)), fmaxf(a2, a3));
    };
#pragma unroll
    for (int u = 0; u < 8; ++u) scan(keep[u]);
    for (int i = tid + 2048; i < n4; i += 256) scan(__ldg(src + i));
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
    const int e = act_grid_exponent(mx);
    const int e1 = e >> 1, e2 = e - e1;  // 2^e = 2^e1 * 2^e2, both factors finite
    const float f1 = __int_as_float((127 + e1) << 23), f2 = __int_as_float((127 + e2) << 23);
    if (tid == 0) {
        const float nan = __int_as_float(0x7fc00000);
        unscale[2 * row] = bad ? nan : __int_as_float((127 - e1) << 23);
        unscale[2 * row + 1] = bad ? nan : __int_as_float((127 - e2) << 23);
    }
    auto emit = [&](int i, const float4 &t) {
        const float xv[4] = {t.x, t.y, t.z, t.w};
        if constexpr (ACT_PLANES == 2) {
            // the digits are bytes 0 of word and 1 of word + 128 of x * 2^e + 1.5 * 2^23 (its low 23
            // bits hold v in two's complement), as in the streaming GEMV
            uint32_t b[4], c[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = __float_as_uint(__fadd_rn(bad ? 0.0f : xv[j] * f1 * f2, 12582912.0f));
                c[j] = b[j] + 128u;
            }
            pl[0][i] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
            pl[ACT_PLANES - 1][i] = __byte_perm(__byte_perm(c[0], c[1], 0x0051), __byte_perm(c[2], c[3], 0x0051), 0x5410);
            return;
        }
        constexpr int HALF = 1 << (ACT_DIGIT_BITS - 1), MASK = (1 << ACT_DIGIT_BITS) - 1;
        uint32_t w[ACT_PLANES];
#pragma unroll
        for (int p = 0; p < ACT_PLANES; ++p) w[p] = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            int v = bad ? 0 : rint_small(xv[b] * f1 * f2);  // |v| < 2^ACT_GRID_BITS
#pragma unroll
            for (int p = 0; p < ACT_PLANES - 1; ++p) {
                const int dp = ((v + HALF) & MASK) - HALF;
                w[p] |= (uint32_t)(dp & 0xff) << (8 * b);
                v = (v - dp) >> ACT_DIGIT_BITS;
            }
            w[ACT_PLANES - 1] |= (uint32_t)(v & 0xff) << (8 * b);
        }
#pragma unroll
        for (int p = 0; p < ACT_PLANES; ++p) pl[p][i] = w[p];
    };
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        if (i < n4) emit(i, keep[u]);
    }
    for (int i = tid + 2048; i < n4; i += 256) emit(i, __ldg(src + i));
}

}  // namespace

bool skinny_supports(const nne_qlinear *ql, size_t m) {
    if (!ql || !ql->tmap_wsk) return false;
    return m >= 3 && m <= (size_t)SK_ROWS;
}

int skinny_prepare_layer(nne_qlinear *ql) {
    ql->tmap_wsk = nullptr;
    if (ql->n == 0 || ql->k == 0 || ql->k % 16 != 0) return NNE_OK;
    // One product is at most 128 * 64 = 2^13 in magnitude and a tile's int32 accumulator in TMEM
    // adds k of them: exact only up to k = 2^18.  Longer rows go to the generic kernel.
    if (ql->n > 0x7fffff00u || ql->k > NNE_TENSOR_INT_MAX_K) return NNE_OK;
    if ((reinterpret_cast<uintptr_t>(ql->q) & 15u) != 0) return NNE_OK;
    CUtensorMap *map = new CUtensorMap;
    int st = tma_make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ql->q, ql->k, ql->n, SK_BKB, SK_BM,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NNE_OK) {
        delete map;
        return NNE_OK;  // no tensor maps on this driver: the layer simply does not take this path
    }
    ql->tmap_wsk = map;
    return NNE_OK;
}

void skinny_release_layer(nne_qlinear *ql) {
    if (ql->tmap_wsk) delete static_cast<CUtensorMap *>(ql->tmap_wsk);
    ql->tmap_wsk = nullptr;
}

namespace {

int set_smem_attr(const nne_ctx *ctx) {
    return ensure_dynamic_smem(ctx->device, qlinear_skinny_i8_kernel, SK_SMEM_BYTES);
}

size_t sk_tiles(size_t n) { return (n + SK_BM - 1) / SK_BM; }
size_t sk_num_kb(size_t k) { return (k + SK_BKB - 1) / SK_BKB; }
size_t sk_sums_bytes(size_t n, size_t m) { return sk_tiles(n) * m * SK_BM * sizeof(long long); }
size_t sk_arrivals_bytes(size_t n) { return (sk_tiles(n) * 4 * sizeof(int) + 255) & ~(size_t)255; }
size_t sk_xd_bytes(size_t k) { return ((size_t)SK_N * k + 255) & ~(size_t)255; }

// Fills everything of a layer's descriptor except the activation side and the work areas.
void sk_fill_layer(SkLayer &L, const nne_qlinear *ql, float *y, size_t ldy) {
    L.tmap_w = *static_cast<const CUtensorMap *>(ql->tmap_wsk);
    L.scales = ql->scales;
    L.bias = ql->bias;
    L.y = y;
    L.ldy = ldy;
    L.n = (int)ql->n;
    L.k = (int)ql->k;
    L.num_kb = (int)sk_num_kb(ql->k);
    L.tiles = (int)sk_tiles(ql->n);
}

int sk_launch(nne_ctx *ctx, const SkLayer *one, const SkLayer *many_dev, int count, const SkInput *in_one,
              const SkInput *in_many_dev, int in_count, size_t m, long long total, uint4 *zero_base,
              size_t zero_bytes, cudaStream_t s) {
    NNE_TRY(set_smem_attr(ctx));
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    {
        size_t zblocks = (zero_bytes / 16 + 2047) / 2048;  // 8 uint4 per thread
        if (zblocks < 1) zblocks = 1;
        if (zblocks > 128) zblocks = 128;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(SK_ROWS * in_count + zblocks));
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cfg.attrs = pdl;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
        cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_prepass_kernel, *in_one, in_many_dev, in_count,
                                           (int)m, zero_base, zero_bytes / 16);
        count_launch();
        if (e != cudaSuccess)
            return fail(NNE_ERR_CUDA, "skinny pre-pass launch failed: %s", cudaGetErrorString(e));
    }
    int grid = ctx->sm_count;
    if (grid > total) grid = (int)total;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)SK_THREADS);
    cfg.dynamicSmemBytes = SK_SMEM_BYTES;
    cfg.stream = s;
    cfg.attrs = pdl;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, qlinear_skinny_i8_kernel, *one, many_dev, count, (int)m,
                                       total, ctx->err_word);
    count_launch();
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "skinny kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace

int launch_skinny(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy, cudaStream_t s) {
    nne_ctx *ctx = ql->ctx;
    const size_t k = ql->k, n = ql->n;
    // stream-ordered workspace: [sums | arrivals] (zeroed by the pre-pass), unscale, digit planes
    const size_t sums_bytes = sk_sums_bytes(n, m);
    const size_t zero_bytes = sums_bytes + sk_arrivals_bytes(n);  // a multiple of 16
    const size_t uns_bytes = 256;
    uint8_t *ws = nullptr;
    NNE_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void **>(&ws), zero_bytes + uns_bytes + sk_xd_bytes(k), s));
    SkInput in;
    in.x = x;
    in.unscale = reinterpret_cast<float *>(ws + zero_bytes);
    in.xd = reinterpret_cast<int8_t *>(ws + zero_bytes + uns_bytes);
    in.k = (int)k;
    SkLayer L;
    sk_fill_layer(L, ql, y, ldy);
    L.sums = reinterpret_cast<long long *>(ws);
    L.arrivals = reinterpret_cast<int *>(ws + sums_bytes);
    L.unscale = in.unscale;
    L.unit0 = 0;
    int st = tma_make_map_2d(&L.tmap_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, in.xd, k, SK_N, SK_BKB, SK_N,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (st == NNE_OK)
        st = sk_launch(ctx, &L, nullptr, 1, &in, nullptr, 1, m, (long long)L.tiles * L.num_kb,
                       reinterpret_cast<uint4 *>(ws), zero_bytes, s);
    cudaFreeAsync(ws, s);
    return st;
}

// ---- plan: several layers in one launch ------------------------------------------------------------
// The plan owns its work areas (partial sums, counters, digit planes) and the device copies of
// the descriptors, all allocated once at creation: a run allocates nothing.  Layers that read
// the same x (q/k/v, gate/up) share one set of digit planes.
struct SkPlan {
    nne_ctx *ctx = nullptr;
    uint8_t *ws = nullptr;
    SkLayer *layers_dev = nullptr;
    SkInput *inputs_dev = nullptr;
    SkLayer first_layer;   // passed by value too (the kernel's parameter block wants one)
    SkInput first_input;
    int count = 0, in_count = 0;
    size_t m = 0, zero_bytes = 0;
    long long total = 0;
};

bool skinny_plan_supports(nne_qlinear *const *layers, const float *const *x, float *const *y,
                          size_t count, size_t m) {
    // m = 2 is taken too: over a list of layers this kernel streams at 5.1 TB/s where the dp4a GEMV,
    // arithmetic bound at two rows, reaches 3.0 (a single two-row forward stays with the GEMV,
    // whose launch-to-result chain is shorter).
    if (count == 0 || count > 4096 || m < 2 || m > (size_t)SK_ROWS) return false;
    for (size_t i = 0; i < count; ++i) {
        if (!layers[i] || !layers[i]->tmap_wsk) return false;
        if ((reinterpret_cast<uintptr_t>(x[i]) & 15u) || (reinterpret_cast<uintptr_t>(y[i]) & 3u)) return false;
    }
    return true;
}

int skinny_plan_create(nne_ctx *ctx, nne_qlinear *const *layers, const float *const *x, float *const *y,
                       const size_t *ldy_or_null, size_t count, size_t m, SkPlan **out) {
    *out = nullptr;
    std::unique_ptr<SkPlan> plan(new SkPlan());
    plan->ctx = ctx;
    plan->count = (int)count;
    plan->m = m;
    // distinct inputs
    std::vector<int> input_of(count);
    std::vector<SkInput> inputs;
    for (size_t i = 0; i < count; ++i) {
        int found = -1;
        for (size_t j = 0; j < inputs.size(); ++j)
            if (inputs[j].x == x[i] && (size_t)inputs[j].k == layers[i]->k) found = (int)j;
        if (found < 0) {
            SkInput in;
            in.x = x[i];
            in.xd = nullptr;
            in.unscale = nullptr;
            in.k = (int)layers[i]->k;
            inputs.push_back(in);
            found = (int)inputs.size() - 1;
        }
        input_of[i] = found;
    }
    plan->in_count = (int)inputs.size();
    // one allocation: [sums and arrivals of every layer | unscale per input | digit planes per input]
    size_t zero_bytes = 0;
    for (size_t i = 0; i < count; ++i) zero_bytes += sk_sums_bytes(layers[i]->n, m) + sk_arrivals_bytes(layers[i]->n);
    size_t bytes = zero_bytes + 256 * inputs.size();
    for (const SkInput &in : inputs) bytes += sk_xd_bytes((size_t)in.k);
    NNE_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&plan->ws), bytes));
    struct Guard {
        SkPlan *p;
        ~Guard() {
            if (!p) return;
            cudaFree(p->ws);
            cudaFree(p->layers_dev);
            cudaFree(p->inputs_dev);
        }
    } guard{plan.get()};
    plan->zero_bytes = zero_bytes;
    uint8_t *cur = plan->ws + zero_bytes;
    for (SkInput &in : inputs) {
        in.unscale = reinterpret_cast<float *>(cur);
        cur += 256;
    }
    std::vector<CUtensorMap> xmaps(inputs.size());
    for (size_t j = 0; j < inputs.size(); ++j) {
        inputs[j].xd = reinterpret_cast<int8_t *>(cur);
        cur += sk_xd_bytes((size_t)inputs[j].k);
        NNE_TRY(tma_make_map_2d(&xmaps[j], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, inputs[j].xd, (size_t)inputs[j].k,
                                SK_N, SK_BKB, SK_N, CU_TENSOR_MAP_SWIZZLE_128B));
    }
    std::vector<SkLayer> descs(count);
    uint8_t *z = plan->ws;
    long long unit = 0;
    for (size_t i = 0; i < count; ++i) {
        SkLayer &L = descs[i];
        sk_fill_layer(L, layers[i], y[i], ldy_or_null ? ldy_or_null[i] : layers[i]->n);
        L.tmap_x = xmaps[input_of[i]];
        L.unscale = inputs[input_of[i]].unscale;
        L.sums = reinterpret_cast<long long *>(z);
        z += sk_sums_bytes(layers[i]->n, m);
        L.arrivals = reinterpret_cast<int *>(z);
        z += sk_arrivals_bytes(layers[i]->n);
        L.unit0 = unit;
        unit += (long long)L.tiles * L.num_kb;
    }
    plan->total = unit;
    NNE_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&plan->layers_dev), count * sizeof(SkLayer)));
    NNE_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&plan->inputs_dev), inputs.size() * sizeof(SkInput)));
    NNE_CUDA_TRY(cudaMemcpy(plan->layers_dev, descs.data(), count * sizeof(SkLayer), cudaMemcpyHostToDevice));
    NNE_CUDA_TRY(cudaMemcpy(plan->inputs_dev, inputs.data(), inputs.size() * sizeof(SkInput),
                            cudaMemcpyHostToDevice));
    plan->first_layer = descs[0];
    plan->first_input = inputs[0];
    guard.p = nullptr;
    *out = plan.release();
    return NNE_OK;
}

int skinny_plan_run(SkPlan *plan, cudaStream_t s) {
    return sk_launch(plan->ctx, &plan->first_layer, plan->layers_dev, plan->count, &plan->first_input,
                     plan->inputs_dev, plan->in_count, plan->m, plan->total,
                     reinterpret_cast<uint4 *>(plan->ws), plan->zero_bytes, s);
}

void skinny_plan_destroy(SkPlan *plan) {
    if (!plan) return;
    cudaFree(plan->ws);
    cudaFree(plan->layers_dev);
    cudaFree(plan->inputs_dev);
    delete plan;
}

}  // namespace nne
