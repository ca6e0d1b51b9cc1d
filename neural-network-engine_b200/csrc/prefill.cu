// Prefill-shape forward (m > 16) on the 5th-generation tensor cores:
//   y[r,j] = (sum_i bf16(x[r,i]) * q[j,i]) * scales[j] (+ bias[j]),  fp32 accumulation in TMEM.
// Device form of QLinear::forward_quantized (reference src/nn/quantized.rs:164-193) for large m.
// int8 -> bf16 is exact (|q| <= 128); rounding x to bf16 is the only approximation: per channel at
// most 2^-8 * ||x||inf * scale_j * sum_k |q_jk|, i.e. up to 3.9 times the path's tolerance (1e-3 of
// that bound) when every rounding error lines up, a few percent of it on N(0,1) activations.
// That is why this kernel runs only on request (NNE_PREFILL=bf16, nne_qlinear_forward_dev_static).
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Per 64-wide k-block and stage:
//   warp 0      TMA producer, 4 stages deep: bf16 activations tile [128 x 64] (128B-swizzled,
//               straight into the UMMA layout) and int8 weight tile [256 x 64] (dense staging)
//   warps 2-9   dequantizers: int8 staging -> one of two bf16 tiles in the 128B-swizzled K-major
//               UMMA layout, then fence.proxy.async and an mbarrier arrive
//   warp 1      one thread issues 4 tcgen05.mma (128x256x16, kind::f16, bf16 in, f32 out in TMEM)
//               and tcgen05.commit releases the stage
//   warps 10-13 epilogue: tcgen05.ld of the finished accumulator (double buffered, 2 x 256 TMEM
//               columns), multiply by the channel scale, add bias, store f32
// Activations are converted f32 -> bf16 once per call by a small pre-pass into a stream-ordered
// workspace.  No load in this file uses cluster multicast.
//
// Every mbarrier wait is bounded: after ~2 s it raises the context's device error word, the CTA
// drains, frees its TMEM and returns, so a broken pipeline can never hang the GPU.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace nne {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;    // TMA ring: bf16 activations tile + int8 weights tile per stage
constexpr int BSTAGES = 2;   // ring of dequantized bf16 weight tiles (dequantizers -> MMA)
constexpr int A_BYTES = BM * BK * 2;   // 16 KB bf16 activations
constexpr int B_BYTES = BN * BK * 2;   // 32 KB bf16 weights (dequantized here)
constexpr int WQ_BYTES = BN * BK;      // 16 KB int8 weights (TMA staging)
constexpr int STAGE_BYTES = A_BYTES + WQ_BYTES;  // one TMA stage
constexpr int BAR_BYTES = 256;
// TMA stages first, then the bf16 weight tiles (all 1 KB aligned), + 1 KB alignment slack
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BSTAGES * B_BYTES + BAR_BYTES + 1024;
constexpr int NUM_CONVERT_WARPS = 8, NUM_EPI_WARPS = 4;
constexpr int THREADS = 32 * (2 + NUM_CONVERT_WARPS + NUM_EPI_WARPS);  // 448
constexpr uint32_t TMEM_COLS = 512;

// Shared-memory matrix descriptor for a K-major bf16 tile in the 128B-swizzled canonical layout:
// rows are 128 bytes (64 bf16), groups of 8 rows are 1024 bytes apart (SBO), LBO is unused.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);   // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset (ignored when swizzled)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                       // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = 256.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                           ((uint32_t)(BM >> 4) << 24);

// Four int8 in a word -> two bf16x2 words, exactly.  For a byte b = u7 - 128*s (u7 its low 7
// bits, s its sign bit): 0x4300|u7 is the bf16 128+u7, 0x4300|(s<<7) is the bf16 128 or 256,
// and their difference is b.
__device__ __forceinline__ void cvt_i8x4_bf16(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t mag = w & 0x7F7F7F7Fu, sgn = w & 0x80808080u;
    const uint32_t p01 = __byte_perm(mag, 0x43434343u, 0x4140);
    const uint32_t p23 = __byte_perm(mag, 0x43434343u, 0x4342);
    const uint32_t s01 = __byte_perm(sgn, 0x43434343u, 0x4140);
    const uint32_t s23 = __byte_perm(sgn, 0x43434343u, 0x4342);
    __nv_bfloat162 a = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&p01),
                               *reinterpret_cast<const __nv_bfloat162 *>(&s01));
    __nv_bfloat162 b = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&p23),
                               *reinterpret_cast<const __nv_bfloat162 *>(&s23));
    lo = *reinterpret_cast<uint32_t *>(&a);
    hi = *reinterpret_cast<uint32_t *>(&b);
}

struct Bars {
    uint64_t full[STAGES];     // TMA bytes of the stage have landed
    uint64_t empty[STAGES];    // the MMAs that read the stage's activations have completed
    uint64_t bready[BSTAGES];  // bf16 weight tile is written and fenced
    uint64_t bfree[BSTAGES];   // the MMAs that read the bf16 weight tile have completed
    uint64_t acc_full[2];      // accumulator buffer holds a finished tile
    uint64_t acc_empty[2];     // accumulator buffer has been drained
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Bars) <= BAR_BYTES, "barrier block too large");

__global__ void __launch_bounds__(THREADS, 1)
qlinear_prefill_kernel(const __grid_constant__ CUtensorMap tmap_x,
                       const __grid_constant__ CUtensorMap tmap_w,
                       const float *__restrict__ scales, const float *__restrict__ bias,
                       float *__restrict__ y, int m, int n, int k, size_t ldy, int tiles_m,
                       int num_tiles, int *err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *btiles = smem + STAGES * STAGE_BYTES;
    Bars *bars = reinterpret_cast<Bars *>(btiles + BSTAGES * B_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (k + BK - 1) / BK;
    volatile int *abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int b = 0; b < BSTAGES; ++b) {
            mbar_init(smem_u32(&bars->bready[b]), NUM_CONVERT_WARPS);
            mbar_init(smem_u32(&bars->bfree[b]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->acc_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), NUM_EPI_WARPS);
        }
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

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, err, 1);
                    if (!ok) break;
                    uint8_t *st = smem + stage * STAGE_BYTES;
                    const uint32_t full = smem_u32(&bars->full[stage]);
                    mbar_arrive_expect_tx(full, A_BYTES + WQ_BYTES);
                    tma_load_2d(smem_u32(st), &tmap_x, kb * BK, m0, full);
                    tma_load_2d(smem_u32(st + A_BYTES), &tmap_w, kb * BK, n0, full);
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
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0, acc = 0, bst = 0;
            uint32_t phase = 0, acc_phase = 0, bphase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase ^ 1, abort_flag, err, 2);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 3) &&
                         mbar_wait(smem_u32(&bars->bready[bst]), bphase, abort_flag, err, 4);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a_desc = make_kmajor_sw128_desc(smem_u32(smem + stage * STAGE_BYTES));
                    const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(btiles + bst * B_BYTES));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // +32 bytes per 16-element k step inside the 128-byte swizzle span
                        umma_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                                  IDESC, (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bars->empty[stage]));  // activations + int8 staging reusable
                    umma_commit(smem_u32(&bars->bfree[bst]));    // bf16 weight tile reusable
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    if (++bst == BSTAGES) { bst = 0; bphase ^= 1; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&bars->acc_full[acc]));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 2 + NUM_CONVERT_WARPS) {
        // ---------------- dequantizers: int8 staging -> swizzled bf16 ----------------
        const int ct = threadIdx.x - 64;          // 0..255
        const int chunk = ct & 3;                 // 16-byte chunk (16 k values) of the 64-byte row
        const int row0 = ct >> 2, sw = row0 & 7;  // row & 7 is the same for the thread's four rows
        const int off0 = ((2 * chunk) ^ sw) << 4, off1 = ((2 * chunk + 1) ^ sw) << 4;
        int stage = 0, bst = 0;
        uint32_t phase = 0, bphase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag, err, 5) &&
                     mbar_wait(smem_u32(&bars->bfree[bst]), bphase ^ 1, abort_flag, err, 7);
                if (!ok) break;
                // all four loads first (the stores below could alias them for the compiler), then
                // convert and store
                const uint4 *wq4 = reinterpret_cast<const uint4 *>(smem + stage * STAGE_BYTES + A_BYTES) + ct;
                uint4 v[BN / 64];
#pragma unroll
                for (int it = 0; it < BN / 64; ++it) v[it] = wq4[it * 256];
                uint8_t *rowp0 = btiles + bst * B_BYTES + (row0 >> 3) * 1024 + sw * 128;
#pragma unroll
                for (int it = 0; it < BN / 64; ++it) {
                    uint4 o0, o1;
                    cvt_i8x4_bf16(v[it].x, o0.x, o0.y);
                    cvt_i8x4_bf16(v[it].y, o0.z, o0.w);
                    cvt_i8x4_bf16(v[it].z, o1.x, o1.y);
                    cvt_i8x4_bf16(v[it].w, o1.z, o1.w);
                    uint8_t *rowp = rowp0 + it * 8 * 1024;  // 64 rows further = 8 groups of 8 rows
                    *reinterpret_cast<uint4 *>(rowp + off0) = o0;
                    *reinterpret_cast<uint4 *>(rowp + off1) = o1;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->bready[bst]));
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
                if (++bst == BSTAGES) { bst = 0; bphase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) belong to this warp
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool vec_ok = ((ldy & 3) == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
            ok = mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase, abort_flag, err, 6);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            float *yrow = y + (size_t)row * ldy;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                  (uint32_t)(acc * BN + c * 32), r);
                tmem_ld_wait();
                const int j0 = n0 + c * 32;
                if (row < m && j0 < n) {
                    if (vec_ok && j0 + 32 <= n) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const float4 sc = __ldg(reinterpret_cast<const float4 *>(scales + j0) + v);
                            float4 o;
                            o.x = __fmul_rn(__uint_as_float(r[4 * v + 0]), sc.x);
                            o.y = __fmul_rn(__uint_as_float(r[4 * v + 1]), sc.y);
                            o.z = __fmul_rn(__uint_as_float(r[4 * v + 2]), sc.z);
                            o.w = __fmul_rn(__uint_as_float(r[4 * v + 3]), sc.w);
                            if (bias) {
                                const float4 bv = __ldg(reinterpret_cast<const float4 *>(bias + j0) + v);
                                o.x = __fadd_rn(o.x, bv.x);
                                o.y = __fadd_rn(o.y, bv.y);
                                o.z = __fadd_rn(o.z, bv.z);
                                o.w = __fadd_rn(o.w, bv.w);
                            }
                            *reinterpret_cast<float4 *>(yrow + j0 + 4 * v) = o;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 32; ++v) {
                            const int j = j0 + v;
                            if (j < n) {
                                float o = __fmul_rn(__uint_as_float(r[v]), __ldg(scales + j));
                                if (bias) o = __fadd_rn(o, __ldg(bias + j));
                                yrow[j] = o;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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

// f32 -> bf16 (round to nearest even), 8 elements per thread.  n8 = element count / 8.
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(x) + 2 * i);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(x) + 2 * i + 1);
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t *>(&p0);
        o.y = *reinterpret_cast<uint32_t *>(&p1);
        o.z = *reinterpret_cast<uint32_t *>(&p2);
        o.w = *reinterpret_cast<uint32_t *>(&p3);
        reinterpret_cast<uint4 *>(out)[i] = o;
    }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

int make_map_2d(CUtensorMap *map, CUtensorMapDataType dt, size_t elem_bytes, const void *base,
                size_t inner, size_t outer, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(NNE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)(inner * elem_bytes)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(NNE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NNE_OK;
}

}  // namespace

int tma_make_map_2d(CUtensorMap *map, CUtensorMapDataType dt, size_t elem_bytes, const void *base,
                    size_t inner, size_t outer, uint32_t box_inner, uint32_t box_outer,
                    CUtensorMapSwizzle sw) {
    return make_map_2d(map, dt, elem_bytes, base, inner, outer, box_inner, box_outer, sw);
}

bool prefill_supports(const nne_qlinear *ql, size_t m) {
    if (!ql || !ql->tmap_w) return false;
    if (m == 0 || m > 0x7fffff00u) return false;
    return true;
}

int prefill_prepare_layer(nne_qlinear *ql) {
    ql->tmap_w = nullptr;
    // TMA needs 16-byte aligned rows: k % 16 == 0 covers both the int8 map (k bytes per row) and
    // the bf16 activations map (2k bytes per row).
    if (ql->n == 0 || ql->k == 0 || ql->k % 16 != 0) return NNE_OK;
    if (ql->n > 0x7fffff00u || ql->k > 0x7fffff00u) return NNE_OK;
    if ((reinterpret_cast<uintptr_t>(ql->q) & 15u) != 0) return NNE_OK;
    if (!encode_fn()) return NNE_OK;
    CUtensorMap *map = new CUtensorMap;
    int st = make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ql->q, ql->k, ql->n, BK, BN,
                         CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != NNE_OK) {
        delete map;
        return st;
    }
    ql->tmap_w = map;
    return NNE_OK;
}

void prefill_release_layer(nne_qlinear *ql) {
    if (ql->tmap_w) delete static_cast<CUtensorMap *>(ql->tmap_w);
    ql->tmap_w = nullptr;
}

int launch_prefill(nne_qlinear *ql, const float *x, float *y, size_t m, size_t ldy,
                   cudaStream_t s) {
    nne_ctx *ctx = ql->ctx;
    NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_kernel, SMEM_BYTES));
    // bf16 copy of the activations in a stream-ordered workspace (freed after the kernel).
    const size_t elems = m * ql->k;
    __nv_bfloat16 *xb = nullptr;
    NNE_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void **>(&xb), elems * sizeof(__nv_bfloat16), s));
    {
        const size_t n8 = elems / 8;  // k % 16 == 0
        size_t blocks = (n8 + 255) / 256;
        const size_t cap = (size_t)ctx->sm_count * 8;
        if (blocks > cap) blocks = cap;
        f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, xb, n8);
        NNE_LAUNCH_CHECK();
    }
    CUtensorMap tmap_x;
    int st = make_map_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xb, ql->k, m, BK, BM,
                         CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NNE_OK) {
        cudaFreeAsync(xb, s);
        return st;
    }
    const int tiles_m = (int)((m + BM - 1) / BM);
    const int tiles_n = (int)((ql->n + BN - 1) / BN);
    const long long tiles = (long long)tiles_m * tiles_n;
    if (tiles > 0x7fffffff) {
        cudaFreeAsync(xb, s);
        return fail(NNE_ERR_UNSUPPORTED, "too many output tiles");
    }
    int grid = ctx->sm_count;
    if (grid > tiles) grid = (int)tiles;
    qlinear_prefill_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(
        tmap_x, *static_cast<const CUtensorMap *>(ql->tmap_w), ql->scales, ql->bias, y, (int)m,
        (int)ql->n, (int)ql->k, ldy, tiles_m, (int)tiles, ctx->err_word);
    cudaError_t e = cudaGetLastError();
    count_launch();
    cudaFreeAsync(xb, s);
    if (e != cudaSuccess)
        return fail(NNE_ERR_CUDA, "prefill kernel launch failed: %s", cudaGetErrorString(e));
    return NNE_OK;
}

}  // namespace nne

// ---- forward without any allocation --------------------------------------------------------------
// Some callers must not allocate device memory while they run: a serving loop that handed its whole
// memory budget out at start-up, or a thread that issues work while a collective is in flight and
// cannot afford the device-wide synchronisation an allocation may imply.  For them the bf16 copy of
// the activations, which launch_prefill takes from a stream-ordered allocation, lives in this
// fixed array instead.  Every GPU that loads the library holds these 8 MiB until the process exits.
namespace nne {
namespace {

constexpr size_t STATIC_XBF16_ELEMS = (size_t)4 << 20;  // 4 Mi bf16 = 8 MiB: m * k may not exceed it
static __device__ __align__(256) __nv_bfloat16 g_static_xbf16[STATIC_XBF16_ELEMS];

// In host code `g_static_xbf16` is only a handle of the symbol, not a device address.  The address
// is looked up once per device, with that device current, and cached here.
std::mutex g_static_mu;
__nv_bfloat16 *g_static_ptr[64] = {nullptr};

int static_scratch_for(int device, __nv_bfloat16 **out) {
    if (device < 0 || device >= 64) return fail(NNE_ERR_UNSUPPORTED, "device ordinal %d too large", device);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_xbf16);  // the caller made `device` current
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(NNE_ERR_CUDA, "cudaGetSymbolAddress(g_static_xbf16) failed on device %d: %s",
                        device, cudaGetErrorString(e));
        }
        g_static_ptr[device] = static_cast<__nv_bfloat16 *>(p);
    }
    *out = g_static_ptr[device];
    return NNE_OK;
}

}  // namespace
}  // namespace nne

extern "C" int nne_qlinear_forward_dev_static(nne_qlinear *ql, const float *x_dev, size_t m, size_t k,
                                              float *y_dev, void *stream) {
    using namespace nne;
    NNE_GUARD_BEGIN
    if (!ql || !ql->ctx) return fail(NNE_ERR_INVALID_ARGUMENT, "null layer handle");
    if (k != ql->k)
        return fail(NNE_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%zu], got [%zu]", ql->k, k);
    if (m == 0 || ql->n == 0) return NNE_OK;
    if (!x_dev || !y_dev) return fail(NNE_ERR_INVALID_ARGUMENT, "null activation or output pointer");
    if (!ql->tmap_w || m > 0x7fffff00u || (reinterpret_cast<uintptr_t>(x_dev) & 15u) != 0)
        return fail(NNE_ERR_UNSUPPORTED,
                    "the allocation-free forward needs in_features %% 16 == 0 and 16-byte aligned x");
    size_t elems;
    if (__builtin_mul_overflow(m, k, &elems) || elems > STATIC_XBF16_ELEMS)
        return fail(NNE_ERR_INVALID_ARGUMENT,
                    "m * in_features = %zu * %zu exceeds the fixed workspace of %zu elements; use "
                    "nne_qlinear_forward_dev or split the batch",
                    m, k, STATIC_XBF16_ELEMS);
    nne_ctx *ctx = ql->ctx;
    NNE_TRY(use_ctx(ctx));
    __nv_bfloat16 *xb = nullptr;
    NNE_TRY(static_scratch_for(ctx->device, &xb));  // first call on a device: symbol look-up
    cudaStream_t s = (cudaStream_t)stream;
    NNE_TRY(ensure_dynamic_smem(ctx->device, qlinear_prefill_kernel, SMEM_BYTES));
    {
        // The pre-pass overwrites [0, m*k) of the workspace; nothing in it has to start at zero
        // and nothing beyond m*k is read (the tensor map below ends at row m).
        const size_t n8 = elems / 8;
        size_t blocks = (n8 + 255) / 256;
        const size_t cap = (size_t)ctx->sm_count * 8;
        if (blocks > cap) blocks = cap;
        f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, s>>>(x_dev, xb, n8);
        NNE_LAUNCH_CHECK();
    }
    CUtensorMap tmap_x;
    NNE_TRY(make_map_2d(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xb, ql->k, m, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B));
    const int tiles_m = (int)((m + BM - 1) / BM);
    const int tiles_n = (int)((ql->n + BN - 1) / BN);
    const long long tiles = (long long)tiles_m * tiles_n;
    if (tiles > 0x7fffffff) return fail(NNE_ERR_UNSUPPORTED, "too many output tiles");
    int grid = ctx->sm_count;
    if (grid > tiles) grid = (int)tiles;
    qlinear_prefill_kernel<<<grid, THREADS, SMEM_BYTES, s>>>(
        tmap_x, *static_cast<const CUtensorMap *>(ql->tmap_w), ql->scales, ql->bias, y_dev, (int)m,
        (int)ql->n, (int)ql->k, ql->n, tiles_m, (int)tiles, ctx->err_word);
    NNE_LAUNCH_CHECK();
    return NNE_OK;
    NNE_GUARD_END
}

