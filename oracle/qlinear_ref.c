/*
 * CPU oracle for the int8 quantized-linear path of elvin-mark/neural-network-engine.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is a plain-C restatement of the
 * arithmetic in the reference file src/nn/quantized.rs.  Only the test-suite, the smoke
 * check and the CPU-baseline leg of the benchmark may load it; the CUDA library never does.
 *
 * PARITY UNPINNED: the reference is a Rust crate, no Rust toolchain exists where this is
 * built, and the reference's own tests for this path (tests/nn/quantization_tests.rs) hold
 * no golden vectors, only statistical thresholds on unseeded random inputs.  The pins that do
 * exist are (1) those four thresholds, replayed on seeded inputs by the CPU test-suite,
 * (2) an independent numpy restatement of the quantize step that must agree byte for byte, and
 * (3) an independent numpy restatement of the forward's AVX2 dot product (lane order, horizontal
 * sums, scalar tail, with an exactly emulated fused multiply-add) that must agree bit for bit.
 * Two restatements that agree are still not the reference running: parity stays unpinned.
 *
 * Each function cites the reference lines it follows (path within the reference project).
 *
 * Build (see oracle/Makefile): gcc -O2 -ffp-contract=off -fno-fast-math.  The file is built
 * WITHOUT -mavx2/-mfma so the scalar code can never be contracted into FMAs; only the one
 * function that restates the AVX2 kernel carries a target attribute, as the reference does
 * with #[target_feature(enable = "avx2,fma")].
 */
#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NNE_REF_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * Deterministic synthetic inputs.  The reference draws its test inputs from an unseeded
 * thread_rng (src/tensor/mod.rs:110-125), so it defines no reproducible stream; this
 * counter-based generator is this build's own and is shared by every test and bench leg.
 * element i of stream (seed, stream) = mean + std * z_i,  z_i = sqrt(-2 ln u1) cos(2 pi u2),
 * u1 = (splitmix64(key + 2i) >> 11 + 1) / 2^53 in (0,1],  u2 = (splitmix64(key + 2i + 1) >> 11) / 2^53.
 * ---------------------------------------------------------------------------------------- */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

NNE_REF_API uint64_t nne_ref_stream_key(uint64_t seed, uint64_t stream) {
    return splitmix64(splitmix64(seed) ^ (0xD1B54A32D192ED03ull * (stream + 1)));
}

NNE_REF_API void nne_ref_fill_normal(uint64_t seed, uint64_t stream, double mean, double std,
                                     size_t n, float *out) {
    const uint64_t key = nne_ref_stream_key(seed, stream);
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = 0; i < n; ++i) {
        uint64_t a = splitmix64(key + 2 * (uint64_t)i);
        uint64_t b = splitmix64(key + 2 * (uint64_t)i + 1);
        double u1 = (double)((a >> 11) + 1) * (1.0 / 9007199254740992.0);
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
        double z = sqrt(-2.0 * log(u1)) * cos(two_pi * u2);
        out[i] = (float)(mean + std * z);
    }
}

/* ------------------------------------------------------------------------------------------
 * Rust's `(t).round().clamp(-128.0, 127.0) as i8`  (src/nn/quantized.rs:48 and :124).
 * f32::round is round-half-away-from-zero (roundf).  clamp keeps NaN; `as i8` maps NaN to 0
 * and saturates, so after the clamp only the NaN case needs care.
 * ---------------------------------------------------------------------------------------- */
static inline int8_t round_clamp_i8(float t) {
    float r = roundf(t);
    if (r != r) return 0; /* NaN -> 0 */
    if (r < -128.0f) r = -128.0f;
    if (r > 127.0f) r = 127.0f;
    return (int8_t)r;
}

/* absmax exactly as the reference writes it: `let a = v.abs(); if a > max_abs { max_abs = a }`
 * (src/nn/quantized.rs:35-41 and :111-117).  A NaN never compares greater, so it never wins. */
static inline float absmax_f32(const float *v, size_t n) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(v[i]);
        if (a > max_abs) max_abs = a;
    }
    return max_abs;
}

/* Int8Tensor::from_raw, src/nn/quantized.rs:32-57: one scale for the whole tensor. */
NNE_REF_API void nne_ref_int8tensor_from_raw(const float *values, size_t n, int8_t *data,
                                             float *scale_out) {
    float max_abs = absmax_f32(values, n);
    float scale = (max_abs > 0.0f) ? max_abs / 127.0f : 1.0f; /* :43 */
    float inv_scale = 1.0f / scale;                            /* :44 */
    float inv = inv_scale;
    for (size_t i = 0; i < n; ++i) data[i] = round_clamp_i8(values[i] * inv); /* :48 */
    *scale_out = scale;
}

/* Int8Tensor::dequantize, src/nn/quantized.rs:60-67: q as f32 * scale. */
NNE_REF_API void nne_ref_dequantize(const int8_t *data, size_t n, float scale, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = (float)data[i] * scale;
}

/* QLinear::from_linear, src/nn/quantized.rs:107-127: one scale per output row.  The bias copy
 * at :129-132 is a plain memcpy and is left to the caller. */
NNE_REF_API void nne_ref_quantize_rows(const float *w, size_t rows, size_t cols, int8_t *qweight,
                                       float *scales) {
    for (size_t row = 0; row < rows; ++row) {
        const float *row_slice = w + row * cols;
        float max_abs = absmax_f32(row_slice, cols);                            /* :110-117 */
        float scale = (max_abs > 0.0f) ? max_abs / 127.0f : 1.0f;     /* :119 */
        float inv_scale = 1.0f / scale;                                /* :120 */
        float inv = inv_scale;
        scales[row] = scale;                                                    /* :121 */
        int8_t *q = qweight + row * cols;
        for (size_t c = 0; c < cols; ++c) q[c] = round_clamp_i8(row_slice[c] * inv); /* :123-126 */
    }
}

/* QLinear::to_linear, src/nn/quantized.rs:200-209: q as f32 * scales[row]. */
NNE_REF_API void nne_ref_to_linear(const int8_t *qweight, const float *scales, size_t rows,
                                   size_t cols, float *w_out) {
    for (size_t row = 0; row < rows; ++row) {
        float scale = scales[row];
        for (size_t c = 0; c < cols; ++c)
            w_out[row * cols + c] = (float)qweight[row * cols + c] * scale;
    }
}

/* QLinear::memory_bytes, src/nn/quantized.rs:230-237. */
NNE_REF_API size_t nne_ref_qlinear_memory_bytes(size_t out_features, size_t in_features,
                                                int has_bias) {
    return out_features * in_features + out_features * sizeof(float) +
           (has_bias ? out_features * sizeof(float) : 0);
}

/* Portable dot, src/nn/quantized.rs:266-271: left to right, separate multiply and add. */
NNE_REF_API float nne_ref_dot_f32_i8_scalar(const float *x, const int8_t *w, size_t len) {
    float sum = 0.0f;
    for (size_t i = 0; i < len; ++i) {
        float p = x[i] * (float)w[i];
        sum = sum + p;
    }
    return sum;
}

/* dot_f32_i8_avx2, src/nn/quantized.rs:274-324.  Two 8-lane accumulators, element i of each
 * 16-block goes to lane i%16, FMA per block (:299-300); then acc0+acc1 (:305), lo128+hi128
 * (:308-310), movehdup add (:311-312), movehl add_ss (:313-314); scalar tail with separate
 * multiply and add (:318-321). */
__attribute__((target("avx2,fma"))) NNE_REF_API float
nne_ref_dot_f32_i8_avx2(const float *x, const int8_t *w, size_t len) {
    size_t i = 0;
    __m256 acc0 = _mm256_setzero_ps();
    __m256 acc1 = _mm256_setzero_ps();
    while (i + 16 <= len) {
        __m256 x0 = _mm256_loadu_ps(x + i);
        __m256 x1 = _mm256_loadu_ps(x + i + 8);
        __m128i w0 = _mm_loadl_epi64((const __m128i *)(w + i));
        __m128i w1 = _mm_loadl_epi64((const __m128i *)(w + i + 8));
        __m256 wf0 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(w0));
        __m256 wf1 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(w1));
        acc0 = _mm256_fmadd_ps(x0, wf0, acc0);
        acc1 = _mm256_fmadd_ps(x1, wf1, acc1);
        i += 16;
    }
    __m256 acc = _mm256_add_ps(acc0, acc1);
    __m128 hi128 = _mm256_extractf128_ps(acc, 1);
    __m128 lo128 = _mm256_castps256_ps128(acc);
    __m128 sum128 = _mm_add_ps(lo128, hi128);
    __m128 shuf = _mm_movehdup_ps(sum128);
    __m128 sums = _mm_add_ps(sum128, shuf);
    __m128 shuf2 = _mm_movehl_ps(sums, sums);
    __m128 final_sum = _mm_add_ss(sums, shuf2);
    float total = _mm_cvtss_f32(final_sum);
    while (i < len) {
        float p = x[i] * (float)w[i];
        total = total + p;
        i += 1;
    }
    return total;
}

/* dot_f32_i8 dispatch, src/nn/quantized.rs:253-272: AVX2+FMA when the CPU has both. */
NNE_REF_API int nne_ref_has_avx2_fma(void) {
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}

static inline float dot_dispatch(const float *x, const int8_t *w, size_t len, int use_avx2) {
    return use_avx2 ? nne_ref_dot_f32_i8_avx2(x, w, len) : nne_ref_dot_f32_i8_scalar(x, w, len);
}

/* One task of the reference's row split: the closure body at src/nn/quantized.rs:182-193. */
static void forward_row(const int8_t *qweight, const float *scales, const float *bias, size_t n,
                        size_t k, const float *x_row, float *out_row, int use_avx2) {
    for (size_t j = 0; j < n; ++j) {
        float dot = dot_dispatch(x_row, qweight + j * k, k, use_avx2); /* :185-186 */
        float val = dot * scales[j];                          /* :187 */
        if (bias) val = val + bias[j];                                 /* :188-190 */
        out_row[j] = val;                                              /* :191 */
    }
}

typedef struct {
    const int8_t *qweight;
    const float *scales;
    const float *bias;
    size_t n, k, m;
    const float *x;
    float *y;
    int use_avx2;
    size_t next_row; /* shared work counter: rows are claimed one at a time, like rayon tasks */
    pthread_mutex_t lock;
} fwd_job;

static void *fwd_worker(void *arg) {
    fwd_job *job = (fwd_job *)arg;
    for (;;) {
        pthread_mutex_lock(&job->lock);
        size_t r = job->next_row++;
        pthread_mutex_unlock(&job->lock);
        if (r >= job->m) break;
        forward_row(job->qweight, job->scales, job->bias, job->n, job->k, job->x + r * job->k,
                    job->y + r * job->n, job->use_avx2);
    }
    return NULL;
}

/* QLinear::forward_quantized, src/nn/quantized.rs:146-197, after validation and flattening to
 * [m, k].  The reference runs one rayon task per input ROW (:179-182) and nothing finer, so
 * at most min(m, threads) host threads can ever be busy; `threads` <= 0 means 1.
 * use_avx2: 1 = the AVX2/FMA dot (:276), 0 = the portable dot (:267), -1 = runtime detect as
 * the reference does (:257-264).  Returns the number of threads that were started. */
NNE_REF_API int nne_ref_forward(const int8_t *qweight, const float *scales, const float *bias,
                                size_t n, size_t k, const float *x, size_t m, float *y,
                                int threads, int use_avx2) {
    if (use_avx2 < 0) use_avx2 = nne_ref_has_avx2_fma();
    if (m == 0 || n == 0) return 0;
    if (threads <= 0) threads = 1;
    if ((size_t)threads > m) threads = (int)m;
    if (threads == 1) {
        for (size_t r = 0; r < m; ++r)
            forward_row(qweight, scales, bias, n, k, x + r * k, y + r * n, use_avx2);
        return 1;
    }
    fwd_job job = {qweight, scales, bias, n, k, m, x, y, use_avx2, 0, PTHREAD_MUTEX_INITIALIZER};
    pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    int started = 0;
    for (int t = 0; t < threads - 1; ++t)
        if (pthread_create(&tids[started], NULL, fwd_worker, &job) == 0) ++started;
    fwd_worker(&job);
    for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
    free(tids);
    return started + 1;
}

/* The same contraction in double precision, as ground truth beside the f32 orders above:
 * y = (sum_k x*q) * scale + bias with every step in double.  Not a reference code path. */
NNE_REF_API void nne_ref_forward_f64(const int8_t *qweight, const float *scales,
                                     const float *bias, size_t n, size_t k, const float *x,
                                     size_t m, double *y) {
    for (size_t r = 0; r < m; ++r)
        for (size_t j = 0; j < n; ++j) {
            double s = 0.0;
            const int8_t *w = qweight + j * k;
            const float *xr = x + r * k;
            for (size_t i = 0; i < k; ++i) s += (double)xr[i] * (double)w[i];
            s *= (double)scales[j];
            if (bias) s += (double)bias[j];
            y[r * n + j] = s;
        }
}

/* Per-channel tolerance the build is held to: tol_j = 1e-3 * ||x||_inf * scale_j * sum_k |q_jk|,
 * i.e. one thousandth of the a-priori bound on |y_j - b_j|.  Returns ||x||_inf. */
NNE_REF_API float nne_ref_tolerance(const int8_t *qweight, const float *scales, size_t n,
                                    size_t k, const float *x, size_t m, float *tol) {
    float xinf = 0.0f;
    for (size_t i = 0; i < m * k; ++i) {
        float a = fabsf(x[i]);
        if (a > xinf) xinf = a;
    }
    for (size_t j = 0; j < n; ++j) {
        uint64_t s = 0;
        for (size_t i = 0; i < k; ++i) s += (uint64_t)abs((int)qweight[j * k + i]);
        tol[j] = (float)(1e-3 * (double)xinf * (double)scales[j] * (double)s);
    }
    return xinf;
}

/* ------------------------------------------------------------------------------------------
 * The element-wise steps either side of a QLinear in a LLaMA block (the "next" rows of the path):
 * RMSNorm (src/nn/norm.rs:100-180, row function :517-577) and SwiGLU's silu(gate) * up
 * (src/models/llama.rs:343-346 with RawTensor::silu, src/tensor/ops.rs:177-179).
 * ---------------------------------------------------------------------------------------- */

/* hsum256, src/nn/norm.rs:412-421: (lo128 + hi128), then (s0+s2, s1+s3), then lane0 + lane1. */
__attribute__((target("avx2,fma"))) static float ref_hsum256(__m256 v) {
    __m128 v_high = _mm256_extractf128_ps(v, 1);
    __m128 v_low = _mm256_castps256_ps128(v);
    __m128 sum128 = _mm_add_ps(v_low, v_high);
    __m128 shuf = _mm_movehl_ps(sum128, sum128);
    __m128 sum64 = _mm_add_ps(sum128, shuf);
    __m128 shuf2 = _mm_shuffle_ps(sum64, sum64, 1);
    __m128 sum32 = _mm_add_ss(sum64, shuf2);
    return _mm_cvtss_f32(sum32);
}

/* fused_rms_norm_row_avx2, src/nn/norm.rs:539-577: 8 lane accumulators with FMA, hsum, scalar
 * tail with separate multiply and add, rrms = 1 / sqrt(sum/d + eps), out = (x * rrms) * gamma. */
__attribute__((target("avx2,fma"))) static void ref_rms_norm_row_avx2(const float *x, const float *gamma,
                                                                       float eps, size_t d, float *out) {
    __m256 acc_sq = _mm256_setzero_ps();
    size_t i = 0;
    while (i + 8 <= d) {
        __m256 vx = _mm256_loadu_ps(x + i);
        acc_sq = _mm256_fmadd_ps(vx, vx, acc_sq);
        i += 8;
    }
    float sum_sq = ref_hsum256(acc_sq);
    while (i < d) {
        float v = x[i];
        float p = v * v;
        sum_sq = sum_sq + p;
        i += 1;
    }
    float mean_sq = sum_sq / (float)d;
    float rrms = 1.0f / sqrtf(mean_sq + eps);
    for (i = 0; i < d; ++i) {
        float t = x[i] * rrms;
        out[i] = t * gamma[i];
    }
}

/* fused_rms_norm_row, portable branch, src/nn/norm.rs:528-534: left-to-right sum of squares. */
static void ref_rms_norm_row_scalar(const float *x, const float *gamma, float eps, size_t d, float *out) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < d; ++i) {
        float p = x[i] * x[i];
        sum_sq = sum_sq + p;
    }
    float mean_sq = sum_sq / (float)d;
    float rrms = 1.0f / sqrtf(mean_sq + eps);
    for (size_t i = 0; i < d; ++i) {
        float t = x[i] * rrms;
        out[i] = t * gamma[i];
    }
}

/* RMSNorm::forward, no-grad fast path (src/nn/norm.rs:141-165): one row function per row.
 * use_avx2: -1 = detect like the reference (:520), 0 = portable, 1 = AVX2. */
NNE_REF_API void nne_ref_rms_norm(const float *x, const float *gamma, float eps, size_t rows, size_t d,
                                  float *out, int use_avx2) {
    int avx = use_avx2 < 0 ? nne_ref_has_avx2_fma() : use_avx2;
    for (size_t r = 0; r < rows; ++r) {
        if (avx)
            ref_rms_norm_row_avx2(x + r * d, gamma, eps, d, out + r * d);
        else
            ref_rms_norm_row_scalar(x + r * d, gamma, eps, d, out + r * d);
    }
}

/* SwiGLU's element-wise step (src/models/llama.rs:343-346): silu(gate) * up with
 * silu(x) = x / (1 + exp(-x)) (src/tensor/ops.rs:177-179). */
NNE_REF_API void nne_ref_silu_mul(const float *gate, const float *up, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) {
        float g = gate[i];
        float s = g / (1.0f + expf(-g));
        out[i] = s * up[i];
    }
}
