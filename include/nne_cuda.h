/*
 * nne_cuda.h - C ABI of the B200 (sm_100a) backend for the int8 quantized-linear path of
 * elvin-mark/neural-network-engine.
 *
 * This is the whole boundary a host language binds: plain pointers and sizes, no C++ or torch
 * types.  The reference has no FFI for this path today; every entry point below names the
 * reference item (path within the reference project : line) whose work it takes over, which
 * is what the Rust side `src/gpu/cuda/ffi.rs` declares in an `extern "C"` block.
 *
 * Conventions
 *  - Every function returns an nne_status (0 = OK).  No C++ exception crosses the boundary.
 *  - `*_host` buffers are ordinary host memory owned by the caller; the call returns after the
 *    result is in place.  `*_dev` buffers are device pointers on the context's device; the call
 *    is asynchronous on `stream` (a cudaStream_t passed as void*, NULL = the legacy default
 *    stream) and never synchronises.
 *  - Weights are [N, K] row-major (N = out_features, K = in_features, K contiguous), exactly
 *    the layout of `QLinear.qweight` (src/nn/quantized.rs:80-81).
 *  - A layer handle is immutable after creation, so concurrent forwards on one handle are
 *    safe as long as each call uses its own stream and its own x/y buffers.  `_host` forwards
 *    serialise on a per-context mutex.
 *  - There is no CPU fallback: without a usable sm_100 device every call fails with
 *    NNE_ERR_CUDA or NNE_ERR_UNSUPPORTED.
 */
#ifndef NNE_CUDA_H_
#define NNE_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NNE_API __attribute__((visibility("default")))
#else
#define NNE_API
#endif

/* Status codes.  The Rust side maps 1 -> EngineError::InvalidArgument (src/error.rs:41-42),
 * 2 -> EngineError::ShapeMismatch (src/error.rs:11-15), everything else ->
 * EngineError::GpuError(String) (src/error.rs:47-48) carrying nne_last_error's text. */
typedef enum nne_status {
    NNE_OK = 0,
    NNE_ERR_INVALID_ARGUMENT = 1,
    NNE_ERR_SHAPE_MISMATCH = 2,
    NNE_ERR_CUDA = 3,
    NNE_ERR_NCCL = 4,
    NNE_ERR_TIMEOUT = 5,
    NNE_ERR_OUT_OF_MEMORY = 6,
    NNE_ERR_UNSUPPORTED = 7
} nne_status;

typedef struct nne_ctx nne_ctx;         /* one per device: streams, staging, SM count   */
typedef struct nne_qlinear nne_qlinear; /* one device-resident int8 layer               */
typedef struct nne_plan nne_plan;       /* a fixed list of forwards run as one launch   */
typedef struct nne_shard_group nne_shard_group; /* one rank's end of a column-shard exchange */

/* ---- status text -------------------------------------------------------------------------- */

/* Static description of a status code. */
NNE_API const char *nne_status_string(int status);
/* Copies the calling thread's last error message (NUL-terminated, truncated to n) into buf.
 * Takes the place of the String inside EngineError::GpuError (src/error.rs:47-48). */
NNE_API int nne_last_error(char *buf, size_t n);

/* ---- context ------------------------------------------------------------------------------
 * Plays the role of Arc<GpuContext> of the existing device backend (src/gpu/context.rs:20-59,
 * src/gpu/layers.rs:12-16): created once, shared by every layer placed on that device.       */
/* Side effect on the process: creation raises the release threshold of the device's DEFAULT
 * stream-ordered memory pool to "keep everything" (cudaMemPoolAttrReleaseThreshold), so that the
 * forwards' stream-ordered workspaces are reused instead of returned to the driver at every
 * synchronisation.  A host application that shares that pool inherits the setting. */
NNE_API int nne_cuda_ctx_create(int device, nne_ctx **out);
NNE_API int nne_cuda_ctx_destroy(nne_ctx *ctx);
/* Synchronises the device and reads the context's device error word.  Kernels here never spin
 * without a limit: a wait that runs out (about 2 s) sets this word and the kernel returns.  Returns
 * NNE_ERR_TIMEOUT (and clears the word) if that happened since the last check, else NNE_OK.  The
 * `_host` entry points perform this check themselves. */
NNE_API int nne_cuda_ctx_check(nne_ctx *ctx);
/* Exercises the path from a wait that runs out to NNE_ERR_TIMEOUT without breaking anything: runs a
 * one-CTA kernel that waits, with a limit of `limit_us` microseconds, for an event that never
 * comes (which = 0: a shared-memory barrier nobody arrives at; which = 1: an arrival word of the
 * column-shard exchange that nothing raises).  The kernel gives up, sets the error word and
 * returns; the call returns NNE_OK, and the next nne_cuda_ctx_check reports NNE_ERR_TIMEOUT once.
 * The context stays usable.  No counterpart in the reference. */
NNE_API int nne_cuda_ctx_selftest_wait(nne_ctx *ctx, int which, unsigned int limit_us);
/* The streaming GEMV (m <= 2, and every plan it runs) is a persistent kernel with one CTA per SM;
 * a kernel of another library launched beside it (an NCCL collective on a second stream) finds no
 * SM with room for its CTAs and waits for it to end.  This leaves `count` SMs out of that kernel's
 * grid, so that the two overlap.  0 (the default) uses every SM.  No counterpart in the reference. */
NNE_API int nne_cuda_ctx_reserve_sms(nne_ctx *ctx, int count);
/* Device facts the host side sizes its work with.  Any out pointer may be NULL. */
NNE_API int nne_cuda_ctx_info(const nne_ctx *ctx, int *device, int *sm_count, int *cc_major,
                              int *cc_minor, size_t *total_mem_bytes);

/* ---- device buffers -------------------------------------------------------------------------
 * What a device tensor type on the host side needs, so that a stack of QLinears keeps its
 * activations on the GPU between layers: the counterparts of GpuTensor::from_slice's buffer and
 * queue.write_buffer (src/gpu/tensor.rs:19-44) and of GpuTensor::to_cpu (src/gpu/tensor.rs:53-95).
 * upload returns when the bytes are on the device; download first waits for ALL work issued on the
 * device (like to_cpu's device.poll(Wait)) and reports a timed-out kernel as NNE_ERR_TIMEOUT. */
NNE_API int nne_device_alloc(nne_ctx *ctx, size_t bytes, void **out_dev);
NNE_API int nne_device_free(nne_ctx *ctx, void *ptr_dev);
NNE_API int nne_device_upload(nne_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
NNE_API int nne_device_download(nne_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
/* The context's own stream (a cudaStream_t as void*), the one the *_host entry points use: device
 * forwards issued on it are ordered with them and with each other. */
NNE_API void *nne_cuda_ctx_stream(nne_ctx *ctx);

/* ---- quantize / dequantize ----------------------------------------------------------------
 * nne_quantize_rows replaces the row loop of QLinear::from_linear (src/nn/quantized.rs:107-127):
 * per row absmax, scale = max>0 ? max/127 : 1, inv = 1/scale, q = round_half_away(v*inv)
 * clamped to [-128,127], NaN -> 0.  Codes and scales are bit-identical to the reference.      */
NNE_API int nne_quantize_rows(nne_ctx *ctx, const float *w_host, size_t rows, size_t cols,
                              int8_t *q_host, float *scales_host);
NNE_API int nne_quantize_rows_dev(nne_ctx *ctx, const float *w_dev, size_t rows, size_t cols,
                                  int8_t *q_dev, float *scales_dev, void *stream);

/* nne_quantize_tensor replaces Int8Tensor::from_raw (src/nn/quantized.rs:32-57): ONE scale for
 * all n elements.  The _dev form needs a 4-byte device scratch word for the grid-wide absmax;
 * it is part of the context.  *scale_dev receives the f32 scale.                              */
NNE_API int nne_quantize_tensor(nne_ctx *ctx, const float *v_host, size_t n, int8_t *q_host,
                                float *scale_out);
NNE_API int nne_quantize_tensor_dev(nne_ctx *ctx, const float *v_dev, size_t n, int8_t *q_dev,
                                    float *scale_dev, void *stream);

/* nne_dequantize_rows replaces Int8Tensor::dequantize (src/nn/quantized.rs:60-67; rows = 1,
 * cols = n, one scale) and the weight loop of QLinear::to_linear (src/nn/quantized.rs:200-209;
 * one scale per row): out = (f32)q * scale[row].                                              */
NNE_API int nne_dequantize_rows(nne_ctx *ctx, const int8_t *q_host, const float *scales_host,
                                size_t rows, size_t cols, float *out_host);
NNE_API int nne_dequantize_rows_dev(nne_ctx *ctx, const int8_t *q_dev, const float *scales_dev,
                                    size_t rows, size_t cols, float *out_dev, void *stream);

/* ---- layer --------------------------------------------------------------------------------
 * nne_qlinear_create_from_f32 replaces QLinear::from_linear (src/nn/quantized.rs:92-141):
 * uploads the f32 weight [N,K] (and bias [N] or NULL), quantizes ON DEVICE and keeps codes,
 * scales and bias resident.  The _dev form takes device pointers (the f32 weight is not kept).
 * nne_qlinear_create_from_i8 builds the same handle from the public fields of an existing
 * QLinear (src/nn/quantized.rs:79-88), e.g. after Clone or a load from disk.                   */
NNE_API int nne_qlinear_create_from_f32(nne_ctx *ctx, const float *w_host,
                                        const float *bias_host_or_null, size_t n, size_t k,
                                        nne_qlinear **out);
NNE_API int nne_qlinear_create_from_f32_dev(nne_ctx *ctx, const float *w_dev,
                                            const float *bias_dev_or_null, size_t n, size_t k,
                                            void *stream, nne_qlinear **out);
NNE_API int nne_qlinear_create_from_i8(nne_ctx *ctx, const int8_t *q_host,
                                       const float *scales_host, const float *bias_host_or_null,
                                       size_t n, size_t k, nne_qlinear **out);
NNE_API int nne_qlinear_destroy(nne_qlinear *ql);

/* Fills the host copies the reference keeps as pub fields `qweight` and `scales`
 * (src/nn/quantized.rs:80-83; read by tests/nn/quantization_tests.rs:38-39).  Either pointer
 * may be NULL. */
NNE_API int nne_qlinear_download(const nne_qlinear *ql, int8_t *q_host, float *scales_host);
/* in_features / out_features / has_bias and the device pointers of the resident tensors. */
NNE_API int nne_qlinear_info(const nne_qlinear *ql, size_t *n, size_t *k, int *has_bias,
                             const int8_t **q_dev, const float **scales_dev,
                             const float **bias_dev);
/* QLinear::memory_bytes (src/nn/quantized.rs:230-237): N*K + 4N (+4N with bias). */
NNE_API size_t nne_qlinear_memory_bytes(const nne_qlinear *ql);

/* nne_qlinear_forward_host replaces the compute of QLinear::forward_quantized
 * (src/nn/quantized.rs:164-193) for an input already flattened to [m, k]:
 * y[r,j] = (sum_i x[r,i] * q[j,i]) * scales[j] (+ bias[j]).  `k` is the caller's last input
 * dimension and is checked against in_features as the reference does (:156-162), returning
 * NNE_ERR_SHAPE_MISMATCH.  m = 0 is valid and does nothing.  Copies x up, runs, copies y back.
 * Accuracy of every forward entry point below (unless it says otherwise): within
 *     1e-3 * ||x_r||inf * scale_j * sum_i |q[j,i]|
 * of the exact value, per element.  What the kernels actually do: each activation row is rounded to
 * a 16-bit grid (2^-15 of the row's largest |x|: at most 3 % of that tolerance, about 0.1-0.4 % of it
 * on random data); all products and sums are exact integers after that.  For m <= 16 a row's result
 * does not depend on which other rows are in the batch. */
NNE_API int nne_qlinear_forward_host(nne_qlinear *ql, const float *x_host, size_t m, size_t k,
                                     float *y_host);
/* Same contraction on device-resident x [m,k] and y [m,n], asynchronous on `stream`. */
NNE_API int nne_qlinear_forward_dev(nne_qlinear *ql, const float *x_dev, size_t m, size_t k,
                                    float *y_dev, void *stream);
/* Same, but writes y with a row stride of `ldy` floats (ldy >= n): used by a column shard to
 * write its slice straight into the gathered [m, N_total] layout. */
NNE_API int nne_qlinear_forward_dev_strided(nne_qlinear *ql, const float *x_dev, size_t m,
                                            size_t k, float *y_dev, size_t ldy, void *stream);

/* Forward that never allocates.  It has no counterpart in the reference.  Meant for callers that
 * may not allocate device memory while they run - a serving loop whose memory budget was handed
 * out in full at start-up, or a thread that issues work while a collective is in flight and
 * cannot risk the device-wide synchronisation an allocation can bring.  Same contraction as
 * nne_qlinear_forward_dev, but with a LOOSER error bound: it always runs the bf16 tensor-core
 * kernel (codes dequantized to bf16 in shared memory - exact - and activations rounded to bf16,
 * fp32 accumulation), so per output channel j
 *     |y - exact| <= 2^-8 * ||x||inf * scale_j * sum_k |q_jk|   (+ fp32 summation error),
 * i.e. up to 3.9 times the 1e-3 tolerance nne_qlinear_forward_dev keeps; on N(0,1)
 * activations the rounding errors average out to a few percent of that tolerance, and on
 * activations that are exact in bf16 the result equals nne_qlinear_forward_dev's bit for bit.
 * The bf16 copy of the activations lives in a fixed 8 MiB array in the library's device image
 * (every GPU that loads the library holds it until the process exits) instead of a stream-ordered
 * allocation.  Limits: in_features % 16 == 0, x_dev 16-byte aligned, and m * in_features <=
 * 4 194 304 (4 Mi elements); anything larger is refused with NNE_ERR_INVALID_ARGUMENT and a
 * message naming the limit.  The first call on a device looks the array's address up
 * (cudaGetSymbolAddress); make that first call before any stream capture begins.  All calls on
 * a device share the one array and it keeps the last call's contents, so two calls whose kernels
 * can overlap on the GPU (different streams, no dependency) race: keep them on one stream or order
 * them with events.  Calls no cudaMalloc/cudaFree or other allocating routine.                   */
NNE_API int nne_qlinear_forward_dev_static(nne_qlinear *ql, const float *x_dev, size_t m, size_t k,
                                           float *y_dev, void *stream);

/* ---- plan: several forwards as one launch ----------------------------------------------------
 * A plan fixes a list of `count` forwards y_i[m, n_i] = QLinear_i.forward(x_i[m, k_i]) on device
 * buffers that stay in place, and nne_qlinear_plan_run issues all of them on `stream`.  It takes
 * the place of the back-to-back QLinear::forward calls a caller makes on projections that do
 * not depend on each other - q/k/v (src/models/llama.rs:226-228), gate/up
 * (src/models/llama.rs:344-346), or the per-layer timing loop of the decode benchmark - each
 * of which is the contraction of src/nn/quantized.rs:164-193.  For m = 1 and streaming-capable
 * shapes the whole list is ONE kernel launch whose weight stream never drains between layers;
 * for 2 <= m <= 16 it is one pre-pass and one launch of the small-batch tensor-core kernel over
 * all layers (layers given the same x pointer share one set of digit planes; the work areas are
 * allocated at creation, so a run allocates nothing; a plan must not run concurrently with
 * itself); otherwise the plan runs its layers one after the other.  Results are identical to
 * `count` calls of nne_qlinear_forward_dev.  Layers must outlive the plan.
 *
 * Items may also depend on one another: where an item reads a buffer an earlier item of the list
 * writes (or writes one an earlier item reads or writes), the plan orders them - the list behaves
 * like `count` forwards issued one after another on a stream.  The dependencies are found from the
 * pointers when the plan is created.  For m = 1 on streaming shapes the whole list is still ONE
 * launch: the grid meets between dependent layers (an arrival counter in device memory, bounded
 * wait, cooperative launch) while the weight stream runs on into the next layer's rows; the
 * counter carries over from run to run, so such a plan may be captured in a CUDA graph and
 * replayed, but must not run concurrently with itself.  Other sizes run the independent groups one
 * after another.  An item whose output overlaps one of its own inputs is refused
 * (NNE_ERR_INVALID_ARGUMENT), except a residual that is the output buffer itself.  After
 * NNE_ERR_TIMEOUT a plan with dependent items must be destroyed (its counter is left mid-count). */
NNE_API int nne_qlinear_plan_create(nne_ctx *ctx, size_t count, nne_qlinear *const *layers,
                                    const float *const *x_dev, float *const *y_dev, size_t m,
                                    nne_plan **out);
NNE_API int nne_qlinear_plan_run(nne_plan *plan, void *stream);
/* The same run with HOST activations and outputs: x_all_host holds the x_i one after another
 * (m * k_i floats each, list order), y_all_host receives the y_i one after another (m * n_i
 * floats each).  Copies them to and from the plan's device buffers (one copy per run of buffers
 * that continue one another in device memory, so a plan built over one x slab and one y slab
 * costs one copy each way), runs the plan on the context's stream and returns when y_all_host is
 * complete.  When both slabs are pinned host memory (cudaHostAlloc / cudaHostRegister), hold at most
 * 1 MiB together and the runs are 16-byte aligned multiples of four floats (nne_qlinear_forward_host
 * does the same for its x and y), the copies are done by two small kernels instead of
 * the copy engines: they chain with the forward kernels by programmatic dependent launch, so the
 * weight stream starts while x is still crossing PCIe (about a tenth off the round trip of a
 * 12-layer decode step).  In a list with dependent items (above) the part of x_all_host that belongs
 * to an item fed by an earlier item is uploaded like the rest and then overwritten on the device by
 * that item's result: its contents do not matter.  Serialised per context like the other *_host
 * entry points.  The reference has no
 * counterpart; it is what a caller of QLinear::forward on several independent projections
 * (q/k/v: src/models/llama.rs:226-228) gets instead of one host round trip per projection. */
NNE_API int nne_qlinear_plan_run_host(nne_plan *plan, const float *x_all_host, float *y_all_host);
NNE_API int nne_qlinear_plan_destroy(nne_plan *plan);
/* 1 when the whole list runs as one streaming launch, 2 when it runs as pre-pass + small-batch
 * kernel, else the number of layers (each then runs its own forward, of one or two launches). */
NNE_API int nne_qlinear_plan_launches(const nne_plan *plan);

/* ---- the steps either side of a QLinear in a decoder block ------------------------------------
 * RMSNorm over the last dimension, y = (x * rrms) * gamma with rrms = 1 / sqrt(mean(x^2) + eps)
 * (src/nn/norm.rs:141-165, row function :517-577); SwiGLU's element-wise step
 * out = silu(gate) * up, silu(v) = v / (1 + exp(-v)) (src/models/llama.rs:343-346,
 * src/tensor/ops.rs:177-179); the residual add out = a + b (src/models/llama.rs:377-392).
 * Device pointers, asynchronous on `stream`.  fp32, within 1e-5 relative of the reference's
 * results (the sum of squares is taken in another order).  out may alias an input. */
NNE_API int nne_rmsnorm_dev(nne_ctx *ctx, const float *x_dev, const float *gamma_dev, float eps,
                            size_t rows, size_t cols, float *y_dev, void *stream);
NNE_API int nne_silu_mul_dev(nne_ctx *ctx, const float *gate_dev, const float *up_dev, size_t n,
                             float *out_dev, void *stream);
NNE_API int nne_add_dev(nne_ctx *ctx, const float *a_dev, const float *b_dev, size_t n, float *out_dev,
                        void *stream);

/* A plan whose forwards take those steps in their stride.  Item i computes
 *     y = layer.forward(x') (+ residual),   x' = x | RMSNorm(x; gamma, eps) | silu(x) * x2,
 * which is how the QLinears of a LLaMA block meet their neighbours: q/k/v and gate/up read
 * RMSNorm(h) (src/models/llama.rs:377-392), down reads silu(gate) * up (:343-346), o and down add
 * the residual stream.  For m <= 2 on streaming shapes the decode kernel applies the transform while
 * it prepares the activations and adds the residual as it stores, so a chain of such plans never
 * leaves the device and launches nothing but the forwards; for other shapes the plan runs the
 * standalone kernels above around its forwards (into buffers it owns).  Results equal the
 * standalone kernels followed by nne_qlinear_forward_dev bit for bit in the second case and within
 * 1e-5 relative in the first (rrms is summed in another order).  Items may consume earlier items'
 * outputs (see above): a whole decoder block - or a whole stack of them - can be one plan, and at
 * m = 1 one launch. */
enum { NNE_INPUT_PLAIN = 0, NNE_INPUT_RMSNORM = 1, NNE_INPUT_SILU_MUL = 2 };
typedef struct nne_plan_item {
    nne_qlinear *layer;
    const float *x;        /* [m, in_features] */
    float *y;              /* [m, out_features] */
    int input_op;          /* NNE_INPUT_* */
    float eps;             /* RMSNORM */
    const float *gamma;    /* RMSNORM: [in_features] */
    const float *x2;       /* SILU_MUL: [m, in_features] (the "up" half; x is the "gate" half) */
    const float *residual; /* NULL, or [m, out_features] added to the forward's result */
} nne_plan_item;
NNE_API int nne_qlinear_plan_create_fused(nne_ctx *ctx, size_t count, const nne_plan_item *items,
                                          size_t m, nne_plan **out);

/* ---- column shards over the GPUs of one node -------------------------------------------------
 * The reference has no multi-device code.  Its forward computes output channel j from row j of
 * qweight, scales[j] and bias[j] alone (src/nn/quantized.rs:184-192) and quantizes per row
 * (:107-127), so rank g of G can own the rows [b_g, e_g) of a layer as an ordinary nne_qlinear
 * (bit-identical codes) and compute columns [b_g, e_g) of y [m, n_total]; every rank then needs all
 * columns - an all-gather of the output slices.
 *
 * A shard group is one rank's end of that exchange: one process per GPU (handles exchanged by any
 * transport) or one process driving several devices.  It owns a WINDOW of device memory which every
 * peer maps.  Gathered outputs live at the same offset in every rank's window.  Two routes:
 *   route 0, peer stores: a split-phase exchange.  nne_qlinear_plan_run only produces: the decode
 *            kernel (m <= 2 on streaming shapes) stores each result into all G windows itself; for
 *            other shapes a copy kernel pushes the slice out after the local forward.  Ordinary
 *            stores to peer-mapped memory; the run neither announces itself nor waits for anybody.
 *            nne_shard_group_wait completes it: it enqueues a one-warp kernel that announces this
 *            rank's runs issued so far in every window and returns once every rank has announced as
 *            many, i.e. once this rank's window holds every slice (bounded: about 2 s, then
 *            NNE_ERR_TIMEOUT through nne_cuda_ctx_check).  EVERY rank must call it for its runs - a
 *            rank that does not is never heard of.  Put it on a stream ordered after the runs:
 *            the run's own stream, before the reader of the gathered output; or a second stream
 *            (after an event), where it overlaps the next run.  nne_qlinear_plan_run_host does run,
 *            wait and copy-back itself.
 *   route 1, NCCL:  ncclAllGather on a communicator the host created (nne_shard_group_set_nccl),
 *            on the run's stream; needs equal slices in rank order.  m = 1 gathers in place; m > 1
 *            gathers [m, width] blocks into a staging area and interleaves them into row-major
 *            [m, n_total].  nne_shard_group_wait is not needed (and harmless).
 * Rules, as for collectives: all ranks issue the same sequence of sharded runs and waits on a
 * group, and a rank issues them on ONE stream (or orders them with events): a run announces the
 * rank's previous run as complete.  A rank
 * may overwrite an output area only when every peer has finished reading what it held: with run,
 * wait and the reads in ONE stream two alternating areas are enough ("a peer has signalled run e+1"
 * implies "it has read run e"); a caller that keeps d runs in flight before it waits needs 2 d areas.
 * A group holds at most 8 ranks.  No multicast object and no TMA access to peer memory is used. */
#define NNE_SHARD_HANDLE_BYTES 64
/* Allocates this rank's window of `window_bytes` (zero-filled; cudaMalloc, so it can be exported). */
NNE_API int nne_shard_group_create(nne_ctx *ctx, int rank, int world, size_t window_bytes,
                                   nne_shard_group **out);
/* Writes the NNE_SHARD_HANDLE_BYTES-byte handle other PROCESSES need to map this window. */
NNE_API int nne_shard_group_handle(const nne_shard_group *group, void *handle_out);
/* all_handles: world x NNE_SHARD_HANDLE_BYTES bytes in rank order (the own entry is ignored). */
NNE_API int nne_shard_group_connect(nne_shard_group *group, const void *all_handles);
/* One process driving all devices: all_groups[p] is rank p's group (peer access is enabled). */
NNE_API int nne_shard_group_connect_local(nne_shard_group *group, nne_shard_group *const *all_groups);
/* The window: device pointer and usable size. */
NNE_API int nne_shard_group_window(const nne_shard_group *group, void **base, size_t *bytes);
/* Completes every sharded run issued on this group so far (route 0): announce, then wait. */
NNE_API int nne_shard_group_wait(nne_shard_group *group, void *stream);
/* ncclComm_t (as void*) of this rank, created by the host, for route 1.  The library calls the
 * NCCL copy the process has loaded (or the one NNE_NCCL_LIB names); it does not link NCCL. */
NNE_API int nne_shard_group_set_nccl(nne_shard_group *group, void *nccl_comm);
/* Unmaps the peers' windows and frees this rank's.  Call it when no rank can still store into this
 * window or read a mapping of it (after a barrier of the host's own making). */
NNE_API int nne_shard_group_destroy(nne_shard_group *group);
/* A plan over column shards: shards[i] holds rows [row_begin[i], row_begin[i] + shards[i].n) of a
 * layer with n_total[i] output channels; x_dev[i] is [m, k_i] (replicated on every rank, anywhere
 * in device memory); y_full_dev[i] is the gathered output [m, n_total[i]] INSIDE this rank's window,
 * at the same window offset on every rank.  nne_qlinear_plan_run runs the forwards and the
 * exchange; nne_qlinear_plan_run_host returns the gathered outputs (m * n_total[i] floats each).
 * A group of one rank runs like an ordinary plan.  Destroy with nne_qlinear_plan_destroy. */
NNE_API int nne_qlinear_plan_create_sharded(nne_shard_group *group, size_t count,
                                            nne_qlinear *const *shards, const size_t *row_begin,
                                            const size_t *n_total, const float *const *x_dev,
                                            float *const *y_full_dev, size_t m, int route,
                                            nne_plan **out);

/* Which kernel a forward of m rows on this layer dispatches to: 1 = streaming GEMV (small m),
 * 2 = tcgen05/TMEM tensor-core kernel (integer form; NNE_PREFILL=bf16 in the environment selects
 * the bf16 form), 3 = generic kernel for shapes the others do not take, 4 = small-batch
 * tensor-core kernel (3 <= m <= 16: int8 weights as the MMA's M side, read once; bit-identical per
 * row to kernel 1; NNE_SKINNY=0 in the environment sends these sizes to kernel 1 instead). */
NNE_API int nne_qlinear_kernel_for(const nne_qlinear *ql, size_t m);
/* Number of kernels this library has launched in the calling process (all contexts). */
NNE_API uint64_t nne_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NNE_CUDA_H_ */
