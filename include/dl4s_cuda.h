/*
 * dl4s_cuda.h — C ABI of libdl4s_cuda.so, an sm_100a (NVIDIA B200) back-end
 * for the scaled-dot-product-attention path of palle-k/DL4S.
 *
 * The library is what a new `CUDA: DeviceType` in DL4S binds to: a SwiftPM C
 * target whose module map lists this header and `link "dl4s_cuda"`, exactly as
 * Sources/MKL/include/module.modulemap does for MKL. Each entry point names the
 * DL4S requirement it implements (paths inside the DL4S repository,
 * Sources/DL4S/...).
 *
 * Conventions
 *  - All tensors are fp32, row-major, contiguous, shapes passed explicitly
 *    (DL4S derives strides from shapes, Memory Management/MemoryOps.swift:253-278).
 *  - Pointers named d_* are device addresses; everything else is host memory.
 *  - Every function returns a dl4s_status (0 = ok). DL4S itself aborts on
 *    violated preconditions (e.g. Tensor/Operators/Matrix.swift:39-41); the
 *    Swift glue turns a non-zero status into fatalError(dl4s_cuda_last_error()).
 *  - Work is enqueued on one stream per device and is asynchronous. Only
 *    dl4s_cuda_memcpy_d2h, dl4s_cuda_get_value_f32 and dl4s_cuda_sync wait.
 *  - Calls act on the calling thread's current device (dl4s_cuda_set_device).
 *    One host thread per device, as in DL4S (its engines are single-threaded).
 *  - There is no CPU fallback: without a CUDA device every compute call fails
 *    with DL4S_ERR_CUDA.
 */
#ifndef DL4S_CUDA_H
#define DL4S_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DL4S_CUDA_VERSION 100

typedef int32_t dl4s_status;
enum {
    DL4S_OK = 0,
    DL4S_ERR_INVALID_ARG = -1,
    DL4S_ERR_OOM = -2,
    DL4S_ERR_CUDA = -3,
    DL4S_ERR_UNSUPPORTED = -4,
    DL4S_ERR_TIMEOUT = -5, /* a bounded device-side wait gave up; see dl4s_cuda_device_status */
    DL4S_ERR_NOT_INITIALIZED = -6,
    DL4S_ERR_NCCL = -7     /* the collective library is missing, or a communicator / collective call failed */
};

/* Arithmetic used by the fused kernels.
 *  DL4S_PREC_FP32      : fp32 FFMA everywhere (check kernels; agrees with the DL4S
 *                        CPU engine to ~1e-5).
 *  DL4S_PREC_F16       : tensor-core path. Operands are rounded to IEEE half
 *                        (11-bit significand, the same as TF32) and multiplied by
 *                        tcgen05 MMAs with fp32 accumulation in tensor memory.
 *  DL4S_PREC_F16_SPLIT : the same path with every weight matrix kept as the sum of
 *                        two halves (the rounded value and the rounded remainder,
 *                        ~22 significant bits); the projections and the feed-forward
 *                        products cost twice the MMA work. Activations and the
 *                        attention products are as in DL4S_PREC_F16. For stacks of
 *                        layers whose output must stay within max-abs 2e-3 of the
 *                        fp32 engine: rounding the weights once is what dominates the
 *                        error of a deep stack (6-layer encoder, d_model 512: max-abs
 *                        3e-3 with DL4S_PREC_F16, 1.5e-3 with DL4S_PREC_F16_SPLIT;
 *                        relative L2 6.7e-4 and 2.9e-4).
 * On both tensor-core paths operands must lie within the half range (|x| < 65504): a
 * value that does not sets bit 0x400 of the device status word (dl4s_cuda_device_status
 * then returns DL4S_ERR_INVALID_ARG); the results of that call are not usable. */
enum { DL4S_PREC_FP32 = 0, DL4S_PREC_F16 = 1, DL4S_PREC_F16_SPLIT = 2 };

/* Feed-forward activation. 0 is what DL4S computes (PointwiseFeedForward.swift:76). */
enum { DL4S_ACT_GELU_SIGMOID = 0, DL4S_ACT_RELU = 1 };

/* ------------------------------------------------------------------ lifecycle
 * DeviceType (Engine/Engine.swift:30-35) has no run-time state in DL4S; a CUDA
 * device needs a context, a stream and a scratch arena. */
dl4s_status dl4s_cuda_device_count(int32_t *count);
/* Creates the per-device state for the listed CUDA ordinals (n == 0: device 0)
 * and makes devices[0] current. Idempotent. */
dl4s_status dl4s_cuda_init(const int32_t *devices, int32_t n);
dl4s_status dl4s_cuda_shutdown(void);
dl4s_status dl4s_cuda_set_device(int32_t device);
dl4s_status dl4s_cuda_get_device(int32_t *device);
/* Blocks until everything enqueued on the current device has finished. */
dl4s_status dl4s_cuda_sync(void);
/* Run the library on a stream owned by the caller (a cudaStream_t); NULL
 * restores the library's own stream. Waits for the work queued on the stream
 * it leaves (the scratch arena is reused in stream order). */
dl4s_status dl4s_cuda_set_stream(void *cuda_stream);
dl4s_status dl4s_cuda_get_stream(void **cuda_stream);
/* Thread-local description of the last failure on this thread. */
const char *dl4s_cuda_last_error(void);
int32_t dl4s_cuda_version(void);
/* Reads and clears the device status word (0 = clean): kernels with bounded waits set bits
 * 0x001-0x100 when a wait runs out (DL4S_ERR_TIMEOUT); a decode step that found its
 * key/value cache full sets 0x200, a tensor-core operand outside the half range 0x400
 * (both DL4S_ERR_INVALID_ARG). Synchronises the stream. */
dl4s_status dl4s_cuda_device_status(int32_t *status_word);
/* Milliseconds the device spent in the last fused call, measured with CUDA
 * events on the library's stream when timing is enabled (enable != 0). */
dl4s_status dl4s_cuda_set_timing(int32_t enable);
dl4s_status dl4s_cuda_get_timing(float *ms);
/* Per-kernel device time, the tracing facility of this back-end (DL4S has only
 * OperationGroup names in debug builds, Tensor/Graph.swift:134-163). Between
 * begin and end one CUDA event is recorded after every kernel the library
 * launches; end waits for the stream and writes a JSON object
 * {"kernel_name": {"launches": n, "total_ms": t}, ...} into `report`. The time
 * of a kernel runs from the end of the previous launch to its own end. */
dl4s_status dl4s_cuda_profile_begin(void);
dl4s_status dl4s_cuda_profile_end(char *report, size_t capacity);
/* The reference's operation groups (OperationGroup.capture(named:), Tensor/Graph.swift:134-163: "Encoder",
 * "EncoderLayer", "MultiHeadAttention", "ScaledDotProductAttention", "PointwiseFeedForward", "LayerNorm", "Dense",
 * "Embedding") as NVTX ranges around the launches they cover, for a timeline profiler. Off by default; on with
 * enable != 0 or DL4S_CUDA_TRACE=1 in the environment at dl4s_cuda_init. While on, the group paths entered
 * ("Encoder/EncoderLayer/MultiHeadAttention", one per line, in order) are also kept on the host (64 KB);
 * trace_read copies them out and clears the list. */
dl4s_status dl4s_cuda_set_trace(int32_t enable);
dl4s_status dl4s_cuda_trace_read(char *report, size_t capacity);
/* Failure injection for tests of the error path (DL4S itself aborts the process on such failures, e.g.
 * Engine/CPU/CPU.swift:71-84 has no failure return): the next `count` operations of kind `what` fail with the
 * status they would report for a real failure and a message that says "injected failure"; count = 0 clears.
 * Works before dl4s_cuda_init and without a device, so the error plumbing of a binding can be tested anywhere.
 *  DL4S_INJECT_MALLOC        dl4s_cuda_malloc                      -> DL4S_ERR_OOM
 *  DL4S_INJECT_H2D           dl4s_cuda_memcpy_h2d / _h2d_async     -> DL4S_ERR_CUDA
 *  DL4S_INJECT_COMM          dl4s_cuda_comm_init                   -> DL4S_ERR_NCCL
 *  DL4S_INJECT_WAIT_TIMEOUT  the next single-CTA tensor-core GEMM launch leaves out one operand load and polls
 *                            with a short limit: its bounded wait runs out, the kernel leaves through its normal
 *                            exit (nothing traps or hangs) and dl4s_cuda_device_status reports DL4S_ERR_TIMEOUT;
 *                            the product of that launch is garbage. */
enum { DL4S_INJECT_MALLOC = 1, DL4S_INJECT_H2D = 2, DL4S_INJECT_COMM = 3, DL4S_INJECT_WAIT_TIMEOUT = 4 };
dl4s_status dl4s_cuda_inject_failure(int32_t what, int32_t count);
/* CUDA graphs. Between begin and end the calls made on the current device are RECORDED (stream capture on
 * the library's stream) instead of run; end returns a handle that replays them with one launch. The recorded
 * calls must not allocate, free, wait or read back: buffers are allocated before, and the same calls have run
 * once eagerly so that the scratch arena has its size (otherwise the call fails with DL4S_ERR_UNSUPPORTED and
 * the capture must still be ended). Pointers and shapes are baked into the graph: a replay reads and writes
 * the same buffers. */
dl4s_status dl4s_cuda_graph_begin(void);
dl4s_status dl4s_cuda_graph_end(void **graph);
dl4s_status dl4s_cuda_graph_launch(void *graph);
dl4s_status dl4s_cuda_graph_destroy(void *graph);
/* Number of kernels the library has launched on the current device so far (a graph launch counts the kernels
 * recorded in it). */
dl4s_status dl4s_cuda_launch_count(uint64_t *count);

/* --------------------------------------------------------------------- memory
 * MemoryOperatorsType (Engine/Engine.swift:39-139), CPU counterpart
 * Engine/CPU/CPU.swift:71-231. Allocation and free are stream-ordered, like the
 * deferred free of the CPU engine (CPU.swift:103-112). `advance` and prefix
 * slices are plain pointer arithmetic on the caller's side. */
dl4s_status dl4s_cuda_malloc(size_t bytes, void **d_ptr);                 /* allocateBuffer, Engine.swift:48,54 */
dl4s_status dl4s_cuda_free(void *d_ptr);                                   /* free, Engine.swift:58,62 */
dl4s_status dl4s_cuda_memcpy_h2d(void *d_dst, const void *src, size_t bytes);   /* assign(from host), Engine.swift:69 */
dl4s_status dl4s_cuda_memcpy_d2h(void *dst, const void *d_src, size_t bytes);   /* assign(to host), Engine.swift:83 */
dl4s_status dl4s_cuda_memcpy_d2d(void *d_dst, const void *d_src, size_t bytes); /* assign(device), Engine.swift:76 */
/* Like memcpy_h2d but returns at once; `src` must be page-locked and stay valid. */
dl4s_status dl4s_cuda_memcpy_h2d_async(void *d_dst, const void *src, size_t bytes);
dl4s_status dl4s_cuda_memcpy_d2h_async(void *dst, const void *d_src, size_t bytes);
/* The same copies on a stream of the caller's (a cudaStream_t) instead of the library's: lets the read-back of
 * one step overlap the next step's kernels. The caller orders them against the library's stream with events.
 * (dl4s_cuda_set_stream is not meant for this: it waits for the stream it leaves.) */
dl4s_status dl4s_cuda_memcpy_h2d_async_on(void *d_dst, const void *src, size_t bytes, void *cuda_stream);
dl4s_status dl4s_cuda_memcpy_d2h_async_on(void *dst, const void *d_src, size_t bytes, void *cuda_stream);
dl4s_status dl4s_cuda_host_alloc(size_t bytes, void **ptr);                /* page-locked staging memory */
dl4s_status dl4s_cuda_host_free(void *ptr);
dl4s_status dl4s_cuda_get_value_f32(const float *d_src, float *value);     /* getValue, Engine.swift:87 */
dl4s_status dl4s_cuda_set_value_f32(float *d_dst, float value);            /* setPointee, Engine.swift:132 */
/* Strided sub-tensor copy between device buffers: the general (copying) case of
 * get(slice:) / set(slice:) (Engine.swift:100-127; CPU.swift:137-213).
 * Element i of the dim-D box `extent` is read at sum(i_k*src_stride_k)+src_offset. */
dl4s_status dl4s_cuda_copy_strided_f32(const float *d_src, const int64_t *src_strides, int64_t src_offset,
                                       float *d_dst, const int64_t *dst_strides, int64_t dst_offset,
                                       const int64_t *extent, int32_t dim);

/* ----------------------------------------------------- EngineType primitives
 * fp32 instances of the EngineType requirements an unfused attention graph
 * uses (Engine/Engine.swift:143-581); CPU counterparts in
 * Engine/CPU/CPUEngine.swift. */
dl4s_status dl4s_cuda_fill_f32(float value, float *d_result, int64_t count);                         /* fill, Engine.swift:153 */
dl4s_status dl4s_cuda_fill_i32(int32_t value, int32_t *d_result, int64_t count);
dl4s_status dl4s_cuda_vadd(const float *d_lhs, const float *d_rhs, float *d_result, int64_t count);  /* vAdd :161 */
dl4s_status dl4s_cuda_vsub(const float *d_lhs, const float *d_rhs, float *d_result, int64_t count);  /* vSub :176 */
dl4s_status dl4s_cuda_vmul(const float *d_lhs, const float *d_rhs, float *d_result, int64_t count);  /* vMul :184 */
dl4s_status dl4s_cuda_vdiv(const float *d_lhs, const float *d_rhs, float *d_result, int64_t count);  /* vDiv :192 */
dl4s_status dl4s_cuda_vneg(const float *d_val, float *d_result, int64_t count);                      /* vNeg :168 */
/* numpy-rule broadcasting, shapes right-aligned (CPUEngine.swift:90-214). The
 * result shape is the broadcast of both. Division by a broadcast scalar is a
 * multiplication by its fp32 reciprocal, as in CPUEngine.swift:628-636. */
dl4s_status dl4s_cuda_broadcast_add(const float *d_lhs, const int64_t *lshape, int32_t ldim,
                                    const float *d_rhs, const int64_t *rshape, int32_t rdim, float *d_result); /* :242 */
dl4s_status dl4s_cuda_broadcast_sub(const float *d_lhs, const int64_t *lshape, int32_t ldim,
                                    const float *d_rhs, const int64_t *rshape, int32_t rdim, float *d_result); /* :249 */
dl4s_status dl4s_cuda_broadcast_mul(const float *d_lhs, const int64_t *lshape, int32_t ldim,
                                    const float *d_rhs, const int64_t *rshape, int32_t rdim, float *d_result); /* :256 */
dl4s_status dl4s_cuda_broadcast_div(const float *d_lhs, const int64_t *lshape, int32_t ldim,
                                    const float *d_rhs, const int64_t *rshape, int32_t rdim, float *d_result); /* :263 */
dl4s_status dl4s_cuda_exp(const float *d_val, float *d_result, int64_t count);        /* :363 */
dl4s_status dl4s_cuda_log(const float *d_val, float *d_result, int64_t count);        /* :369 */
dl4s_status dl4s_cuda_sqrt(const float *d_val, float *d_result, int64_t count);       /* :375 */
dl4s_status dl4s_cuda_relu(const float *d_val, float *d_result, int64_t count);       /* :381 */
dl4s_status dl4s_cuda_heaviside(const float *d_val, float *d_result, int64_t count);  /* :387 */
dl4s_status dl4s_cuda_sin(const float *d_val, float *d_result, int64_t count);        /* :393 */
dl4s_status dl4s_cuda_cos(const float *d_val, float *d_result, int64_t count);        /* :399 */
dl4s_status dl4s_cuda_tanh(const float *d_val, float *d_result, int64_t count);       /* :423 */
/* Reduction over `axes` (ascending) of a tensor of `shape`; the result has the
 * reduced axes removed. reduce_max also writes the arg-max position along the
 * axis when d_context is not NULL and exactly one axis is reduced. */
dl4s_status dl4s_cuda_reduce_sum(const float *d_val, const int64_t *shape, int32_t dim,
                                 const int32_t *axes, int32_t naxes, float *d_result);               /* :272,302 */
dl4s_status dl4s_cuda_reduce_max(const float *d_val, const int64_t *shape, int32_t dim,
                                 const int32_t *axes, int32_t naxes, float *d_result, int32_t *d_context); /* :280,310 */
/* permuteAxes with DL4S's convention: source axis i becomes destination axis
 * arangement[i] (Tensor/Operators/Shape.swift:127-129; CPUEngine.swift:897-935). */
dl4s_status dl4s_cuda_permute_axes(const float *d_val, const int64_t *shape, int32_t dim,
                                   const int32_t *arangement, float *d_result);                      /* :478 */
/* stack: concatenates n buffers along `axis`; shapes[i] holds `dim` extents each. */
dl4s_status dl4s_cuda_stack(const float *const *d_buffers, const int64_t *shapes, int32_t n, int32_t dim,
                            int32_t axis, float *d_result);                                          /* :536 */
/* unstack: the inverse of stack (the backward of Tensor(stacking:), Tensor/Operators/Stack.swift:79-122): buffer i
 * of shape shapes[i] receives its slab of the stacked tensor. unstack_add adds d_add[i] to the slab on the way
 * (gradient accumulation). CPUEngine.swift:1025-1085. */
dl4s_status dl4s_cuda_unstack(const float *d_stacked, float *const *d_results, const int64_t *shapes, int32_t n,
                              int32_t dim, int32_t axis);                                            /* :551 */
dl4s_status dl4s_cuda_unstack_add(const float *d_stacked, const float *const *d_add, float *const *d_results,
                                  const int64_t *shapes, int32_t n, int32_t dim, int32_t axis);      /* :543 */
/* band: keeps src[i,j] for i-below <= j <= i+above, zero elsewhere; a negative
 * has_* flag of 0 means "unbounded" (nil in DL4S). CPUEngine.swift:1135-1158. */
dl4s_status dl4s_cuda_band(const float *d_src, int64_t rows, int64_t cols, int32_t below, int32_t has_below,
                           int32_t above, int32_t has_above, float *d_result);                      /* :233 */
/* gemm: C = alpha*op(A)*op(B) + beta*C, row-major, A stored [M,K] ([K,M] when
 * trans_a), B stored [K,N] ([N,K] when trans_b). Engine.swift:225;
 * CPUFloat.swift:263-292. `precision` selects FFMA or tensor cores: the tensor-core kernels take alpha = 1, beta = 0,
 * M >= 128 and N, K multiples of 64, with or without transposed operands (the products of a matmul's backward,
 * Tensor/Operators/Matrix.swift:139-173: dA = dC B^T, dB = A^T dC); other calls run on the fp32 kernel. */
dl4s_status dl4s_cuda_gemm(const float *d_a, const float *d_b, float *d_c, int64_t M, int64_t N, int64_t K,
                           float alpha, float beta, int32_t trans_a, int32_t trans_b, int32_t precision);

/* Dropout (NN/Layer/Dropout.swift:47-55): y = x * bernoulli(1 - rate), NOT rescaled by 1/(1 - rate). DL4S draws the
 * mask on the host from a process-global generator (Random.swift:148-157) and copies it to the device per call; here
 * the mask is a counter-based hash evaluated where the value is produced. Element i of dropout site `counter` is
 * kept when hash32(seed, counter, i) < floor((1 - rate) * 2^32), with
 *   h = (uint32)i * 0x9E3779B1 + (uint32)seed;  h ^= h >> 16; h *= 0x85EBCA6B; h ^= h >> 13; h *= 0xC2B2AE35; h ^= h >> 16;
 *   h += (((uint32)(i >> 32)) ^ counter) * 0x27D4EB2F + (uint32)(seed >> 32);
 *   h ^= h >> 15; h *= 0x2C1B3C6D; h ^= h >> 12; h *= 0x297A2D39; h ^= h >> 15;
 * in 32-bit wrap-around arithmetic, so a host can regenerate any mask (the parity tests do).
 *   dropout          the layer itself on a buffer of `count` elements.
 *   set_dropout      rate and seed of the dropout fused into the layer calls of the current device: the output
 *                    projection of MultiHeadAttention (MultiHeadAttention.swift:122), the second Dense of
 *                    PointwiseFeedForward (PointwiseFeedForward.swift:78) and the embedded inputs
 *                    (Transformer.swift:87), each inside the kernel that produces the values (element index = the
 *                    row-major index in that [rows, D] result). rate 0 (the default) turns it off; the decoding
 *                    steps never apply it (inference).
 *   dropout_counter  every site that applies dropout takes the next counter value (in call order: per encoder layer
 *                    first the attention site, then the feed-forward site); reads it, and sets it when set_to is not
 *                    NULL. A recorded graph replays the counters it was recorded with. */
dl4s_status dl4s_cuda_dropout(const float *d_x, float *d_result, int64_t count, float rate, uint64_t seed, uint32_t counter);
dl4s_status dl4s_cuda_set_dropout(float rate, uint64_t seed);
dl4s_status dl4s_cuda_dropout_counter(uint32_t *current, const uint32_t *set_to);

/* ------------------------------------------------------------- fused hot path */

/* ScaledDotProductAttention.callAsFunction
 * (NN/Models/Transformer/ScaledDotProductAttention.swift:43-64):
 *   out = softmax((q * 1/temperature) k^T - mask*1e9, last axis) v
 * q [B,H,Sq,dk], k [B,H,Sk,dk], v [B,H,Sk,dv] -> out [B,H,Sq,dv].
 * The mask is given in one of two ways (both may be absent):
 *  - structurally: d_key_lengths[B] (keys j >= length blocked: makeEncoderMasks,
 *    TransformerUtil.swift:29-36) and/or causal != 0 (keys j > i blocked:
 *    makeDecoderMasks, TransformerUtil.swift:38-50). Never materialised; tiles
 *    that are fully blocked are never loaded.
 *  - densely: d_mask with mask_shape[4], each extent 1 or the full extent, 1 =
 *    blocked (fp32 path only).
 * A row whose keys are all blocked yields the uniform average of all Sk value
 * rows, as the reference's finite -1e9 does. */
dl4s_status dl4s_cuda_sdpa_forward(const float *d_q, const float *d_k, const float *d_v,
                                   int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv,
                                   float temperature, const int32_t *d_key_lengths, int32_t causal,
                                   const float *d_mask, const int64_t *mask_shape,
                                   float *d_out, int32_t precision);

/* The same function for one query per sequence (Sq == 1) against a long
 * context: q [B,H,1,dk], k,v [B,H,Lmax,d*], d_key_lengths[B] (NULL: all Lmax).
 * HBM-bound split-K kernel: the context is cut into chunks, each reduced by one
 * thread block with 128-bit loads, partial (max, sum, out) records are merged
 * by a second kernel. fp32 throughout. Rows at or beyond a length are never read. */
dl4s_status dl4s_cuda_sdpa_decode(const float *d_q, const float *d_k, const float *d_v,
                                  int64_t B, int64_t H, int64_t Lmax, int64_t dk, int64_t dv,
                                  float temperature, const int32_t *d_key_lengths, float *d_out);

/* The same decode attention for hosts that must not allocate device memory at
 * the point where decode runs. It has no counterpart in the reference (DL4S
 * allocates a fresh buffer per operation). dl4s_cuda_sdpa_decode keeps its
 * split-K records in a scratch arena that grows through cudaMalloc; that call
 * fails once a serving process has handed all of HBM to its own cache manager,
 * and it synchronises the whole device, which a latency-bound decode step
 * cannot accept. This variant calls no cudaMalloc / cudaFree or any other
 * allocating routine: the records live in a fixed 8 MiB array inside the
 * library image (held by every GPU that loads the library until exit).
 *  - dk == dv == d in {64, 128}; q, k, v 16-byte aligned; d_key_lengths may be NULL.
 *  - Limit: B*H*ceil(Lmax/chunk)*(d+2) <= 2,097,152 floats for some chunk in
 *    {256, 512, ..., 8192}; larger problems are rejected with
 *    DL4S_ERR_UNSUPPORTED and a message, nothing is launched.
 *  - dl4s_cuda_init looks the array's address up for each device it is given
 *    (cudaGetSymbolAddress with that device current) and loads the two decode
 *    kernels, so the 8 MiB are taken at initialisation and no module load can
 *    happen at decode time: call dl4s_cuda_init before the host claims the rest
 *    of HBM and before any stream capture. One host thread per device, as for
 *    every other call.
 *  - A key length above Lmax is read as Lmax (all entry points of this path).
 *  - All calls share the one array, and it keeps the previous call's contents.
 *    Nothing in it has to start at zero (every record a call reads is written
 *    by that call first), but two calls that overlap on the GPU - different
 *    streams or devices' threads racing on one device - corrupt each other. */
dl4s_status dl4s_cuda_sdpa_decode_noalloc(const float *d_q, const float *d_k, const float *d_v,
                                          int64_t B, int64_t H, int64_t Lmax, int64_t d,
                                          float temperature, const int32_t *d_key_lengths, float *d_out);

/* LayerNorm.callAsFunction (NN/Layer/LayerNorm.swift:62-77) on x viewed as
 * [outer, rows, D]: mean and E[x^2]-mean^2 over rows*D elements per outer
 * index, y = (x-mean) * 1/(sqrt(var)+1e-5) * scale[D] + shift[D]. If
 * d_residual is not NULL the input is x + residual (the residual additions of
 * MultiHeadAttention.swift:123 and PointwiseFeedForward.swift:79). */
dl4s_status dl4s_cuda_layernorm(const float *d_x, const float *d_residual, int64_t outer, int64_t rows, int64_t D,
                                const float *d_scale, const float *d_shift, float *d_out);

/* Backward of dl4s_cuda_layernorm: the gradients DL4S's autograd obtains by chaining the backward closures of the
 * primitives LayerNorm.callAsFunction is written with (LayerNorm.swift:62-77; Reduce.swift:87-110), in closed form.
 * d_x is the layer's input (x + residual of the forward call), d_dy the upstream gradient, both [outer, rows, D];
 * d_dx [outer, rows, D] (also the gradient of the residual); d_dscale, d_dshift [D] may both be NULL. fp32. */
dl4s_status dl4s_cuda_layernorm_backward(const float *d_x, const float *d_dy, int64_t outer, int64_t rows, int64_t D,
                                         const float *d_scale, float *d_dx, float *d_dscale, float *d_dshift);

/* MultiHeadAttention.callAsFunction (NN/Models/Transformer/MultiHeadAttention.swift:97-127),
 * dropout inactive: out = LayerNorm_{per batch element over Sq x D}(
 *   concat_h SDPA(xq Wq, xk Wk, xv Wv) Wo + xq ).
 * xq [B,Sq,D]; xk, xv [B,Sk,D]; Wq,Wk [D,H*dk]; Wv [D,H*dv]; Wo [H*dv,D]. */
dl4s_status dl4s_cuda_mha_forward(const float *d_xq, const float *d_xk, const float *d_xv,
                                  int64_t B, int64_t Sq, int64_t Sk, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                  const float *d_wq, const float *d_wk, const float *d_wv, const float *d_wo,
                                  const float *d_ln_scale, const float *d_ln_shift,
                                  const int32_t *d_key_lengths, int32_t causal,
                                  const float *d_mask, const int64_t *mask_shape,
                                  float *d_out, int32_t precision);

/* Backward of ScaledDotProductAttention.callAsFunction: the gradients DL4S's autograd obtains by chaining the
 * backward closures of mmul (Tensor/Operators/Matrix.swift:139-173), the softmax composition
 * (Unary.swift:190-194) and the division by the temperature, in one call:
 *   d_dout [B,H,Sq,dv] -> d_dq [B,H,Sq,dk], d_dk [B,H,Sk,dk], d_dv [B,H,Sk,dv]
 * for contiguous q, k, v and the same mask arguments as dl4s_cuda_sdpa_forward. The probabilities are
 * recomputed (the forward call keeps nothing).
 *  DL4S_PREC_FP32: fp32 FFMA kernels (agree with the CPU engine's gradients to 1e-5); scratch of 2*B*H*Sq*Sk
 *                  floats from the device arena; head sizes up to 256; dense masks.
 *  DL4S_PREC_F16 / _SPLIT: flash-style tensor-core kernel (dk == dv in {64, 128}, structural masks, 16-byte
 *                  aligned buffers; otherwise the fp32 kernels run): per key tile S = Q K^T and dP = dout V^T are
 *                  recomputed, dV += P^T dout, dK += dS^T Q, dQ += dS K with tcgen05 MMAs, nothing of size Sq x Sk
 *                  is stored. dq rows are summed over key tiles with atomic adds (last-bit differences between
 *                  runs); dk and dv are summed in a fixed order. */
dl4s_status dl4s_cuda_sdpa_backward(const float *d_q, const float *d_k, const float *d_v, const float *d_dout,
                                    int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv,
                                    float temperature, const int32_t *d_key_lengths, int32_t causal,
                                    const float *d_mask, const int64_t *mask_shape,
                                    float *d_dq, float *d_dk, float *d_dv, int32_t precision);

/* The two halves of MultiHeadAttention.callAsFunction around the point where a
 * layer that spans GPUs exchanges data (MultiHeadAttention.swift:109-119 and
 * :121-124). Attention is independent per (batch, head), so a GPU that owns Hl of
 * the H heads runs the first half with its column slices of Wq/Wk [D,Hl*dk] and
 * Wv [D,Hl*dv] and produces d_heads_out [B,Sq,Hl*dv]; after the head outputs of
 * all GPUs are gathered into [B,Sq,H*dv] (one NCCL all-gather, done by the
 * caller), the second half applies Wo [HDv,D], adds the residual (the layer's
 * query input) and normalises. dl4s_cuda_mha_forward is the two halves back to back.
 * The head outputs only feed the tensor-core operand of Wo, so on the tensor-core
 * path they may travel as IEEE half (half_output / half_input != 0; the buffer then
 * holds 2-byte elements), which halves the bytes of the all-gather. This needs
 * self-attention (xq == xk == xv) and shapes for which
 * dl4s_cuda_mha_heads_half_supported reports 1; otherwise DL4S_ERR_UNSUPPORTED.
 * The second half reads the gathered head outputs where the all-gather left them:
 * d_heads is `groups` column blocks of HDv/groups columns, element (m, g*C + c)
 * at d_heads[g*group_stride + m*C + c] (elements, not bytes; m = b*Sq + s counted
 * from the first row of the caller's batch slice). groups = 1 is the plain
 * [B*Sq, HDv] matrix and ignores group_stride. */
dl4s_status dl4s_cuda_mha_heads_forward(const float *d_xq, const float *d_xk, const float *d_xv,
                                        int64_t B, int64_t Sq, int64_t Sk, int64_t D, int64_t Hl, int64_t dk, int64_t dv,
                                        const float *d_wq, const float *d_wk, const float *d_wv,
                                        const int32_t *d_key_lengths, int32_t causal,
                                        void *d_heads_out, int32_t precision, int32_t half_output);
dl4s_status dl4s_cuda_mha_heads_half_supported(int64_t B, int64_t S, int64_t D, int64_t Hl, int64_t dk, int64_t dv,
                                               int64_t HDv, int32_t *supported);
dl4s_status dl4s_cuda_mha_output_forward(const void *d_heads, const float *d_residual,
                                         int64_t B, int64_t Sq, int64_t D, int64_t HDv,
                                         const float *d_wo, const float *d_ln_scale, const float *d_ln_shift,
                                         float *d_out, int32_t precision, int32_t half_input,
                                         int64_t groups, int64_t group_stride);

/* ------------------------------------------------------------ a layer that spans GPUs
 * DL4S is single-device; these calls have no counterpart there. MultiHeadAttention.callAsFunction
 * (MultiHeadAttention.swift:97-127) with its heads spread over `world` GPUs of one node, one rank per GPU (a
 * process, or a thread with its own current device). The library owns the NCCL communicator, the second stream the
 * collective runs on and the gather buffers. NCCL (libnccl.so.2, or the path in DL4S_NCCL_LIB) is loaded when the
 * first of these calls needs it; hosts without it can use everything else.
 *   comm_unique_id  rank 0 obtains the 128-byte id and hands it to the other ranks by any means (a file, a socket,
 *                   the launcher's store).
 *   comm_init       the calling thread's current device joins as `rank` of `world` (collective: every rank calls
 *                   it). world == 1 needs no id and no NCCL.
 *   comm_destroy    leaves the communicator and frees its buffers.
 *   comm_info       rank, world (0 / 1 if the device never joined) and the NCCL version in use (0: not loaded). */
#define DL4S_COMM_ID_BYTES 128
dl4s_status dl4s_cuda_comm_unique_id(uint8_t *id);
dl4s_status dl4s_cuda_comm_init(int32_t rank, int32_t world, const uint8_t *id);
dl4s_status dl4s_cuda_comm_destroy(void);
dl4s_status dl4s_cuda_comm_info(int32_t *rank, int32_t *world, int32_t *nccl_version);
/* Of the last dl4s_cuda_mha_forward_sharded call on this device (waits for it): the summed device time from "head
 * outputs written" to "gather finished" over its chunks, and the part of it the compute stream spent waiting for a
 * gather (the exposed part; the rest ran under the next chunk's kernels). Zeros for a world of one. */
dl4s_status dl4s_cuda_comm_timing(float *gather_ms, float *exposed_ms);
/* The head-sharded layer. Every rank passes the FULL input d_x [B,S,D] (replicated), ITS column slices of the
 * projections d_wq_local, d_wk_local [D,(H/world)*dk], d_wv_local [D,(H/world)*dv] (heads
 * [rank*H/world, (rank+1)*H/world)), and the full Wo [H*dv,D] and LayerNorm parameters. Rank g runs projections and
 * attention for its heads on the whole batch, ONE ncclAllGather per batch chunk collects the head outputs of all
 * ranks (as IEEE half on the tensor-core paths), then rank g applies Wo + residual + LayerNorm to its batch slice of
 * the chunk. With chunks > 1 the gather of chunk c runs on a second stream under the compute of chunk c+1.
 * The output stays sharded by batch: d_out holds the rows this rank owns, [rows, S, D];
 * dl4s_cuda_mha_sharded_plan reports how many (and, if batch_index is not NULL, which batch elements, in output
 * order) for a rank of a world with the same B and chunks; it is host arithmetic and needs no device. Every rank must make the same calls in the same order with the same B, S, chunks
 * (each call contains collectives). Self-attention only; the mask is structural (d_key_lengths[B] and/or causal). */
dl4s_status dl4s_cuda_mha_forward_sharded(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                          const float *d_wq_local, const float *d_wk_local, const float *d_wv_local,
                                          const float *d_wo, const float *d_ln_scale, const float *d_ln_shift,
                                          const int32_t *d_key_lengths, int32_t causal, float *d_out,
                                          int32_t precision, int32_t chunks);
dl4s_status dl4s_cuda_mha_sharded_plan(int64_t B, int32_t world, int32_t rank, int32_t chunks, int64_t *rows,
                                       int64_t *batch_index);

/* One step of incremental decoding through a decoder self-attention layer with a key/value cache: the caller of
 * dl4s_cuda_sdpa_decode. DL4S has no cache — Transformer.callAsFunction(inputSequence:...)
 * (NN/Models/Transformer/Transformer.swift:118-137) re-runs the whole decoder on the growing prefix for every
 * generated token; the last row of MultiHeadAttention over the prefix with the causal mask
 * (TransformerDecoderBlock.swift:61-65) is what this call computes from the cache.
 *   d_x [B, D]            the current token's input row per sequence (also the residual)
 *   d_k_cache, d_v_cache  [B, H, Lmax, dk] / [B, H, Lmax, dv]; rows [0, lengths[b]) hold the prefix
 *   d_lengths [B]         tokens already cached per sequence; NOT modified (the caller adds 1 afterwards)
 * The token's k and v projections are written to row lengths[b] of the caches, attention runs over
 * lengths[b] + 1 keys, then Wo, the residual and the LayerNorm over the token's [1, D] block -> d_out [B, D].
 * fp32 throughout (the step is bound by reading the weights and the cache). A full cache sets bit 0x200 of the
 * device status word and leaves the cache unchanged. */
dl4s_status dl4s_cuda_mha_decode_step(const float *d_x, int64_t B, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                      const float *d_wq, const float *d_wk, const float *d_wv, const float *d_wo,
                                      const float *d_ln_scale, const float *d_ln_shift,
                                      float *d_k_cache, float *d_v_cache, int64_t Lmax,
                                      const int32_t *d_lengths, float *d_out);

/* TransformerDecoder.callAsFunction (NN/Models/Transformer/TransformerDecoder.swift:49-62) over whole sequences:
 * `layers` blocks of TransformerDecoderBlock.callAsFunction (TransformerDecoderBlock.swift:61-68),
 *   decAttn = MHA(x, x, x, decoderMask); encAttn = MHA(decAttn, enc, enc, encoderMask); x' = FFN(encAttn),
 * with decoderMask = causal OR padding by d_dec_lengths[B] and encoderMask = padding by d_enc_lengths[B]
 * (makeDecoderMasks / makeEncoderMasks, TransformerUtil.swift:29-50; either pointer may be NULL: no padding).
 * d_x [B,St,D] decoder input, d_enc [B,Ss,D] encoder states. d_params holds, per layer and in the order of
 * TransformerDecoderBlock.parameters: self-attention Wq, Wk [D,H*dk], Wv [D,H*dv], Wo [H*dv,D], ln_scale, ln_shift
 * [D]; encoder attention the same six; W1 [D,F], b1 [F], W2 [F,D], b2 [D], ln_scale, ln_shift [D]. */
dl4s_status dl4s_cuda_decoder_forward(const float *d_x, const float *d_enc, int64_t B, int64_t St, int64_t Ss, int64_t D,
                                      int64_t H, int64_t dk, int64_t dv, int64_t F, int64_t layers, const float *d_params,
                                      const int32_t *d_dec_lengths, const int32_t *d_enc_lengths, int32_t act,
                                      float *d_out, int32_t precision);

/* Incremental decoding through a whole decoder stack (no counterpart in DL4S, which re-runs the decoder on the
 * growing prefix for every token, Transformer.swift:122-134). The cache holds, per layer, the self-attention keys
 * and values of the tokens decoded so far [B,H,Lmax,d] and the encoder keys and values, projected ONCE per input
 * sequence [B,H,Ss,d] (they do not change while a sequence is decoded).
 *   mha_kv_project     k = x Wk, v = x Wv for x [B,S,D], written head-major into caches [B,H,Lmax,d] (rows 0..S-1):
 *                      the projection half of MultiHeadAttention.swift:110-115 for keys and values.
 *   cache_create       allocates the caches for B sequences, Lmax decoded tokens and Ss encoder positions; d_params
 *                      (layout of dl4s_cuda_decoder_forward) must stay valid while the cache lives.
 *   cache_set_encoder  projects d_enc [B,Ss,D] through every layer's encoder-attention Wk / Wv and resets the
 *                      decoded length to 0: the start of a new batch of sequences.
 *   decoder_step       one token per sequence, d_x [B,D] -> d_out [B,D], through every layer: self-attention over
 *                      the cache and the token (dl4s_cuda_mha_decode_step), encoder attention of the token's query
 *                      over the projected encoder keys/values (the decode attention kernel), feed-forward; then the
 *                      decoded length advances by one. fp32.
 *   cache_lengths      device address of the decoded length per sequence [B] (int32), e.g. to rewind.
 * Each token's LayerNorm runs over its own [1, D] block. DL4S's LayerNorm inside MultiHeadAttention normalises the
 * whole [prefix, D] block of a sequence at once, so its statistics move every earlier row with every new token
 * and NO cache can reproduce what the reference recomputes; dl4s_cuda_decoder_forward on the prefix does. */
dl4s_status dl4s_cuda_mha_kv_project(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                     const float *d_wk, const float *d_wv, float *d_k_cache, float *d_v_cache, int64_t Lmax);
dl4s_status dl4s_cuda_decoder_cache_create(int64_t B, int64_t Lmax, int64_t Ss, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                           int64_t F, int64_t layers, const float *d_params, void **cache);
dl4s_status dl4s_cuda_decoder_cache_set_encoder(void *cache, const float *d_enc, const int32_t *d_enc_lengths);
dl4s_status dl4s_cuda_decoder_cache_lengths(void *cache, int32_t **d_lengths);
dl4s_status dl4s_cuda_decoder_step(void *cache, const float *d_x, int32_t act, float *d_out);
dl4s_status dl4s_cuda_decoder_cache_destroy(void *cache);
/* x[b,:] = E[ids[b * ids_stride]] * sqrt(D) + PE[position,:]: Transformer.prepareInputs (Transformer.swift:82-88)
 * for the one token per sequence a decoding step feeds back; the ids stay on the device. */
dl4s_status dl4s_cuda_embed_at(const int32_t *d_ids, int64_t ids_stride, int64_t B, int64_t position, int64_t D,
                               const float *d_embedding, int64_t vocab, int32_t ignore_index, float *d_out);

/* Transformer.callAsFunction(inputSequence:startToken:endToken:maxLength:) (Transformer.swift:118-137): greedy
 * decoding of one sequence. input_ids (host, n_in tokens) go through embedding + positional encoding and the
 * encoder; then, per step, the decoder's last row is multiplied with the tied embedding matrix (no bias, no
 * softmax, as in :127-129) and the arg-max token is appended, until end_token or max_length tokens. The tokens stay
 * on the device between steps (the host looks at them every 8 steps to stop early). tokens (host) must hold
 * max_length entries; the end token, if produced, is the last one counted in *n_tokens, as in the reference.
 *   cached = 0  the reference's schedule: the decoder is re-run on [start] + tokens for every step
 *               (dl4s_cuda_decoder_forward; `precision` selects its arithmetic). Token-for-token what DL4S computes.
 *   cached = 1  one dl4s_cuda_decoder_step per token with key/value caches (fp32): one token of work per step,
 *               per-token LayerNorm statistics (see above), so the sequence may differ from cached = 0. */
dl4s_status dl4s_cuda_transformer_greedy_decode(const int32_t *input_ids, int64_t n_in, int32_t start_token, int32_t end_token,
                                                int64_t max_length, int64_t vocab, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                                int64_t F, int64_t enc_layers, int64_t dec_layers, const float *d_embedding,
                                                const float *d_enc_params, const float *d_dec_params, int32_t act,
                                                int32_t precision, int32_t cached, int32_t *tokens, int64_t *n_tokens);

/* Output head of the Transformer (NN/Models/Transformer/Transformer.swift:105-108):
 *   d_out [M, V] = logSoftmax(d_x [M, D] . d_embedding[V, D]^T + d_bias [V]) over the vocabulary,
 * with the (tied) embedding matrix as the projection (Matrix.swift:79-117 with transposeOther) and logSoftmax as
 * in Tensor/Operators/Unary.swift:198-204. d_bias may be NULL. DL4S_PREC_F16 runs the product on the tensor
 * cores when M >= 128 and V, D are multiples of 64; the log-softmax is fp32 in place on the logits.
 * dl4s_cuda_log_softmax_rows is that last step alone (d_out may equal d_x). Greedy decoding takes the argmax of
 * a row with dl4s_cuda_reduce_max's index output (Transformer.swift:130). */
dl4s_status dl4s_cuda_output_head(const float *d_x, int64_t M, int64_t D, const float *d_embedding, int64_t V,
                                  const float *d_bias, float *d_out, int32_t precision);
dl4s_status dl4s_cuda_log_softmax_rows(const float *d_x, int64_t rows, int64_t n, float *d_out);

/* PointwiseFeedForward.callAsFunction (NN/Models/Transformer/PointwiseFeedForward.swift:67-82):
 * out = LayerNorm_row( act(x W1 + b1) W2 + b2 + x ), x [M,D], W1 [D,F], W2 [F,D]. */
dl4s_status dl4s_cuda_ffn_forward(const float *d_x, int64_t M, int64_t D, int64_t F,
                                  const float *d_w1, const float *d_b1, const float *d_w2, const float *d_b2,
                                  const float *d_ln_scale, const float *d_ln_shift, int32_t act,
                                  float *d_out, int32_t precision);

/* TransformerEncoder.callAsFunction (NN/Models/Transformer/TransformerEncoder.swift:61-71):
 * `layers` blocks of FFN(MHA(x,x,x,padding mask)). d_params holds, per layer and
 * in this order: Wq, Wk [D,H*dk], Wv [D,H*dv], Wo [H*dv,D], ln1_scale, ln1_shift
 * [D], W1 [D,F], b1 [F], W2 [F,D], b2 [D], ln2_scale, ln2_shift [D].
 * d_lengths[B] may be NULL (no padding). */
dl4s_status dl4s_cuda_encoder_forward(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H,
                                      int64_t dk, int64_t dv, int64_t F, int64_t layers,
                                      const float *d_params, const int32_t *d_lengths, int32_t act,
                                      float *d_out, int32_t precision);

/* The same forward with the tensor-core weights converted once instead of on every call. DL4S keeps parameters as
 * fp32 tensors (TransformerEncoder.swift:29-59); the half (or two-half) copies the tensor cores read do not change
 * between inference calls, so a caller prepares them once per model:
 *   prepare  converts Wq|Wk|Wv, Wo, W1, W2 of all layers of d_params (layout as above) for `precision`
 *            (DL4S_PREC_F16 or DL4S_PREC_F16_SPLIT) into device memory owned by the handle. d_params must stay
 *            valid: biases and LayerNorm parameters are read from it on every forward.
 *   refresh  converts again after the parameters changed (an optimiser step).
 *   forward  is dl4s_cuda_encoder_forward without the conversion pass; shapes outside the tensor-core pipeline
 *            are refused with DL4S_ERR_UNSUPPORTED.
 *   destroy  frees the copies (after graphs that recorded a forward with them are destroyed). */
dl4s_status dl4s_cuda_encoder_prepare(int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int64_t layers,
                                      const float *d_params, int32_t precision, void **prepared);
dl4s_status dl4s_cuda_encoder_prepared_refresh(void *prepared);
dl4s_status dl4s_cuda_encoder_prepared_destroy(void *prepared);
dl4s_status dl4s_cuda_encoder_forward_prepared(void *prepared, const float *d_x, int64_t B, int64_t S,
                                               const int32_t *d_lengths, int32_t act, float *d_out);

/* Transformer.prepareInputs (NN/Models/Transformer/Transformer.swift:82-88) with
 * Embedding (NN/Layer/Embedding.swift:152-165) and PositionalEncoding
 * (PositionalEncoding.swift:52-71): x[b,s,:] = E[ids[b,s]]*sqrt(D) + PE[s,:];
 * an id equal to ignore_index embeds as zeros. */
dl4s_status dl4s_cuda_embed_positional(const int32_t *d_ids, int64_t B, int64_t S, int64_t D,
                                       const float *d_embedding, int64_t vocab, int32_t ignore_index,
                                       float *d_out);

#ifdef __cplusplus
}
#endif
#endif /* DL4S_CUDA_H */
