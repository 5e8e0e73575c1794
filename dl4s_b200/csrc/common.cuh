// Shared host-side state and helpers of libdl4s_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/dl4s_cuda.h"

namespace dl4s {

constexpr int kMaxDevices = 16;
constexpr int kLnPartialSlots = 1 << 20;   // 16 MB: one pair of sums per 32 rows x column part of the largest fused-statistics product
constexpr int kTileCounterSlots = 64;
constexpr int kMaxRetired = 64;            // internal buffers kept for live graphs, see DeviceState::retired

// Per-device state. The scratch arena is grow-only and reused by every fused
// call on the device's stream (stream order makes reuse safe).
struct DeviceState {
    bool live = false;
    int ordinal = -1;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;  // own_stream or a caller-provided one
    void *arena = nullptr;
    size_t arena_bytes = 0;
    int32_t *status_word = nullptr;  // device word set by bounded waits that gave up
    double *ln_partials = nullptr;   // kLnPartialSlots x 2 partial sums of the chunked LayerNorm
    // Work counters of the persistent GEMM: kTileCounterSlots x {next tile, CTAs done}. A launch takes the
    // next slot; the last CTA to leave zeroes its slot again.
    int32_t *tile_counters = nullptr;
    int tile_counter_next = 0;
    // Split-K partial sums of the few-rows fp32 GEMM (grow-only, separate from the arena because callers
    // lay out the arena themselves around their GEMM calls).
    float *skinny_partials = nullptr;
    size_t skinny_bytes = 0;
    // Programmatic dependent launch between the kernels of the tensor-core pipelines (DL4S_PDL=0 turns it off).
    bool pdl = true;
    // Graph capture (dl4s_cuda_graph_begin/end): calls are recorded instead of run; nothing that would
    // allocate or wait may happen in between.
    bool capturing = false;
    uint64_t launches_at_capture_begin = 0;
    // Graphs returned by dl4s_cuda_graph_end and not yet destroyed. Their kernels hold the addresses of the
    // internal buffers (arena, skinny_partials, pe_table) as they were at capture time, so while any graph
    // lives a buffer that has to grow is retired (kept allocated) instead of freed; the retired buffers go
    // when the last graph is destroyed.
    int live_graphs = 0;
    // Tensor-core GEMMs take their tiles from a device-wide counter (1) instead of a fixed round-robin schedule (0).
    // Set while the launches share the SMs with a collective's kernel, where a CTA that starts late should take
    // fewer tiles; otherwise the fixed schedule saves the counter's round trips.
    int dynamic_tiles = 0;
    void *retired[kMaxRetired] = {};
    int n_retired = 0;
    // Sinusoidal positional-encoding table [pe_rows, pe_dim], built on first use and kept.
    float *pe_table = nullptr;
    int64_t pe_rows = 0, pe_dim = 0;
    int sm_count = 0;
    uint64_t launches = 0;
    bool timing = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    // Dropout (dl4s_cuda_set_dropout): rate 0 = inactive. Every site that applies dropout takes the next counter
    // value, so masks differ between sites, layers and calls and a host can regenerate any of them.
    float dropout_rate = 0.f;
    uint64_t dropout_seed = 0;
    uint32_t dropout_counter = 0;
    // Operation-group trace (dl4s_cuda_set_trace): NVTX ranges + a host-side list of the group paths entered.
    bool tracing = false;
    int trace_depth = 0;
    const char *trace_stack[16] = {};
    char *trace_log = nullptr;      // kTraceLogBytes, newline-separated "A/B/C" paths
    size_t trace_len = 0;
    // Per-kernel profile (dl4s_cuda_profile_begin/end): one event after every launch.
    bool profiling = false;
    int prof_n = 0;                       // launches recorded; event prof_n closes the last one
    cudaEvent_t *prof_events = nullptr;   // kMaxProfileLaunches + 1 events, created on first use
    const char **prof_names = nullptr;
};
constexpr int kMaxProfileLaunches = 4096;
constexpr size_t kTraceLogBytes = 1 << 16;

// The operation groups of the reference (OperationGroup.capture(named:), Tensor/Graph.swift:134-163: "Encoder",
// "EncoderLayer", "MultiHeadAttention", "ScaledDotProductAttention", "PointwiseFeedForward", "LayerNorm", ...) as
// NVTX ranges around the launches they cover, when tracing is on.
void trace_push(DeviceState *st, const char *name);
void trace_pop(DeviceState *st);
struct ScopedGroup {
    DeviceState *st;
    ScopedGroup(DeviceState *s, const char *name) : st(s) { if (st->tracing) trace_push(st, name); }
    ~ScopedGroup() { if (st->tracing) trace_pop(st); }
};

// Failure injection for tests (dl4s_cuda_inject_failure): true when a pending injected failure of kind `what` was
// consumed by this call.
bool take_injected_failure(int what);
void profile_record(DeviceState *st, const char *name);

DeviceState *current();                 // nullptr (and last error set) when not initialised
dl4s_status fail(dl4s_status code, const char *fmt, ...);
dl4s_status check_cuda(cudaError_t e, const char *what);
// Returns a pointer to at least `bytes` of device scratch (256-byte aligned).
dl4s_status arena_reserve(DeviceState *st, size_t bytes, void **ptr);
// Frees an internal buffer that is being replaced, or keeps it for the graphs that still name its address.
dl4s_status release_internal(DeviceState *st, void *ptr);

#define DL4S_CUDA_TRY(expr)                                            \
    do {                                                               \
        cudaError_t _e = (expr);                                       \
        if (_e != cudaSuccess) return ::dl4s::check_cuda(_e, #expr);   \
    } while (0)

#define DL4S_TRY(expr)                         \
    do {                                       \
        dl4s_status _s = (expr);               \
        if (_s != DL4S_OK) return _s;          \
    } while (0)

#define DL4S_REQUIRE(cond, ...)                                              \
    do {                                                                     \
        if (!(cond)) return ::dl4s::fail(DL4S_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

#define DL4S_STATE(st)                      \
    ::dl4s::DeviceState *st = ::dl4s::current(); \
    if (!st) return DL4S_ERR_NOT_INITIALIZED

// Counts the launch and surfaces launch-configuration errors at once.
inline dl4s_status after_launch(DeviceState *st, const char *name)
{
    st->launches++;
    if (st->profiling && !st->capturing) profile_record(st, name);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(e, name);
    return DL4S_OK;
}

struct ScopedTimer {
    DeviceState *st;
    explicit ScopedTimer(DeviceState *s) : st(s)
    {
        if (st->timing && !st->capturing) cudaEventRecord(st->ev0, st->stream);
    }
    ~ScopedTimer()
    {
        if (st->timing && !st->capturing) {
            cudaEventRecord(st->ev1, st->stream);
            cudaEventSynchronize(st->ev1);
            cudaEventElapsedTime(&st->last_ms, st->ev0, st->ev1);
        }
    }
};

// ---- device status word (read and cleared by dl4s_cuda_device_status) ----
// 0x001-0x100: a bounded wait of a tensor-core kernel gave up; 0x200: a decode step found its cache full;
// 0x400: a value became infinite (or was not finite to begin with) when the tensor-core path rounded it to IEEE
// half, i.e. an operand outside |x| < 65504.
constexpr int32_t kStatusAttnTimeout = 0x080;   // k_attn_prefill_tc
constexpr int32_t kStatusGemmTimeout = 0x100;   // k_gemm_tc
constexpr int32_t kStatusTimeoutMask = 0x1FF;
constexpr int32_t kStatusCacheFull = 0x200;
constexpr int32_t kStatusHalfRange = 0x400;
#ifdef __CUDACC__
// True when either half of a packed half2 has all exponent bits set (inf or NaN).
__device__ __forceinline__ bool half2_not_finite(uint32_t h)
{
    return ((h & 0x7C00u) == 0x7C00u) | ((h & 0x7C000000u) == 0x7C000000u);
}
// Four floats as packed halves (hi) and the packed half-rounded remainders v - hi (lo).
__device__ __forceinline__ void split_hilo(const float4 &v, uint2 &hi, uint2 &lo)
{
    const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
    const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
    const __half2 l0 = __floats2half2_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
    hi.x = *reinterpret_cast<const uint32_t *>(&h0);
    hi.y = *reinterpret_cast<const uint32_t *>(&h1);
    lo.x = *reinterpret_cast<const uint32_t *>(&l0);
    lo.y = *reinterpret_cast<const uint32_t *>(&l1);
}
#endif

// ---- dropout (NN/Layer/Dropout.swift:47-55: inputs * bernoulli(1 - rate), no rescaling) ----
// The reference draws the mask on the host from a process-global generator (Random.swift:148-157) and copies it to
// the device per call. Here element i of site `counter` is kept when a counter-based hash of (seed, counter, i) is
// below threshold = (1 - rate) * 2^32: no state, no mask in memory, and the host can compute the same bits.
struct DropoutSpec {
    uint32_t threshold = 0;   // 0: dropout inactive, everything is kept
    uint32_t seed_lo = 0, seed_hi = 0, counter = 0;
};
__host__ __device__ __forceinline__ uint32_t dropout_hash(uint64_t index, uint32_t seed_lo, uint32_t seed_hi, uint32_t counter)
{
    uint32_t h = (uint32_t)index * 0x9E3779B1u + seed_lo;
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    h += ((uint32_t)(index >> 32) ^ counter) * 0x27D4EB2Fu + seed_hi;
    h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
    return h;
}
__host__ __device__ __forceinline__ bool dropout_keep(const DropoutSpec &d, uint64_t index)
{
    return d.threshold == 0 || dropout_hash(index, d.seed_lo, d.seed_hi, d.counter) < d.threshold;
}

// ---- programmatic dependent launch ----
// Kernels of one pipeline are launched with the programmatic-serialization attribute: the next kernel's CTAs may
// be scheduled (and run their prologue: barrier set-up, tensor-memory allocation) while the previous kernel is
// still draining, and wait in pdl_wait() — which returns when the previous kernel has finished and its writes are
// visible — before they touch global memory. Every kernel launched this way calls pdl_wait() before its first
// global access; a kernel that skipped it would race with its predecessor. Without the attribute both calls
// do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(DeviceState *st, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                              Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st->stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    // Inside a graph the kernel-to-kernel edges are already tight; measured, the early-resident CTAs only cost there.
    if (st->pdl && !st->capturing) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// The spec of the next dropout site on this device (inactive when the rate is 0); takes one counter value.
inline DropoutSpec next_dropout(DeviceState *st)
{
    DropoutSpec d;
    if (st->dropout_rate > 0.f) {
        double keep = (1.0 - (double)st->dropout_rate) * 4294967296.0;
        d.threshold = keep >= 4294967295.0 ? 0xFFFFFFFFu : (keep < 1.0 ? 1u : (uint32_t)keep);
        d.seed_lo = (uint32_t)st->dropout_seed;
        d.seed_hi = (uint32_t)(st->dropout_seed >> 32);
        d.counter = st->dropout_counter++;
    }
    return d;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

// ---- internal kernels shared between translation units (host launchers) ----

// Strides (in elements) of a 4-D logical tensor [B,H,S,d] with unit inner stride.
struct Strides4 {
    int64_t b, h, s;
};
inline Strides4 strides_bhsd(int64_t H, int64_t S, int64_t d) { return {H * S * d, S * d, d}; }
inline Strides4 strides_bshd(int64_t H, int64_t S, int64_t d) { return {S * H * d, d, H * d}; }

struct MaskSpec {
    const int32_t *d_key_lengths = nullptr;
    int causal = 0;
    const float *d_mask = nullptr;
    int64_t ms[4] = {1, 1, 1, 1};
};

// attn_ref.cu — fp32 FFMA attention (check kernel, general masks).
dl4s_status launch_attn_ref(DeviceState *st, const float *q, Strides4 qs, const float *k, Strides4 ks,
                            const float *v, Strides4 vs, float *o, Strides4 os, int64_t B, int64_t H,
                            int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, float inv_temperature,
                            const MaskSpec &mask);

// attn_decode.cu
dl4s_status launch_attn_decode(DeviceState *st, const float *q, const float *k, const float *v, int64_t B,
                               int64_t H, int64_t Lmax, int64_t dk, int64_t dv, float inv_temperature,
                               const int32_t *d_key_lengths, float *out, float *scratch, int64_t chunk,
                               int64_t nsplit);

// fused.cu: dl4s_cuda_mha_heads_forward with an optional half copy of the input held by the caller.
dl4s_status mha_heads_forward_impl(const float *d_xq, const float *d_xk, const float *d_xv, int64_t B, int64_t Sq, int64_t Sk,
                                   int64_t D, int64_t Hl, int64_t dk, int64_t dv, const float *d_wq, const float *d_wk,
                                   const float *d_wv, const int32_t *d_key_lengths, int32_t causal, void *d_heads_out,
                                   int32_t precision, int32_t half_output, const void *d_x_half);
// gemm_tc.cu: fp32 -> half, 16-byte aligned buffers.
dl4s_status launch_f32_to_f16(DeviceState *st, const float *x, void *y, int64_t n);

// comm.cu: frees a device's communicator, second stream and gather buffers.
void comm_release_device(int ordinal);

// Resolves the fixed split-K array of dl4s_cuda_sdpa_decode_noalloc and loads the decode kernels (device current).
dl4s_status decode_static_prepare(DeviceState *st);

// gemm_f32.cu — C = alpha*op(A)op(B) + beta*C with a fused epilogue.
enum Epilogue { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_BIAS_RELU = 3, EPI_BIAS_RESIDUAL = 4, EPI_RESIDUAL = 5 };
// `drop`: dropout of the product (+ bias) before the residual is added, for the residual flavours.
dl4s_status launch_gemm_f32(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N,
                            int64_t K, float alpha, float beta, int trans_a, int trans_b, int epilogue,
                            const float *bias, const float *residual, const DropoutSpec *drop = nullptr);

// fused.cu: the sinusoidal positional-encoding table of the device covers at least `rows` positions of width D.
dl4s_status ensure_positional_table(DeviceState *st, int64_t rows, int64_t D);

// layernorm.cu
dl4s_status launch_layernorm(DeviceState *st, const float *x, const float *residual, int64_t outer,
                             int64_t rows, int64_t D, const float *scale, const float *shift, float *out,
                             void *out_half = nullptr);

// LayerNorm over [rows, D] blocks whose partial sums a GEMM epilogue already wrote (tc.cuh: EPI_RESIDUAL_STATS).
bool layernorm_stats_usable(int64_t outer, int64_t rows, int64_t D, int parts_per_row_block);
dl4s_status launch_layernorm_from_stats(DeviceState *st, const float *x, int64_t outer, int64_t rows, int64_t D,
                                        const float *scale, const float *shift, float *out, void *out_half,
                                        const double *stats, int parts_per_row_block);

}  // namespace dl4s
