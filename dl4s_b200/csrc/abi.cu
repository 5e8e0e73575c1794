// Lifecycle, error reporting and MemoryOperatorsType entry points.
#include "common.cuh"

#include <cstdlib>

#include <atomic>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

namespace dl4s {

static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;
static thread_local int t_current = -1;
static thread_local char t_err[512] = "";

dl4s_status fail(dl4s_status code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

dl4s_status check_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return DL4S_OK;
    dl4s_status code = (e == cudaErrorMemoryAllocation) ? DL4S_ERR_OOM : DL4S_ERR_CUDA;
    return fail(code, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

DeviceState *current()
{
    if (t_current < 0) {
        // A thread that did not pick a device uses the first live one.
        for (int i = 0; i < kMaxDevices; ++i)
            if (g_dev[i].live) { t_current = i; break; }
    }
    if (t_current < 0 || !g_dev[t_current].live) {
        fail(DL4S_ERR_NOT_INITIALIZED, "dl4s_cuda_init has not been called (or failed) for this device");
        return nullptr;
    }
    cudaSetDevice(g_dev[t_current].ordinal);
    return &g_dev[t_current];
}

dl4s_status arena_reserve(DeviceState *st, size_t bytes, void **ptr)
{
    if (bytes > st->arena_bytes) {
        if (st->capturing)
            return fail(DL4S_ERR_UNSUPPORTED, "the scratch arena would have to grow (%zu > %zu bytes) while a graph is being "
                        "captured: run the same calls once before dl4s_cuda_graph_begin", bytes, st->arena_bytes);
        // Everything that used the old arena was enqueued before this call.
        DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
        DL4S_TRY(release_internal(st, st->arena));
        st->arena = nullptr;
        st->arena_bytes = 0;
        size_t want = align_up(bytes + bytes / 8, (size_t)1 << 20);
        DL4S_CUDA_TRY(cudaMalloc(&st->arena, want));
        st->arena_bytes = want;
    }
    *ptr = st->arena;
    return DL4S_OK;
}

dl4s_status release_internal(DeviceState *st, void *ptr)
{
    if (!ptr) return DL4S_OK;
    if (st->live_graphs > 0) {
        // A graph recorded earlier replays kernels that read and write this buffer.
        if (st->n_retired == kMaxRetired)
            return fail(DL4S_ERR_UNSUPPORTED, "%d internal buffers are already kept alive for recorded graphs: destroy the graphs "
                        "(dl4s_cuda_graph_destroy) before running larger shapes", kMaxRetired);
        st->retired[st->n_retired++] = ptr;
        return DL4S_OK;
    }
    DL4S_CUDA_TRY(cudaFree(ptr));
    return DL4S_OK;
}

static std::atomic<int> g_inject[8];

bool take_injected_failure(int what)
{
    if (what < 1 || what >= 8) return false;
    int n = g_inject[what].load();
    while (n > 0) {
        if (g_inject[what].compare_exchange_weak(n, n - 1)) return true;
    }
    return false;
}

void trace_push(DeviceState *st, const char *name)
{
    nvtxRangePushA(name);
    if (st->trace_depth < 16) st->trace_stack[st->trace_depth] = name;
    st->trace_depth++;
    if (!st->trace_log) return;
    // append the path "A/B/C\n" if it fits
    size_t need = 1;
    const int depth = st->trace_depth < 16 ? st->trace_depth : 16;
    for (int i = 0; i < depth; ++i) need += strlen(st->trace_stack[i]) + 1;
    if (st->trace_len + need >= kTraceLogBytes) return;
    for (int i = 0; i < depth; ++i) {
        size_t n = strlen(st->trace_stack[i]);
        memcpy(st->trace_log + st->trace_len, st->trace_stack[i], n);
        st->trace_len += n;
        st->trace_log[st->trace_len++] = (i + 1 < depth) ? '/' : '\n';
    }
    st->trace_log[st->trace_len] = 0;
}

void trace_pop(DeviceState *st)
{
    nvtxRangePop();
    if (st->trace_depth > 0) st->trace_depth--;
}

void profile_record(DeviceState *st, const char *name)
{
    if (st->prof_n >= kMaxProfileLaunches) return;
    st->prof_names[st->prof_n] = name;
    st->prof_n++;
    cudaEventRecord(st->prof_events[st->prof_n], st->stream);
}

static dl4s_status init_one(int ordinal)
{
    DeviceState &d = g_dev[ordinal];
    if (d.live) return DL4S_OK;
    DL4S_CUDA_TRY(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    DL4S_CUDA_TRY(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(DL4S_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library contains sm_100a code only",
                    ordinal, prop.major, prop.minor);
    d.ordinal = ordinal;
    d.sm_count = prop.multiProcessorCount;
    DL4S_CUDA_TRY(cudaStreamCreateWithFlags(&d.own_stream, cudaStreamNonBlocking));
    d.stream = d.own_stream;
    DL4S_CUDA_TRY(cudaMalloc((void **)&d.status_word, sizeof(int32_t)));
    DL4S_CUDA_TRY(cudaMemset(d.status_word, 0, sizeof(int32_t)));
    DL4S_CUDA_TRY(cudaMalloc((void **)&d.ln_partials, sizeof(double) * 2 * kLnPartialSlots));
    DL4S_CUDA_TRY(cudaMalloc((void **)&d.tile_counters, sizeof(int32_t) * 2 * kTileCounterSlots));
    DL4S_CUDA_TRY(cudaMemset(d.tile_counters, 0, sizeof(int32_t) * 2 * kTileCounterSlots));
    DL4S_CUDA_TRY(cudaEventCreate(&d.ev0));
    DL4S_CUDA_TRY(cudaEventCreate(&d.ev1));
    d.launches = 0;
    // The no-allocation decode entry point must find its array and kernels resident: take them now.
    DL4S_TRY(decode_static_prepare(&d));
    {
        const char *e = getenv("DL4S_PDL");
        d.pdl = !(e && e[0] == '0');
        // DL4S_CUDA_TRACE=1: operation-group ranges from the start (see dl4s_cuda_set_trace)
        const char *t = getenv("DL4S_CUDA_TRACE");
        if (t && t[0] == '1') {
            d.trace_log = new char[kTraceLogBytes];
            d.trace_log[0] = 0;
            d.trace_len = 0;
            d.tracing = true;
        }
    }
    d.live = true;
    return DL4S_OK;
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_device_count(int32_t *count)
{
    if (!count) return fail(DL4S_ERR_INVALID_ARG, "count is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { *count = 0; return check_cuda(e, "cudaGetDeviceCount"); }
    *count = n;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_init(const int32_t *devices, int32_t n)
{
    std::lock_guard<std::mutex> lk(g_mu);
    int32_t count = 0;
    DL4S_TRY(dl4s_cuda_device_count(&count));
    if (count == 0) return fail(DL4S_ERR_CUDA, "no CUDA device is visible; this library has no CPU fallback");
    int32_t dflt = 0;
    if (n <= 0 || !devices) { devices = &dflt; n = 1; }
    for (int i = 0; i < n; ++i) {
        if (devices[i] < 0 || devices[i] >= count || devices[i] >= kMaxDevices)
            return fail(DL4S_ERR_INVALID_ARG, "device ordinal %d out of range (0..%d)", devices[i], count - 1);
        DL4S_TRY(init_one(devices[i]));
    }
    t_current = devices[0];
    cudaSetDevice(devices[0]);
    return DL4S_OK;
}

dl4s_status dl4s_cuda_shutdown(void)
{
    std::lock_guard<std::mutex> lk(g_mu);
    for (int i = 0; i < kMaxDevices; ++i) {
        DeviceState &d = g_dev[i];
        if (!d.live) continue;
        cudaSetDevice(d.ordinal);
        cudaStreamSynchronize(d.stream);
        comm_release_device(d.ordinal);
        if (d.arena) cudaFree(d.arena);
        for (int r = 0; r < d.n_retired; ++r) cudaFree(d.retired[r]);
        if (d.status_word) cudaFree(d.status_word);
        if (d.ln_partials) cudaFree(d.ln_partials);
        if (d.tile_counters) cudaFree(d.tile_counters);
        if (d.pe_table) cudaFree(d.pe_table);
        if (d.skinny_partials) cudaFree(d.skinny_partials);
        cudaEventDestroy(d.ev0);
        cudaEventDestroy(d.ev1);
        cudaStreamDestroy(d.own_stream);
        delete[] d.trace_log;
        d = DeviceState();
    }
    t_current = -1;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_set_device(int32_t device)
{
    if (device < 0 || device >= kMaxDevices || !g_dev[device].live)
        return fail(DL4S_ERR_NOT_INITIALIZED, "device %d was not passed to dl4s_cuda_init", device);
    t_current = device;
    DL4S_CUDA_TRY(cudaSetDevice(device));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_get_device(int32_t *device)
{
    DL4S_STATE(st);
    *device = st->ordinal;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_sync(void)
{
    DL4S_STATE(st);
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_set_stream(void *cuda_stream)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(!st->capturing, "the stream cannot change while a graph is being captured");
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    st->stream = cuda_stream ? (cudaStream_t)cuda_stream : st->own_stream;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_get_stream(void **cuda_stream)
{
    DL4S_STATE(st);
    *cuda_stream = (void *)st->stream;
    return DL4S_OK;
}

const char *dl4s_cuda_last_error(void) { return t_err; }

int32_t dl4s_cuda_version(void) { return DL4S_CUDA_VERSION; }

dl4s_status dl4s_cuda_device_status(int32_t *status_word)
{
    DL4S_STATE(st);
    int32_t w = 0;
    DL4S_CUDA_TRY(cudaMemcpyAsync(&w, st->status_word, sizeof(w), cudaMemcpyDeviceToHost, st->stream));
    DL4S_CUDA_TRY(cudaMemsetAsync(st->status_word, 0, sizeof(w), st->stream));
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    if (status_word) *status_word = w;
    if (w & kStatusTimeoutMask) return fail(DL4S_ERR_TIMEOUT, "a bounded device-side wait gave up (status word 0x%x)", w);
    if (w & 0xF0000) return fail(DL4S_ERR_TIMEOUT, "a bounded device-side wait gave up (status word 0x%x)", w);
    if (w & kStatusCacheFull) return fail(DL4S_ERR_INVALID_ARG, "a decode step found its key/value cache full (status word 0x%x)", w);
    if (w & kStatusHalfRange)
        return fail(DL4S_ERR_INVALID_ARG, "a tensor-core operand left the IEEE half range (|x| >= 65504 or not finite): the results of "
                    "the calls since the last status read are not usable (status word 0x%x)", w);
    if (w != 0) return fail(DL4S_ERR_CUDA, "unknown device status word 0x%x", w);
    return DL4S_OK;
}

dl4s_status dl4s_cuda_set_timing(int32_t enable)
{
    DL4S_STATE(st);
    st->timing = enable != 0;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_get_timing(float *ms)
{
    DL4S_STATE(st);
    *ms = st->last_ms;
    return DL4S_OK;
}

// ---------------------------------------------------------------------- graphs
struct GraphHandle {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;   // kernels of this library recorded in the graph
    int device = -1;
};

dl4s_status dl4s_cuda_graph_begin(void)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(!st->capturing, "a capture is already open on this device");
    DL4S_REQUIRE(!st->profiling, "end the per-kernel profile before capturing a graph");
    DL4S_CUDA_TRY(cudaStreamBeginCapture(st->stream, cudaStreamCaptureModeThreadLocal));
    st->capturing = true;
    st->launches_at_capture_begin = st->launches;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_graph_end(void **graph)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(st->capturing, "dl4s_cuda_graph_begin was not called");
    st->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(st->stream, &g);
    const uint64_t recorded = st->launches - st->launches_at_capture_begin;
    st->launches = st->launches_at_capture_begin;   // nothing ran
    if (e != cudaSuccess) return check_cuda(e, "cudaStreamEndCapture");
    DL4S_REQUIRE(graph, "graph is NULL");
    GraphHandle *h = new GraphHandle();
    h->graph = g;
    h->kernels = recorded;
    h->device = st->ordinal;
    e = cudaGraphInstantiate(&h->exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        delete h;
        return check_cuda(e, "cudaGraphInstantiate");
    }
    *graph = h;
    st->live_graphs++;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_graph_launch(void *graph)
{
    DL4S_STATE(st);
    GraphHandle *h = static_cast<GraphHandle *>(graph);
    DL4S_REQUIRE(h && h->exec, "not a graph of this library");
    DL4S_REQUIRE(h->device == st->ordinal, "the graph was captured on device %d, the current device is %d", h->device, st->ordinal);
    DL4S_REQUIRE(!st->capturing, "a graph cannot be launched into a capture");
    DL4S_CUDA_TRY(cudaGraphLaunch(h->exec, st->stream));
    st->launches += h->kernels;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_graph_destroy(void *graph)
{
    GraphHandle *h = static_cast<GraphHandle *>(graph);
    if (!h) return DL4S_OK;
    if (h->exec) cudaGraphExecDestroy(h->exec);
    if (h->graph) cudaGraphDestroy(h->graph);
    const int device = h->device;
    delete h;
    // With the last graph of a device gone nothing names the retired internal buffers any more.
    if (device >= 0 && device < kMaxDevices && g_dev[device].live) {
        DeviceState &d = g_dev[device];
        if (d.live_graphs > 0 && --d.live_graphs == 0 && d.n_retired > 0) {
            int prev = -1;
            cudaGetDevice(&prev);
            cudaSetDevice(d.ordinal);
            cudaStreamSynchronize(d.stream);   // a replay may still be running
            for (int r = 0; r < d.n_retired; ++r) cudaFree(d.retired[r]);
            d.n_retired = 0;
            if (prev >= 0) cudaSetDevice(prev);
        }
    }
    return DL4S_OK;
}

dl4s_status dl4s_cuda_profile_begin(void)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(!st->capturing, "the per-kernel profile cannot start inside a graph capture");
    if (!st->prof_events) {
        st->prof_events = new cudaEvent_t[kMaxProfileLaunches + 1];
        st->prof_names = new const char *[kMaxProfileLaunches];
        for (int i = 0; i <= kMaxProfileLaunches; ++i) DL4S_CUDA_TRY(cudaEventCreate(&st->prof_events[i]));
    }
    st->prof_n = 0;
    DL4S_CUDA_TRY(cudaEventRecord(st->prof_events[0], st->stream));
    st->profiling = true;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_profile_end(char *report, size_t capacity)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(st->profiling, "dl4s_cuda_profile_begin was not called");
    st->profiling = false;
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    // Aggregate by kernel name (pointer identity of the literal is enough, strcmp is safer).
    struct Row { const char *name; int n; double ms; };
    Row rows[64];
    int nrows = 0;
    for (int i = 0; i < st->prof_n; ++i) {
        float ms = 0.f;
        DL4S_CUDA_TRY(cudaEventElapsedTime(&ms, st->prof_events[i], st->prof_events[i + 1]));
        int r = 0;
        for (; r < nrows; ++r) if (strcmp(rows[r].name, st->prof_names[i]) == 0) break;
        if (r == nrows) { if (nrows == 64) continue; rows[nrows++] = Row{st->prof_names[i], 0, 0.0}; }
        rows[r].n++;
        rows[r].ms += ms;
    }
    if (report && capacity) {
        size_t off = 0;
        auto put = [&](const char *fmt, auto... a) {
            if (off < capacity) { int w = snprintf(report + off, capacity - off, fmt, a...); if (w > 0) off += (size_t)w; }
        };
        put("{");
        for (int r = 0; r < nrows; ++r)
            put("%s\"%s\": {\"launches\": %d, \"total_ms\": %.6f}", r ? ", " : "", rows[r].name, rows[r].n, rows[r].ms);
        put("}");
        if (off >= capacity) report[capacity - 1] = 0;
    }
    return DL4S_OK;
}

dl4s_status dl4s_cuda_inject_failure(int32_t what, int32_t count)
{
    if (what < 1 || what >= 8) return fail(DL4S_ERR_INVALID_ARG, "unknown failure kind %d", what);
    g_inject[what].store(count > 0 ? count : 0);
    return DL4S_OK;
}

dl4s_status dl4s_cuda_set_trace(int32_t enable)
{
    DL4S_STATE(st);
    if (enable && !st->trace_log) {
        st->trace_log = new char[kTraceLogBytes];
        st->trace_log[0] = 0;
        st->trace_len = 0;
    }
    st->tracing = enable != 0;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_trace_read(char *report, size_t capacity)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(report && capacity > 0, "no room for the report");
    size_t n = st->trace_log ? st->trace_len : 0;
    if (n >= capacity) n = capacity - 1;
    if (n) memcpy(report, st->trace_log, n);
    report[n] = 0;
    st->trace_len = 0;
    if (st->trace_log) st->trace_log[0] = 0;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_launch_count(uint64_t *count)
{
    DL4S_STATE(st);
    *count = st->launches;
    return DL4S_OK;
}

// ---------------------------------------------------------------- memory

dl4s_status dl4s_cuda_malloc(size_t bytes, void **d_ptr)
{
    if (take_injected_failure(DL4S_INJECT_MALLOC)) {
        if (d_ptr) *d_ptr = nullptr;
        return fail(DL4S_ERR_OOM, "injected failure: allocation of %zu bytes refused (dl4s_cuda_inject_failure)", bytes);
    }
    DL4S_STATE(st);
    DL4S_REQUIRE(d_ptr, "d_ptr is NULL");
    *d_ptr = nullptr;
    if (bytes == 0) bytes = 16;  // DL4S allocates zero-capacity buffers for scalars' shapes
    if (st->capturing) return fail(DL4S_ERR_UNSUPPORTED, "allocate buffers before dl4s_cuda_graph_begin, not during capture");
    DL4S_CUDA_TRY(cudaMallocAsync(d_ptr, bytes, st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_free(void *d_ptr)
{
    DL4S_STATE(st);
    if (!d_ptr) return DL4S_OK;
    if (st->capturing) return fail(DL4S_ERR_UNSUPPORTED, "free buffers after dl4s_cuda_graph_end, not during capture");
    DL4S_CUDA_TRY(cudaFreeAsync(d_ptr, st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_h2d(void *d_dst, const void *src, size_t bytes)
{
    if (take_injected_failure(DL4S_INJECT_H2D))
        return fail(DL4S_ERR_CUDA, "injected failure: host-to-device copy of %zu bytes refused (dl4s_cuda_inject_failure)", bytes);
    DL4S_STATE(st);
    DL4S_REQUIRE(bytes == 0 || (d_dst && src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, st->stream));
    // Pageable sources may be reused by the caller right away.
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_h2d_async(void *d_dst, const void *src, size_t bytes)
{
    if (take_injected_failure(DL4S_INJECT_H2D))
        return fail(DL4S_ERR_CUDA, "injected failure: host-to-device copy of %zu bytes refused (dl4s_cuda_inject_failure)", bytes);
    DL4S_STATE(st);
    DL4S_REQUIRE(bytes == 0 || (d_dst && src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_d2h(void *dst, const void *d_src, size_t bytes)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(bytes == 0 || (dst && d_src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, st->stream));
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_d2h_async(void *dst, const void *d_src, size_t bytes)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(bytes == 0 || (dst && d_src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, st->stream));
    return DL4S_OK;
}

// Copies on a stream of the caller's, leaving the library's stream alone: the read-back of one step can run on a
// copy engine while the next step computes. Ordering against the library's stream is the caller's (events).
dl4s_status dl4s_cuda_memcpy_h2d_async_on(void *d_dst, const void *src, size_t bytes, void *cuda_stream)
{
    DL4S_STATE(st);
    (void)st;
    DL4S_REQUIRE(bytes == 0 || (d_dst && src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(d_dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)cuda_stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_d2h_async_on(void *dst, const void *d_src, size_t bytes, void *cuda_stream)
{
    DL4S_STATE(st);
    (void)st;
    DL4S_REQUIRE(bytes == 0 || (dst && d_src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)cuda_stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_memcpy_d2d(void *d_dst, const void *d_src, size_t bytes)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(bytes == 0 || (d_dst && d_src), "NULL pointer");
    DL4S_CUDA_TRY(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, st->stream));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_host_alloc(size_t bytes, void **ptr)
{
    DL4S_STATE(st);
    (void)st;
    DL4S_REQUIRE(ptr, "ptr is NULL");
    DL4S_CUDA_TRY(cudaHostAlloc(ptr, bytes ? bytes : 16, cudaHostAllocDefault));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_host_free(void *ptr)
{
    DL4S_STATE(st);
    (void)st;
    if (ptr) DL4S_CUDA_TRY(cudaFreeHost(ptr));
    return DL4S_OK;
}

dl4s_status dl4s_cuda_get_value_f32(const float *d_src, float *value)
{
    return dl4s_cuda_memcpy_d2h(value, d_src, sizeof(float));
}

dl4s_status dl4s_cuda_set_value_f32(float *d_dst, float value)
{
    return dl4s_cuda_fill_f32(value, d_dst, 1);
}

}  // extern "C"
