// A MultiHeadAttention layer whose heads span the GPUs of one node.
//
// DL4S is single-device. Attention is independent per (batch, head) — the reference loops over them
// (Tensor/Operators/Matrix.swift:106-114) — so the layer splits like this over G ranks (one process or thread
// per GPU, each with its own current device):
//   rank g   holds the columns of Wq/Wk/Wv of heads [g*H/G, (g+1)*H/G) (column-parallel projections, no
//            communication) and runs projections + attention on its heads for the whole batch
//            (MultiHeadAttention.swift:109-119) -> O_g [B, S, (H/G)*dv], written straight into slot g of a
//            rank-major gather buffer [G, B, S, (H/G)*dv];
//   all      ONE collective: ncclAllGather in place over NVLink;
//   rank g   applies Wo, the residual and DL4S's LayerNorm (:121-124) to ITS batch slice (the LayerNorm
//            normalises a whole [S, D] block per batch element, so the second half is split by batch), reading
//            the gather buffer where NCCL left it (a 3-D tensor map walks the G column groups).
// The batch is worked through in chunks, each a complete small layer: the gather of chunk c runs on a second
// stream while chunk c+1's projections and attention compute (launch order on the compute stream:
// H0 H1 O0 H2 O1 ... O_last). On the tensor-core path the head outputs are produced, gathered and consumed as
// IEEE half. All data lies in local HBM before a kernel of this library reads it: no kernel reads peer memory.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, or the path in DL4S_NCCL_LIB), so the library loads and
// runs on hosts without it; only these entry points then fail, with DL4S_ERR_NCCL.
#include "common.cuh"

#include <dlfcn.h>

#include <cstdlib>

namespace dl4s {

// The part of NCCL's public C interface used here (nccl.h): an opaque communicator, a 128-byte id passed by
// value, ncclInt8 = 0 (the gather moves bytes).
struct NcclUniqueId { char internal[DL4S_COMM_ID_BYTES]; };
typedef void *NcclComm;
typedef int (*FnGetUniqueId)(NcclUniqueId *);
typedef int (*FnCommInitRank)(NcclComm *, int, NcclUniqueId, int);
typedef int (*FnCommDestroy)(NcclComm);
typedef int (*FnAllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
typedef const char *(*FnGetErrorString)(int);
typedef int (*FnGetVersion)(int *);

struct NcclApi {
    void *handle = nullptr;
    FnGetUniqueId get_unique_id = nullptr;
    FnCommInitRank comm_init_rank = nullptr;
    FnCommDestroy comm_destroy = nullptr;
    FnAllGather all_gather = nullptr;
    FnGetErrorString error_string = nullptr;
    FnGetVersion get_version = nullptr;
    bool tried = false;
};
static NcclApi g_nccl;

static dl4s_status nccl_load()
{
    if (g_nccl.handle) return DL4S_OK;
    if (!g_nccl.tried) {
        g_nccl.tried = true;
        const char *path = getenv("DL4S_NCCL_LIB");
        void *h = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (h) {
            g_nccl.get_unique_id = (FnGetUniqueId)dlsym(h, "ncclGetUniqueId");
            g_nccl.comm_init_rank = (FnCommInitRank)dlsym(h, "ncclCommInitRank");
            g_nccl.comm_destroy = (FnCommDestroy)dlsym(h, "ncclCommDestroy");
            g_nccl.all_gather = (FnAllGather)dlsym(h, "ncclAllGather");
            g_nccl.error_string = (FnGetErrorString)dlsym(h, "ncclGetErrorString");
            g_nccl.get_version = (FnGetVersion)dlsym(h, "ncclGetVersion");
            if (g_nccl.get_unique_id && g_nccl.comm_init_rank && g_nccl.comm_destroy && g_nccl.all_gather && g_nccl.error_string)
                g_nccl.handle = h;
            else
                dlclose(h);
        }
    }
    if (!g_nccl.handle)
        return fail(DL4S_ERR_NCCL, "libnccl.so.2 could not be loaded (%s); set DL4S_NCCL_LIB to its path. Single-GPU entry "
                    "points do not need it", dlerror() ? dlerror() : "symbols missing");
    return DL4S_OK;
}

static dl4s_status nccl_check(int r, const char *what)
{
    if (r == 0) return DL4S_OK;
    return fail(DL4S_ERR_NCCL, "NCCL error %d (%s) in %s", r, g_nccl.error_string ? g_nccl.error_string(r) : "?", what);
}

constexpr int kMaxChunks = 64;

// One rank's membership: the communicator, the second stream the collective runs on, the events that order it
// against the compute stream, and the gather buffers (grow-only).
struct CommState {
    bool live = false;
    int rank = 0, world = 1;
    NcclComm comm = nullptr;
    cudaStream_t stream = nullptr;
    // per chunk: head outputs written (compute stream) / gather finished (second stream) / the compute stream's
    // wait for the gather begins / ends. Timed, so that a caller can ask how long the gathers took and how much of
    // that the compute stream spent waiting (dl4s_cuda_comm_timing).
    cudaEvent_t ready[kMaxChunks] = {}, done[kMaxChunks] = {}, wait0[kMaxChunks] = {}, wait1[kMaxChunks] = {};
    int last_chunks = 0;
    void *gather = nullptr;
    size_t gather_bytes = 0;
    void *xh = nullptr;           // half copy of the replicated input of the current call (tensor-core paths)
    size_t xh_bytes = 0;
};
static CommState g_comm[kMaxDevices];

// Contiguous slice of `n` items for part `i` of `parts`; the first n % parts parts take one extra item.
static void slice_range(int64_t n, int64_t parts, int64_t i, int64_t *lo, int64_t *hi)
{
    const int64_t base = n / parts, extra = n % parts;
    *lo = i * base + (i < extra ? i : extra);
    *hi = *lo + base + (i < extra ? 1 : 0);
}

struct ChunkPlan {
    int64_t c0, c1;     // the chunk's batch range
    int64_t lb0, lb1;   // this rank's slice inside the chunk (relative to c0)
    int64_t out0;       // row of the rank's output buffer where that slice goes
};

static int make_plan(int64_t B, int world, int rank, int chunks, ChunkPlan *plan)
{
    if (chunks < 1) chunks = 1;
    if (chunks > B) chunks = (int)B;
    if (chunks > kMaxChunks) chunks = kMaxChunks;
    int64_t out0 = 0;
    for (int c = 0; c < chunks; ++c) {
        slice_range(B, chunks, c, &plan[c].c0, &plan[c].c1);
        slice_range(plan[c].c1 - plan[c].c0, world, rank, &plan[c].lb0, &plan[c].lb1);
        plan[c].out0 = out0;
        out0 += plan[c].lb1 - plan[c].lb0;
    }
    return chunks;
}

// Everything a CommState owns; leaves it in its initial state. Returns what ncclCommDestroy said.
static dl4s_status comm_release(CommState &c)
{
    if (c.stream) cudaStreamSynchronize(c.stream);
    dl4s_status result = DL4S_OK;
    if (c.comm && g_nccl.comm_destroy) result = nccl_check(g_nccl.comm_destroy(c.comm), "ncclCommDestroy");
    for (int i = 0; i < kMaxChunks; ++i) {
        cudaEvent_t evs[4] = {c.ready[i], c.done[i], c.wait0[i], c.wait1[i]};
        for (cudaEvent_t e : evs) if (e) cudaEventDestroy(e);
    }
    if (c.stream) cudaStreamDestroy(c.stream);
    if (c.gather) cudaFree(c.gather);
    if (c.xh) cudaFree(c.xh);
    c = CommState();
    return result;
}

// dl4s_cuda_shutdown: the device's membership goes with its state (device current, stream already idle).
void comm_release_device(int ordinal)
{
    CommState &c = g_comm[ordinal];
    if (!c.live && !c.gather && !c.xh && !c.stream && !c.comm) return;
    comm_release(c);
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_comm_unique_id(uint8_t *id)
{
    DL4S_REQUIRE(id, "id is NULL");
    DL4S_TRY(nccl_load());
    NcclUniqueId u;
    DL4S_TRY(nccl_check(g_nccl.get_unique_id(&u), "ncclGetUniqueId"));
    memcpy(id, u.internal, DL4S_COMM_ID_BYTES);
    return DL4S_OK;
}

dl4s_status dl4s_cuda_comm_init(int32_t rank, int32_t world, const uint8_t *id)
{
    if (take_injected_failure(DL4S_INJECT_COMM))
        return fail(DL4S_ERR_NCCL, "injected failure: communicator creation refused for rank %d of %d (dl4s_cuda_inject_failure)",
                    rank, world);
    DL4S_STATE(st);
    DL4S_REQUIRE(world >= 1 && rank >= 0 && rank < world, "rank %d is not in a world of %d", rank, world);
    DL4S_REQUIRE(!st->capturing, "join the communicator before dl4s_cuda_graph_begin");
    CommState &c = g_comm[st->ordinal];
    DL4S_REQUIRE(!c.live, "device %d already belongs to a communicator: call dl4s_cuda_comm_destroy first", st->ordinal);
    if (c.gather || c.xh) {   // left by calls made as a world of one before joining
        DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
        if (c.gather) DL4S_CUDA_TRY(cudaFree(c.gather));
        if (c.xh) DL4S_CUDA_TRY(cudaFree(c.xh));
    }
    c = CommState();
    c.rank = rank;
    c.world = world;
    if (world > 1) {
        DL4S_REQUIRE(id, "id is NULL");
        DL4S_TRY(nccl_load());
        // anything that fails from here on releases what has been created so far
        auto create = [&]() -> dl4s_status {
            NcclUniqueId u;
            memcpy(u.internal, id, DL4S_COMM_ID_BYTES);
            DL4S_TRY(nccl_check(g_nccl.comm_init_rank(&c.comm, world, u, rank), "ncclCommInitRank"));
            DL4S_CUDA_TRY(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
            for (int i = 0; i < kMaxChunks; ++i) {
                DL4S_CUDA_TRY(cudaEventCreate(&c.ready[i]));
                DL4S_CUDA_TRY(cudaEventCreate(&c.done[i]));
                DL4S_CUDA_TRY(cudaEventCreate(&c.wait0[i]));
                DL4S_CUDA_TRY(cudaEventCreate(&c.wait1[i]));
            }
            return DL4S_OK;
        };
        const dl4s_status r = create();
        if (r != DL4S_OK) {
            comm_release(c);
            return r;
        }
    }
    c.live = true;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_comm_destroy(void)
{
    DL4S_STATE(st);
    CommState &c = g_comm[st->ordinal];
    if (!c.live && !c.gather && !c.xh) return DL4S_OK;
    cudaStreamSynchronize(st->stream);
    return comm_release(c);
}

dl4s_status dl4s_cuda_comm_info(int32_t *rank, int32_t *world, int32_t *nccl_version)
{
    DL4S_STATE(st);
    const CommState &c = g_comm[st->ordinal];
    if (rank) *rank = c.live ? c.rank : 0;
    if (world) *world = c.live ? c.world : 1;
    if (nccl_version) {
        *nccl_version = 0;
        if (g_nccl.handle && g_nccl.get_version) {
            int v = 0;
            if (g_nccl.get_version(&v) == 0) *nccl_version = v;
        }
    }
    return DL4S_OK;
}

dl4s_status dl4s_cuda_comm_timing(float *gather_ms, float *exposed_ms)
{
    DL4S_STATE(st);
    CommState &c = g_comm[st->ordinal];
    float g = 0.f, e = 0.f;
    if (c.live && c.last_chunks > 0) {
        DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
        DL4S_CUDA_TRY(cudaStreamSynchronize(c.stream));
        for (int i = 0; i < c.last_chunks; ++i) {
            float ms = 0.f;
            DL4S_CUDA_TRY(cudaEventElapsedTime(&ms, c.ready[i], c.done[i]));
            g += ms;
            DL4S_CUDA_TRY(cudaEventElapsedTime(&ms, c.wait0[i], c.wait1[i]));
            e += ms;
        }
    }
    if (gather_ms) *gather_ms = g;
    if (exposed_ms) *exposed_ms = e;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_mha_sharded_plan(int64_t B, int32_t world, int32_t rank, int32_t chunks, int64_t *rows, int64_t *batch_index)
{
    // Pure host arithmetic: needs no device, so a launcher can size its buffers before anything is initialised.
    DL4S_REQUIRE(B >= 1 && rows, "bad arguments");
    DL4S_REQUIRE(world >= 1 && rank >= 0 && rank < world, "rank %d is not in a world of %d", rank, world);
    ChunkPlan plan[kMaxChunks];
    const int n = make_plan(B, world, rank, world > 1 ? chunks : 1, plan);
    int64_t total = 0;
    for (int i = 0; i < n; ++i) {
        for (int64_t b = plan[i].lb0; b < plan[i].lb1; ++b) {
            if (batch_index) batch_index[total] = plan[i].c0 + b;
            ++total;
        }
    }
    *rows = total;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_mha_forward_sharded(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                          const float *d_wq_local, const float *d_wk_local, const float *d_wv_local,
                                          const float *d_wo, const float *d_ln_scale, const float *d_ln_shift,
                                          const int32_t *d_key_lengths, int32_t causal, float *d_out, int32_t precision,
                                          int32_t chunks)
{
    DL4S_STATE(st);
    CommState &c = g_comm[st->ordinal];
    const int world = c.live ? c.world : 1, rank = c.live ? c.rank : 0;
    DL4S_REQUIRE(d_x && d_wq_local && d_wk_local && d_wv_local && d_wo && d_ln_scale && d_ln_shift && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && S >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(H % world == 0, "%lld heads do not split evenly over %d ranks", (long long)H, world);
    DL4S_REQUIRE(!st->capturing, "the sharded layer orders two streams with events and cannot be recorded into a graph");
    const int64_t Hl = H / world, C = Hl * dv;
    ChunkPlan plan[kMaxChunks];
    const int nchunks = make_plan(B, world, rank, world > 1 ? chunks : 1, plan);

    // Head outputs travel as half where the tensor-core kernels produce and consume them.
    int half = precision != DL4S_PREC_FP32;
    int64_t bc_max = 0;
    for (int i = 0; i < nchunks && half; ++i) {
        const int64_t sizes[2] = {plan[i].c1 - plan[i].c0, plan[i].lb1 - plan[i].lb0};
        for (int k = 0; k < 2 && half; ++k) {
            if (sizes[k] == 0) continue;
            int32_t ok = 0;
            DL4S_TRY(dl4s_cuda_mha_heads_half_supported(sizes[k], S, D, Hl, dk, dv, H * dv, &ok));
            if (!ok) half = 0;
        }
    }
    for (int i = 0; i < nchunks; ++i)
        if (plan[i].c1 - plan[i].c0 > bc_max) bc_max = plan[i].c1 - plan[i].c0;
    const size_t esz = half ? 2 : 4;
    const size_t chunk_bytes = align_up((size_t)(world * bc_max * S * C) * esz, 256);
    if ((size_t)nchunks * chunk_bytes > c.gather_bytes) {
        DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
        if (c.stream) DL4S_CUDA_TRY(cudaStreamSynchronize(c.stream));
        if (c.gather) DL4S_CUDA_TRY(cudaFree(c.gather));
        c.gather = nullptr;
        c.gather_bytes = 0;
        DL4S_CUDA_TRY(cudaMalloc(&c.gather, (size_t)nchunks * chunk_bytes));
        c.gather_bytes = (size_t)nchunks * chunk_bytes;
    }
    ScopedGroup group(st, "MultiHeadAttention");
    // Tensor-core paths: the replicated input is rounded to half ONCE per call, in one pass at full HBM speed before
    // any gather is in flight, instead of chunk by chunk under the gathers' traffic (every rank needs all of it
    // for its projections, so this pass does not shrink with the number of ranks).
    const void *xh = nullptr;
    if (half && nchunks > 1) {
        const size_t need = (size_t)(B * S * D) * 2;
        if (need > c.xh_bytes) {
            DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
            if (c.xh) DL4S_CUDA_TRY(cudaFree(c.xh));
            c.xh = nullptr;
            c.xh_bytes = 0;
            DL4S_CUDA_TRY(cudaMalloc(&c.xh, need));
            c.xh_bytes = need;
        }
        DL4S_TRY(launch_f32_to_f16(st, d_x, c.xh, B * S * D));
        xh = c.xh;
    }

    auto gathered = [&](int i) { return static_cast<char *>(c.gather) + (size_t)i * chunk_bytes; };
    auto heads = [&](int i) -> dl4s_status {
        const int64_t c0 = plan[i].c0, Bc = plan[i].c1 - plan[i].c0;
        const float *xp = d_x + c0 * S * D;
        void *slot = gathered(i) + (size_t)(rank * Bc * S * C) * esz;
        return mha_heads_forward_impl(xp, xp, xp, Bc, S, S, D, Hl, dk, dv, d_wq_local, d_wk_local, d_wv_local,
                                      d_key_lengths ? d_key_lengths + c0 : nullptr, causal, slot, precision, half,
                                      xh ? static_cast<const char *>(xh) + (size_t)(c0 * S * D) * 2 : nullptr);
    };
    // ONE collective per chunk: in-place all-gather of the head outputs on the second stream.
    auto gather = [&](int i) -> dl4s_status {
        if (world == 1) return DL4S_OK;
        const int64_t Bc = plan[i].c1 - plan[i].c0;
        const size_t n = (size_t)(Bc * S * C) * esz;
        DL4S_CUDA_TRY(cudaEventRecord(c.ready[i], st->stream));
        DL4S_CUDA_TRY(cudaStreamWaitEvent(c.stream, c.ready[i], 0));
        DL4S_TRY(nccl_check(g_nccl.all_gather(gathered(i) + (size_t)rank * n, gathered(i), n, /*ncclInt8*/ 0, c.comm, c.stream),
                            "ncclAllGather"));
        DL4S_CUDA_TRY(cudaEventRecord(c.done[i], c.stream));
        return DL4S_OK;
    };
    auto output = [&](int i) -> dl4s_status {
        const int64_t c0 = plan[i].c0, Bc = plan[i].c1 - plan[i].c0, lb0 = plan[i].lb0, Bl = plan[i].lb1 - plan[i].lb0;
        // The compute stream waits for the gather even when this rank owns no row of the chunk: the next call
        // writes the same buffer.
        if (world > 1) {
            DL4S_CUDA_TRY(cudaEventRecord(c.wait0[i], st->stream));
            DL4S_CUDA_TRY(cudaStreamWaitEvent(st->stream, c.done[i], 0));
            DL4S_CUDA_TRY(cudaEventRecord(c.wait1[i], st->stream));
        }
        if (Bl == 0) return DL4S_OK;
        const void *hp = gathered(i) + (size_t)(lb0 * S * C) * esz;
        return dl4s_cuda_mha_output_forward(hp, d_x + (c0 + lb0) * S * D, Bl, S, D, world * C, d_wo, d_ln_scale, d_ln_shift,
                                            d_out + plan[i].out0 * S * D, precision, half, world, Bc * S * C);
    };
    c.last_chunks = world > 1 ? nchunks : 0;
    // While gathers are in flight their kernel holds some SMs: the products take their tiles from the device-wide
    // counter, so a CTA that starts late behind it simply takes fewer.
    struct DynamicTiles {
        DeviceState *st;
        int saved;
        DynamicTiles(DeviceState *s, int on) : st(s), saved(s->dynamic_tiles) { st->dynamic_tiles = on; }
        ~DynamicTiles() { st->dynamic_tiles = saved; }
    } dynamic_tiles(st, world > 1 && nchunks > 1);
    int pending = -1;
    for (int i = 0; i < nchunks; ++i) {
        DL4S_TRY(heads(i));
        DL4S_TRY(gather(i));
        if (pending >= 0) DL4S_TRY(output(pending));
        pending = i;
    }
    return output(pending);
}

}  // extern "C"
