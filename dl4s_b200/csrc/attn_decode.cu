// Decode attention: ScaledDotProductAttention
// (NN/Models/Transformer/ScaledDotProductAttention.swift:43-64) called with one
// query per sequence against a long context, fp32 throughout.
//
// HBM-bound: every K and V row is read exactly once, so the kernel is a stream
// of 128-bit coalesced loads. The context of each (batch, head) pair is cut
// into fixed chunks (split-K over the context); one thread block reduces one
// chunk to a record (running max m, sum l, unnormalised output o[D]) in a
// scratch buffer, and a second kernel merges the records of a pair with the
// usual log-sum-exp rescaling. Rows at or beyond a sequence's length are never
// read; chunks that start beyond it exit at once. Algorithmic bytes per
// (batch, head): 2 * 4 * D * length (K and V rows) + 2 * 4 * D (q in, out).
#include "common.cuh"

namespace dl4s {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_UNROLL = 8;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS) k_attn_decode_partial(const float *__restrict__ q, const float *__restrict__ k,
                                                                     const float *__restrict__ v, int64_t H, int64_t Lmax,
                                                                     float inv_t, const int32_t *__restrict__ lens,
                                                                     float *__restrict__ scratch, int chunk, int nsplit)
{
    constexpr int LPR = D / 4;        // lanes per row (one float4 each)
    constexpr int RPW = 32 / LPR;     // rows a warp loads per instruction
    extern __shared__ float smem[];
    float *sc = smem;                 // [chunk] scores, then probabilities
    float *red = smem + chunk;        // [DEC_WARPS * D] cross-warp reduction
    __shared__ float s_stat[DEC_WARPS];

    const int split = blockIdx.x;
    const int64_t h = blockIdx.y, b = blockIdx.z, bh = b * H + h;
    int64_t len = lens ? lens[b] : Lmax;
    if (len > Lmax) len = Lmax;       // a length beyond the buffers reads what exists, as the other attention kernels do
    const bool uniform = (len <= 0);  // every key blocked: the reference's finite -1e9 gives equal weights
    if (uniform) len = Lmax;
    const int64_t begin = (int64_t)split * chunk;
    float *rec = scratch + (bh * nsplit + split) * (D + 2);
    if (begin >= len) {
        if (threadIdx.x == 0) { rec[0] = -INFINITY; rec[1] = 0.f; }
        return;
    }
    const int n = (int)((len - begin) < chunk ? (len - begin) : chunk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, li = lane % LPR;

    // q * 1/temperature, as the reference scales q before the product.
    float4 qv = reinterpret_cast<const float4 *>(q + bh * D)[li];
    qv.x *= inv_t; qv.y *= inv_t; qv.z *= inv_t; qv.w *= inv_t;

    const float4 *kb = reinterpret_cast<const float4 *>(k + (bh * Lmax + begin) * D);
    // Phase 1: scores. Each warp instruction covers RPW rows; DEC_UNROLL of them are in flight.
    float mx = -INFINITY;
    for (int r0 = warp * RPW * DEC_UNROLL; r0 < n; r0 += DEC_WARPS * RPW * DEC_UNROLL) {
        float4 kv[DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            int r = r0 + u * RPW + sub;
            kv[u] = (r < n) ? __ldcs(kb + (int64_t)r * LPR + li) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float s = qv.x * kv[u].x;
            s = fmaf(qv.y, kv[u].y, s);
            s = fmaf(qv.z, kv[u].z, s);
            s = fmaf(qv.w, kv[u].w, s);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            int r = r0 + u * RPW + sub;
            if (r < n) {
                if (uniform) s = s - 1e9f;
                if (li == 0) sc[r] = s;
                mx = fmaxf(mx, s);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_stat[warp] = mx;
    __syncthreads();
    mx = s_stat[0];
#pragma unroll
    for (int w = 1; w < DEC_WARPS; ++w) mx = fmaxf(mx, s_stat[w]);
    float sum = 0.f;
    for (int r = threadIdx.x; r < n; r += DEC_THREADS) {
        float e = expf(sc[r] - mx);
        sc[r] = e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();  // probabilities visible; s_stat free for reuse
    if (lane == 0) s_stat[warp] = sum;

    // Phase 2: o = sum_j p_j * v_j.
    const float4 *vb = reinterpret_cast<const float4 *>(v + (bh * Lmax + begin) * D);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = warp * RPW * DEC_UNROLL; r0 < n; r0 += DEC_WARPS * RPW * DEC_UNROLL) {
        float4 vv[DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            int r = r0 + u * RPW + sub;
            vv[u] = (r < n) ? __ldcs(vb + (int64_t)r * LPR + li) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            int r = r0 + u * RPW + sub;
            float pj = (r < n) ? sc[r] : 0.f;
            acc.x = fmaf(pj, vv[u].x, acc.x);
            acc.y = fmaf(pj, vv[u].y, acc.y);
            acc.z = fmaf(pj, vv[u].z, acc.z);
            acc.w = fmaf(pj, vv[u].w, acc.w);
        }
    }
    // Fold the RPW row groups of a warp, then the warps.
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (sub == 0) reinterpret_cast<float4 *>(red + warp * D)[li] = acc;
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += DEC_THREADS) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) t += red[w * D + c];
        rec[2 + c] = t;
    }
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) t += s_stat[w];
        rec[0] = mx;
        rec[1] = t;
    }
}

template <int D>
__global__ void __launch_bounds__(D) k_attn_decode_merge(const float *__restrict__ scratch, float *__restrict__ out, int nsplit)
{
    const int64_t bh = blockIdx.x;
    const float *rec = scratch + bh * nsplit * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, rec[s * (D + 2)]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        float m = rec[s * (D + 2)];
        if (m == -INFINITY) continue;
        float w = expf(m - M);
        l = fmaf(w, rec[s * (D + 2) + 1], l);
        o = fmaf(w, rec[s * (D + 2) + 2 + threadIdx.x], o);
    }
    out[bh * D + threadIdx.x] = o * (1.0f / l);
}

dl4s_status launch_attn_decode(DeviceState *st, const float *q, const float *k, const float *v, int64_t B, int64_t H,
                               int64_t Lmax, int64_t dk, int64_t dv, float inv_temperature, const int32_t *d_key_lengths,
                               float *out, float *scratch, int64_t chunk, int64_t nsplit)
{
    if (dk != dv || (dk != 64 && dk != 128)) return fail(DL4S_ERR_UNSUPPORTED, "decode kernel handles dk == dv in {64,128}");
    DL4S_REQUIRE(H <= 65535 && B <= 65535, "grid too large");
    dim3 grid((unsigned)nsplit, (unsigned)H, (unsigned)B);
    size_t smem = ((size_t)chunk + DEC_WARPS * dk) * sizeof(float);
    if (dk == 128) {
        k_attn_decode_partial<128><<<grid, DEC_THREADS, smem, st->stream>>>(q, k, v, H, Lmax, inv_temperature, d_key_lengths,
                                                                           scratch, (int)chunk, (int)nsplit);
        DL4S_TRY(after_launch(st, "k_attn_decode_partial"));
        k_attn_decode_merge<128><<<(unsigned)(B * H), 128, 0, st->stream>>>(scratch, out, (int)nsplit);
    } else {
        k_attn_decode_partial<64><<<grid, DEC_THREADS, smem, st->stream>>>(q, k, v, H, Lmax, inv_temperature, d_key_lengths,
                                                                          scratch, (int)chunk, (int)nsplit);
        DL4S_TRY(after_launch(st, "k_attn_decode_partial"));
        k_attn_decode_merge<64><<<(unsigned)(B * H), 64, 0, st->stream>>>(scratch, out, (int)nsplit);
    }
    return after_launch(st, "k_attn_decode_merge");
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// The split-K records normally live in the library's scratch arena, which grows
// with cudaMalloc on demand. Some hosts cannot afford that call where decode
// runs: a serving loop that has handed all of HBM to its own KV-cache manager
// (cudaMalloc would fail with out-of-memory), or a latency-critical step that
// must not take cudaMalloc's implicit device-wide synchronisation. For them the
// records go into this fixed array, which is part of the loaded module: every
// GPU that loads the library holds these 8 MiB until the process exits.
//
// In host code the array's name is only a stand-in for the symbol, not a device
// address; the address is obtained once per device with cudaGetSymbolAddress
// (with that device current) and passed to the kernels.
constexpr size_t kStaticDecodeFloats = (size_t)2 << 20;   // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_static_decode_scratch[kStaticDecodeFloats];
static float *g_static_decode_ptr[kMaxDevices] = {nullptr};

static dl4s_status static_decode_scratch(DeviceState *st, float **ptr)
{
    if (!g_static_decode_ptr[st->ordinal]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
        if (e != cudaSuccess) return check_cuda(e, "cudaGetSymbolAddress(g_static_decode_scratch)");
        g_static_decode_ptr[st->ordinal] = static_cast<float *>(p);
    }
    *ptr = g_static_decode_ptr[st->ordinal];
    return DL4S_OK;
}

// Called by dl4s_cuda_init with the device current: looks the array's address up and makes the driver load the
// decode kernels now. With lazy module loading the array and the kernels would otherwise be brought onto the
// device by the first decode call, which is exactly when a host that has since claimed all of HBM cannot spare
// the 8 MiB.
dl4s_status decode_static_prepare(DeviceState *st)
{
    float *p = nullptr;
    DL4S_TRY(static_decode_scratch(st, &p));
    cudaFuncAttributes attr;
    DL4S_CUDA_TRY(cudaFuncGetAttributes(&attr, k_attn_decode_partial<128>));
    DL4S_CUDA_TRY(cudaFuncGetAttributes(&attr, k_attn_decode_partial<64>));
    DL4S_CUDA_TRY(cudaFuncGetAttributes(&attr, k_attn_decode_merge<128>));
    DL4S_CUDA_TRY(cudaFuncGetAttributes(&attr, k_attn_decode_merge<64>));
    return DL4S_OK;
}

}  // namespace dl4s

using namespace dl4s;

extern "C" dl4s_status dl4s_cuda_sdpa_decode_noalloc(const float *d_q, const float *d_k, const float *d_v, int64_t B, int64_t H,
                                                     int64_t Lmax, int64_t d, float temperature,
                                                     const int32_t *d_key_lengths, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_q && d_k && d_v && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 0 && H >= 0 && Lmax >= 1, "bad extents");
    if (B * H == 0) return DL4S_OK;   // nothing to do, as in dl4s_cuda_sdpa_decode
    DL4S_REQUIRE(d == 64 || d == 128, "the no-allocation decode handles head size 64 or 128 (got %lld)", (long long)d);
    DL4S_REQUIRE(temperature != 0.0f, "temperature must not be zero");
    DL4S_REQUIRE(B <= 65535 && H <= 65535, "B and H must each be at most 65535");
    DL4S_REQUIRE((((uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v) & 15) == 0, "q, k and v must be 16-byte aligned");
    // The context is cut into the smallest power-of-two chunk (256..8192 keys) whose
    // partial records fit the fixed array: B*H*ceil(Lmax/chunk)*(d+2) floats.
    int64_t chunk = 256, nsplit = ceil_div(Lmax, chunk);
    while ((size_t)(B * H * nsplit * (d + 2)) > kStaticDecodeFloats && chunk < 8192) {
        chunk *= 2;
        nsplit = ceil_div(Lmax, chunk);
    }
    if ((size_t)(B * H * nsplit * (d + 2)) > kStaticDecodeFloats)
        return fail(DL4S_ERR_UNSUPPORTED,
                    "problem too large for the fixed scratch: B*H*ceil(Lmax/8192)*(d+2) = %lld floats exceeds %zu; "
                    "use dl4s_cuda_sdpa_decode",
                    (long long)(B * H * nsplit * (d + 2)), kStaticDecodeFloats);
    float *scratch = nullptr;
    DL4S_TRY(static_decode_scratch(st, &scratch));
    ScopedTimer timer(st);
    return launch_attn_decode(st, d_q, d_k, d_v, B, H, Lmax, d, d, 1.0f / temperature, d_key_lengths, d_out, scratch, chunk,
                              nsplit);
}
