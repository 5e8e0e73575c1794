// Output head of the Transformer (NN/Models/Transformer/Transformer.swift:105-108):
//   logSoftmax(decoded . E^T + outputBias) over the vocabulary,
// with E the (tied) embedding matrix [V, D]. The product is a GEMM with the second operand
// transposed; the log-softmax (Tensor/Operators/Unary.swift:198-204) runs in place on the logits.
#include "common.cuh"
#include "tc.cuh"

namespace dl4s {

__device__ __forceinline__ float block_reduce_max(float v, float *sh)
{
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    v = lane < nw ? sh[lane] : -INFINITY;
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float block_reduce_sum(float v, float *sh)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    v = lane < nw ? sh[lane] : 0.f;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// y = (x - max) - log(sum(exp(x - max))) per row (Unary.swift:198-204). One CTA per row. The row (128 KB at a
// vocabulary of 32000) is read twice: once for the maximum and the sum together (each thread keeps a running
// maximum and rescales its partial sum when the maximum grows; the partials are combined with the row maximum),
// once to write the result; the grid is sized so that the rows in flight fit the L2 and the second read hits it.
// x and y may be the same buffer.
__global__ void __launch_bounds__(512) k_log_softmax_rows(const float *x, int64_t rows, int64_t n, float *y)
{
    __shared__ float sh[32];
    const bool vec = (n % 4 == 0) && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float *xr = x + r * n;
        float *yr = y + r * n;
        float m = -INFINITY, s = 0.f;
        auto take = [&](float v) {
            if (v > m) {
                s = s * expf(m - v);   // exp(-inf) = 0 on the first element
                m = v;
            }
            s += expf(v - m);
        };
        if (vec) {
            const float4 *x4 = reinterpret_cast<const float4 *>(xr);
            for (int64_t i = threadIdx.x; i < n / 4; i += blockDim.x) {
                const float4 v = x4[i];
                const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
                if (vm > m) {
                    s = s * expf(m - vm);
                    m = vm;
                }
                s += (expf(v.x - m) + expf(v.y - m)) + (expf(v.z - m) + expf(v.w - m));
            }
        } else {
            for (int64_t i = threadIdx.x; i < n; i += blockDim.x) take(xr[i]);
        }
        const float row_max = block_reduce_max(m, sh);
        const float part = (m == -INFINITY) ? 0.f : s * expf(m - row_max);
        const float total = block_reduce_sum(part, sh);
        const float negm = -row_max, neglse = -logf(total);
        if (vec) {
            const float4 *x4 = reinterpret_cast<const float4 *>(xr);
            float4 *y4 = reinterpret_cast<float4 *>(yr);
            for (int64_t i = threadIdx.x; i < n / 4; i += blockDim.x) {
                const float4 v = x4[i];
                y4[i] = make_float4((v.x + negm) + neglse, (v.y + negm) + neglse, (v.z + negm) + neglse, (v.w + negm) + neglse);
            }
        } else {
            for (int64_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = (xr[i] + negm) + neglse;
        }
    }
}

dl4s_status launch_log_softmax_rows(DeviceState *st, const float *x, int64_t rows, int64_t n, float *y)
{
    if (rows == 0 || n == 0) return DL4S_OK;
    // rows in flight: at most ~64 MB (half the L2), and no more than four CTAs per SM
    int64_t per_sm = 4;
    while (per_sm > 1 && (int64_t)st->sm_count * per_sm * n * (int64_t)sizeof(float) > (64ll << 20)) --per_sm;
    int64_t blocks = rows < (int64_t)st->sm_count * per_sm ? rows : (int64_t)st->sm_count * per_sm;
    k_log_softmax_rows<<<(unsigned)blocks, 512, 0, st->stream>>>(x, rows, n, y);
    return after_launch(st, "k_log_softmax_rows");
}

// E [V, D] fp32 -> E^T [D, V] half: the [K, N] operand layout of the tensor-core GEMM.
// lo != nullptr: the half-rounded remainders go there (the two-half form of a weight matrix).
__global__ void __launch_bounds__(256) k_transpose_to_f16(const float *__restrict__ e, int64_t V, int64_t D, __half *__restrict__ et,
                                                          __half *__restrict__ lo)
{
    __shared__ float tile[32][33];
    const int64_t v0 = (int64_t)blockIdx.x * 32, d0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    for (int j = ty; j < 32; j += 8) {
        const int64_t v = v0 + j, d = d0 + tx;
        tile[j][tx] = (v < V && d < D) ? e[v * D + d] : 0.f;
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int64_t d = d0 + j, v = v0 + tx;
        if (d < D && v < V) {
            const float w = tile[tx][j];
            const __half h = __float2half_rn(w);
            et[d * V + v] = h;
            if (lo) lo[d * V + v] = __float2half_rn(w - __half2float(h));
        }
    }
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_log_softmax_rows(const float *d_x, int64_t rows, int64_t n, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(rows >= 0 && n >= 0 && (rows * n == 0 || (d_x && d_out)), "bad arguments");
    return launch_log_softmax_rows(st, d_x, rows, n, d_out);
}

dl4s_status dl4s_cuda_output_head(const float *d_x, int64_t M, int64_t D, const float *d_embedding, int64_t V,
                                  const float *d_bias, float *d_out, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_embedding && d_out, "NULL buffer");
    DL4S_REQUIRE(M >= 1 && D >= 1 && V >= 1, "bad extents");
    DL4S_REQUIRE(precision == DL4S_PREC_FP32 || precision == DL4S_PREC_F16 || precision == DL4S_PREC_F16_SPLIT,
                 "unknown precision %d", precision);
    ScopedTimer timer(st);
    const int epi = d_bias ? EPI_BIAS : EPI_NONE;
    const int split = precision == DL4S_PREC_F16_SPLIT ? 1 : 0;   // the embedding is the weight operand
    if (precision != DL4S_PREC_FP32 && gemm_tc_supported(M, V, D) && V <= 65535 * 32 &&
        (((uintptr_t)d_x | (uintptr_t)d_out) & 15) == 0) {
        // x and E^T as half operands, fp32 logits
        const size_t xb = align_up((size_t)(M * D) * 2, 1024), eb = align_up((size_t)(D * V) * (split ? 4 : 2), 1024);
        void *base = nullptr;
        DL4S_TRY(arena_reserve(st, xb + eb, &base));
        void *xh = base, *eth = (char *)base + xb;
        DL4S_TRY(launch_f32_to_f16(st, d_x, xh, M * D));
        dim3 grid((unsigned)ceil_div(V, 32), (unsigned)ceil_div(D, 32));
        k_transpose_to_f16<<<grid, 256, 0, st->stream>>>(d_embedding, V, D, (__half *)eth, split ? (__half *)eth + D * V : nullptr);
        DL4S_TRY(after_launch(st, "k_transpose_to_f16"));
        GemmTcOut o;
        o.mode = OUT_F32;
        o.c = d_out;
        DL4S_TRY(launch_gemm_tc_h(st, xh, eth, M, V, D, epi, d_bias, nullptr, o, 1, 0, split));
    } else {
        DL4S_TRY(launch_gemm_f32(st, d_x, d_embedding, d_out, M, V, D, 1.0f, 0.0f, 0, 1, epi, d_bias, nullptr));
    }
    return launch_log_softmax_rows(st, d_out, M, V, d_out);
}

}  // extern "C"
