// Backward of DL4S's LayerNorm (NN/Layer/LayerNorm.swift:62-77), the gradients its autograd obtains by chaining the
// backward closures of the primitives the layer is written with (reduceMean, variance = E[x^2] - mean^2, sqrt,
// the broadcast operators), in closed form. With n = rows * D elements per outer index,
//   m = mean(x), v = mean(x^2) - m^2, s = sqrt(v) + 1e-5, xh = (x - m) / s, y = xh * scale + shift
//   a = dy * scale
//   dx = ( a - mean(a) - xh * mean(a * xh) * (s / sqrt(v)) ) / s
//   dscale[c] = sum over (outer, rows) of dy * xh,   dshift[c] = sum of dy
// (the factor s / sqrt(v) is there because the reference adds epsilon to the standard deviation, not to the variance).
// fp32, HBM-bound: x and dy are read three times by the dx kernel (statistics, the two means, the result) and once
// by the parameter-gradient kernel. One CTA per outer index; sums are taken in double in a fixed order.
#include "common.cuh"

namespace dl4s {

constexpr int LNB_THREADS = 512;

__device__ __forceinline__ double lnb_block_sum(double v, double *sh)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < LNB_THREADS / 32; ++w) t += sh[w];   // every thread adds in the same order
    return t;
}

// stats[o] = {mean, 1 / s, s / sqrt(v)} are left for the parameter-gradient kernel.
__global__ void __launch_bounds__(LNB_THREADS) k_layernorm_bwd_dx(const float *__restrict__ x, const float *__restrict__ dy,
                                                                  const float *__restrict__ scale, int64_t cnt, int64_t D,
                                                                  float *__restrict__ dx, float *__restrict__ stats)
{
    __shared__ double sh[LNB_THREADS / 32];
    const int64_t o = blockIdx.x;
    const float *xo = x + o * cnt, *go = dy + o * cnt;
    double s1 = 0.0, s2 = 0.0;
    for (int64_t i = threadIdx.x; i < cnt; i += LNB_THREADS) {
        const double v = xo[i];
        s1 += v;
        s2 += v * v;
    }
    s1 = lnb_block_sum(s1, sh);
    s2 = lnb_block_sum(s2, sh);
    const float mean = (float)(s1 / (double)cnt);
    const float var = (float)(s2 / (double)cnt) - mean * mean;
    const float sd = sqrtf(var);
    const float s = sd + 1e-5f;
    const float inv_s = 1.0f / s;
    double a1 = 0.0, a2 = 0.0;
    for (int64_t i = threadIdx.x; i < cnt; i += LNB_THREADS) {
        const float a = go[i] * scale[i % D];
        const float xh = (xo[i] - mean) * inv_s;
        a1 += a;
        a2 += (double)a * xh;
    }
    a1 = lnb_block_sum(a1, sh);
    a2 = lnb_block_sum(a2, sh);
    const float mean_a = (float)(a1 / (double)cnt);
    const float corr = (float)(a2 / (double)cnt) * (s / sd);
    for (int64_t i = threadIdx.x; i < cnt; i += LNB_THREADS) {
        const float a = go[i] * scale[i % D];
        const float xh = (xo[i] - mean) * inv_s;
        dx[o * cnt + i] = (a - mean_a - xh * corr) * inv_s;
    }
    if (threadIdx.x == 0) {
        stats[2 * o] = mean;
        stats[2 * o + 1] = inv_s;
    }
}

// dscale[c] = sum_r dy[r, c] * xh[r, c], dshift[c] = sum_r dy[r, c] over all R = outer * rows rows; one CTA per 32
// columns, the rows split over the CTA's warps, added in a fixed order.
__global__ void __launch_bounds__(LNB_THREADS) k_layernorm_bwd_params(const float *__restrict__ x, const float *__restrict__ dy,
                                                                      const float *__restrict__ stats, int64_t R, int64_t rows_per_outer,
                                                                      int64_t D, float *__restrict__ dscale, float *__restrict__ dshift)
{
    __shared__ double sh1[LNB_THREADS / 32][32], sh2[LNB_THREADS / 32][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + lane;
    double g1 = 0.0, g2 = 0.0;
    if (c < D) {
        for (int64_t r = warp; r < R; r += LNB_THREADS / 32) {
            const int64_t o = r / rows_per_outer;
            const float mean = stats[2 * o], inv_s = stats[2 * o + 1];
            const float g = dy[r * D + c];
            g1 += (double)g * ((x[r * D + c] - mean) * inv_s);
            g2 += g;
        }
    }
    sh1[warp][lane] = g1;
    sh2[warp][lane] = g2;
    __syncthreads();
    if (warp == 0 && c < D) {
        double t1 = 0.0, t2 = 0.0;
        for (int w = 0; w < LNB_THREADS / 32; ++w) { t1 += sh1[w][lane]; t2 += sh2[w][lane]; }
        dscale[c] = (float)t1;
        dshift[c] = (float)t2;
    }
}

}  // namespace dl4s

using namespace dl4s;

extern "C" dl4s_status dl4s_cuda_layernorm_backward(const float *d_x, const float *d_dy, int64_t outer, int64_t rows, int64_t D,
                                                    const float *d_scale, float *d_dx, float *d_dscale, float *d_dshift)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_dy && d_scale && d_dx, "NULL buffer");
    DL4S_REQUIRE(outer >= 0 && rows >= 1 && D >= 1, "bad extents");
    DL4S_REQUIRE((d_dscale == nullptr) == (d_dshift == nullptr), "dscale and dshift come together");
    if (outer == 0) return DL4S_OK;
    DL4S_REQUIRE(outer < (1ll << 31), "too many blocks");
    void *stats = nullptr;
    DL4S_TRY(arena_reserve(st, (size_t)outer * 2 * sizeof(float), &stats));
    ScopedTimer timer(st);
    ScopedGroup group(st, "LayerNorm");
    k_layernorm_bwd_dx<<<(unsigned)outer, LNB_THREADS, 0, st->stream>>>(d_x, d_dy, d_scale, rows * D, D, d_dx, (float *)stats);
    DL4S_TRY(after_launch(st, "k_layernorm_bwd_dx"));
    if (d_dscale) {
        k_layernorm_bwd_params<<<(unsigned)ceil_div(D, 32), LNB_THREADS, 0, st->stream>>>(d_x, d_dy, (const float *)stats, outer * rows, rows, D,
                                                                                           d_dscale, d_dshift);
        DL4S_TRY(after_launch(st, "k_layernorm_bwd_params"));
    }
    return DL4S_OK;
}
