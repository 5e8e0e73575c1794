// fp32 FFMA GEMM (check kernel and fp32 precision path of every projection).
// C = alpha * op(A) op(B) + beta * C, row-major, DL4S conventions
// (Engine/CPU/Numeric/CPUFloat.swift:263-292): A is stored [M,K] or, when
// trans_a, [K,M]; B is stored [K,N] or, when trans_b, [N,K].
// 128x128x16 block tile, 256 threads, 8x8 register tile per thread, smem
// double-buffered through registers. Epilogues fuse the bias / activation /
// residual glue of Dense (NN/Layer/Dense.swift:64-68) and of the residual
// additions in MultiHeadAttention.swift:123 and PointwiseFeedForward.swift:79.
#include "common.cuh"

namespace dl4s {

constexpr int BM = 128, BN = 128, BK = 16, GT = 256;

__device__ __forceinline__ float gelu_sigmoid(float t)
{
    // Tensor/Operators/Unary.swift:245-247 and 184-186, in the reference's order.
    float y = t * 1.702f;
    float z = y * 0.5f;
    float s = 0.5f * tanhf(z);
    s = s + 0.5f;
    return t * s;
}

template <bool TA, bool TB>
__global__ void __launch_bounds__(GT) k_gemm_f32(const float *__restrict__ A, const float *__restrict__ B,
                                                 float *__restrict__ C, int64_t M, int64_t N, int64_t K, float alpha,
                                                 float beta, int epilogue, const float *__restrict__ bias,
                                                 const float *__restrict__ residual, DropoutSpec drop)
{
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    const int tid = threadIdx.x;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 8x8 outputs each

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float ra[8], rb[8];

    auto load_tiles = [&](int64_t k0) {
        // A tile: BM x BK
        if (!TA) {
            int m = tid / 2, ks = (tid % 2) * 8;
            int64_t gm = m0 + m;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int64_t gk = k0 + ks + i;
                ra[i] = (gm < M && gk < K) ? A[gm * K + gk] : 0.f;
            }
        } else {
            int k = tid / 16, ms = (tid % 16) * 8;
            int64_t gk = k0 + k;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int64_t gm = m0 + ms + i;
                ra[i] = (gm < M && gk < K) ? A[gk * M + gm] : 0.f;
            }
        }
        if (!TB) {
            int k = tid / 16, ns = (tid % 16) * 8;
            int64_t gk = k0 + k;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int64_t gn = n0 + ns + i;
                rb[i] = (gn < N && gk < K) ? B[gk * N + gn] : 0.f;
            }
        } else {
            int n = tid / 2, ks = (tid % 2) * 8;
            int64_t gn = n0 + n;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int64_t gk = k0 + ks + i;
                rb[i] = (gn < N && gk < K) ? B[gn * K + gk] : 0.f;
            }
        }
    };
    auto store_tiles = [&](int buf) {
        if (!TA) {
            int m = tid / 2, ks = (tid % 2) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) As[buf][ks + i][m] = ra[i];
        } else {
            int k = tid / 16, ms = (tid % 16) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) As[buf][k][ms + i] = ra[i];
        }
        if (!TB) {
            int k = tid / 16, ns = (tid % 16) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) Bs[buf][k][ns + i] = rb[i];
        } else {
            int n = tid / 2, ks = (tid % 2) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) Bs[buf][ks + i][n] = rb[i];
        }
    };

    int64_t nk = (K + BK - 1) / BK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    for (int64_t kt = 0; kt < nk; ++kt) {
        int buf = kt & 1;
        if (kt + 1 < nk) load_tiles((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[8], b[8];
            // Each thread owns rows ty*4..+4 and 64+ty*4..+4, cols tx*4..+4 and 64+tx*4..+4:
            // 128-bit shared loads without bank conflicts.
            float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][k][ty * 4]);
            float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][k][64 + ty * 4]);
            float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][k][tx * 4]);
            float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][k][64 + tx * 4]);
            a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            store_tiles(buf ^ 1);
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int64_t gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (gn >= N) continue;
            float v = alpha * acc[i][j];
            if (beta != 0.f) v += beta * C[gm * N + gn];
            switch (epilogue) {
                case EPI_BIAS: v = v + bias[gn]; break;
                case EPI_BIAS_GELU: v = gelu_sigmoid(v + bias[gn]); break;
                case EPI_BIAS_RELU: v = v + bias[gn]; v = v > 0.f ? v : 0.f; break;
                case EPI_BIAS_RESIDUAL:
                    v = v + bias[gn];
                    v = (dropout_keep(drop, (uint64_t)(gm * N + gn)) ? v : 0.f) + residual[gm * N + gn];
                    break;
                case EPI_RESIDUAL: v = (dropout_keep(drop, (uint64_t)(gm * N + gn)) ? v : 0.f) + residual[gm * N + gn]; break;
                default: break;
            }
            C[gm * N + gn] = v;
        }
    }
}

// The split-K buffer of the skinny kernel stays below 256 MB.
static bool splits_fit(int64_t M, int64_t N) { return M * N <= (int64_t)(1 << 20); }

// ---- a few rows times a large matrix (one token per sequence through a projection) ----
// With M <= 64 the product is bound by reading B once. One thread per column keeps all M
// accumulators in registers, the rows of A pass through shared memory (transposed, so that four
// rows are one broadcast 128-bit load), and K is split over blockIdx.y so that enough CTAs stream
// B; the partial sums are added in a fixed order by a second kernel (no atomics: the result does
// not depend on scheduling), which also applies the epilogue.
constexpr int SK_THREADS = 256;   // columns per CTA
constexpr int SK_KC = 16;         // k rows staged per step

template <int MR>
__global__ void __launch_bounds__(SK_THREADS) k_gemm_skinny_f32(const float *__restrict__ A, const float *__restrict__ B,
                                                                float *__restrict__ P, int M, int64_t N, int64_t K,
                                                                int64_t k_chunk)
{
    __shared__ __align__(16) float xs[SK_KC][MR];
    const int64_t col = (int64_t)blockIdx.x * SK_THREADS + threadIdx.x;
    const int64_t k_begin = (int64_t)blockIdx.y * k_chunk;
    const int64_t k_end = k_begin + k_chunk < K ? k_begin + k_chunk : K;
    const bool live = col < N;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    // B's values for the next chunk are requested before the current chunk is multiplied.
    float w[SK_KC], wn[SK_KC];
#pragma unroll
    for (int kk = 0; kk < SK_KC; ++kk) w[kk] = (live && k_begin + kk < k_end) ? __ldg(B + (k_begin + kk) * N + col) : 0.f;
    for (int64_t k0 = k_begin; k0 < k_end; k0 += SK_KC) {
        __syncthreads();
        for (int i = threadIdx.x; i < SK_KC * MR; i += SK_THREADS) {
            const int kk = i % SK_KC, m = i / SK_KC;   // consecutive threads read consecutive k of one row
            const int64_t gk = k0 + kk;
            xs[kk][m] = (m < M && gk < k_end) ? A[(int64_t)m * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SK_KC; ++kk) {
            const int64_t gk = k0 + SK_KC + kk;
            wn[kk] = (live && gk < k_end) ? __ldg(B + gk * N + col) : 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < SK_KC; ++kk) {
#pragma unroll
            for (int m4 = 0; m4 < MR / 4; ++m4) {
                const float4 x = *reinterpret_cast<const float4 *>(&xs[kk][m4 * 4]);
                acc[m4 * 4 + 0] = fmaf(x.x, w[kk], acc[m4 * 4 + 0]);
                acc[m4 * 4 + 1] = fmaf(x.y, w[kk], acc[m4 * 4 + 1]);
                acc[m4 * 4 + 2] = fmaf(x.z, w[kk], acc[m4 * 4 + 2]);
                acc[m4 * 4 + 3] = fmaf(x.w, w[kk], acc[m4 * 4 + 3]);
            }
        }
#pragma unroll
        for (int kk = 0; kk < SK_KC; ++kk) w[kk] = wn[kk];
    }
    if (!live) return;
    float *dst = P + (int64_t)blockIdx.y * M * N + col;
#pragma unroll
    for (int m = 0; m < MR; ++m)
        if (m < M) dst[(int64_t)m * N] = acc[m];
}

// The same product for 17..64 rows, where the shared-memory loads of the kernel above (16 broadcast loads per 64
// multiply-adds) bound it: a 64 x 128 tile per CTA over one K split, 256 threads with 4 x 8 outputs each, A and B
// staged through shared memory (three 128-bit shared loads per 32 multiply-adds), 128-bit global loads, the
// next tile's global loads in flight during the current tile. (8 x 8 outputs per thread measured slower: 165
// registers leave too few warps per SM.)
constexpr int ST_BM = 64, ST_BN = 128, ST_BK = 16, ST_THREADS = 256;

__global__ void __launch_bounds__(ST_THREADS) k_gemm_skinny_tiled(const float *__restrict__ A, const float *__restrict__ B,
                                                                  float *__restrict__ P, int M, int64_t N, int64_t K,
                                                                  int64_t k_chunk)
{
    __shared__ __align__(16) float As[2][ST_BK][ST_BM + 4];
    __shared__ __align__(16) float Bs[2][ST_BK][ST_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads: rows ty*4..; columns tx*4.., 64 + tx*4..
    const int64_t n0 = (int64_t)blockIdx.x * ST_BN;
    const int64_t k_begin = (int64_t)blockIdx.y * k_chunk;
    const int64_t k_end = k_begin + k_chunk < K ? k_begin + k_chunk : K;
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float ra[4], rb[8];
    // A tile 64 x 16: thread -> row tid / 4, k (tid % 4) * 4 .. +4.  B tile 16 x 128: k tid / 16, columns (tid % 16) * 8 .. +8.
    // 128-bit global loads where the shapes allow them (K and N multiples of 4, 16-byte aligned bases, whole
    // vectors inside the range): a warp then reads whole 256-byte row segments of B.
    const bool vec_a = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && (k_chunk % 4 == 0);
    const bool vec_b = (N % 4 == 0) && ((uintptr_t)B % 16 == 0);
    auto load_tiles = [&](int64_t k0) {
        const int m = tid / 4, ks = (tid % 4) * 4;
        if (vec_a && m < M && k0 + ks + 3 < k_end) {
            const float4 t = *reinterpret_cast<const float4 *>(A + (int64_t)m * K + k0 + ks);
            ra[0] = t.x; ra[1] = t.y; ra[2] = t.z; ra[3] = t.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t gk = k0 + ks + i;
                ra[i] = (m < M && gk < k_end) ? A[(int64_t)m * K + gk] : 0.f;
            }
        }
        const int kb = tid / 16, ns = (tid % 16) * 8;
        const int64_t gk = k0 + kb;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (vec_b && gk < k_end && n0 + ns + 4 * h + 3 < N) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(B + gk * N + n0 + ns + 4 * h));
                rb[4 * h] = t.x; rb[4 * h + 1] = t.y; rb[4 * h + 2] = t.z; rb[4 * h + 3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t gn = n0 + ns + 4 * h + i;
                    rb[4 * h + i] = (gn < N && gk < k_end) ? __ldg(B + gk * N + gn) : 0.f;
                }
            }
        }
    };
    auto store_tiles = [&](int buf) {
        const int m = tid / 4, ks = (tid % 4) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) As[buf][ks + i][m] = ra[i];
        const int kb = tid / 16, ns = (tid % 16) * 8;
#pragma unroll
        for (int h = 0; h < 2; ++h)
            *reinterpret_cast<float4 *>(&Bs[buf][kb][ns + 4 * h]) = make_float4(rb[4 * h], rb[4 * h + 1], rb[4 * h + 2], rb[4 * h + 3]);
    };
    const int64_t nk = (k_end - k_begin + ST_BK - 1) / ST_BK;
    load_tiles(k_begin);
    store_tiles(0);
    __syncthreads();
    for (int64_t kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) load_tiles(k_begin + (kt + 1) * ST_BK);
#pragma unroll
        for (int k = 0; k < ST_BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][k][ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][k][64 + tx * 4]);
            const float a[4] = {a0.x, a0.y, a0.z, a0.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            store_tiles(buf ^ 1);
            __syncthreads();
        }
    }
    float *dst = P + (int64_t)blockIdx.y * M * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (gn < N) dst[(int64_t)m * N + gn] = acc[i][j];
        }
    }
}

__global__ void __launch_bounds__(256) k_gemm_skinny_reduce(const float *__restrict__ P, int splits, int64_t MN, int64_t N,
                                                            int epilogue, const float *__restrict__ bias,
                                                            const float *__restrict__ residual, float *__restrict__ C, DropoutSpec drop)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += (int64_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) v += P[(int64_t)s * MN + i];
        const int64_t gn = i % N;
        switch (epilogue) {
            case EPI_BIAS: v = v + bias[gn]; break;
            case EPI_BIAS_GELU: v = gelu_sigmoid(v + bias[gn]); break;
            case EPI_BIAS_RELU: v = v + bias[gn]; v = v > 0.f ? v : 0.f; break;
            case EPI_BIAS_RESIDUAL:
                v = v + bias[gn];
                v = (dropout_keep(drop, (uint64_t)i) ? v : 0.f) + residual[i];
                break;
            case EPI_RESIDUAL: v = (dropout_keep(drop, (uint64_t)i) ? v : 0.f) + residual[i]; break;
            default: break;
        }
        C[i] = v;
    }
}

static dl4s_status launch_gemm_skinny(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                                      int epilogue, const float *bias, const float *residual, DropoutSpec drop)
{
    // Two CTAs of this kernel fit an SM; K is split so that all CTAs are resident at once (a second, nearly
    // empty wave would double the time).
    const bool tiled = M > 16;
    const int64_t col_blocks = ceil_div(N, tiled ? ST_BN : SK_THREADS);
    int64_t splits = ((int64_t)st->sm_count * 2) / col_blocks;
    if (splits < 1) splits = 1;
    int64_t k_chunk = align_up((size_t)ceil_div(K, splits), SK_KC);
    if (k_chunk < 4 * SK_KC) k_chunk = 4 * SK_KC;
    splits = ceil_div(K, k_chunk);
    const size_t need = (size_t)(splits * M * N) * sizeof(float);
    if (need > st->skinny_bytes) {
        if (st->capturing)
            return fail(DL4S_ERR_UNSUPPORTED, "the split-K buffer would have to grow while a graph is being captured: run the "
                        "same calls once before dl4s_cuda_graph_begin");
        DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
        DL4S_TRY(release_internal(st, st->skinny_partials));
        st->skinny_partials = nullptr;
        st->skinny_bytes = 0;
        DL4S_CUDA_TRY(cudaMalloc((void **)&st->skinny_partials, need));
        st->skinny_bytes = need;
    }
    dim3 grid((unsigned)col_blocks, (unsigned)splits);
    float *P = st->skinny_partials;
    if (tiled) k_gemm_skinny_tiled<<<grid, ST_THREADS, 0, st->stream>>>(a, b, P, (int)M, N, K, k_chunk);
    else k_gemm_skinny_f32<16><<<grid, SK_THREADS, 0, st->stream>>>(a, b, P, (int)M, N, K, k_chunk);
    DL4S_TRY(after_launch(st, "k_gemm_skinny_f32"));
    int64_t blocks = ceil_div(M * N, 256);
    if (blocks > (int64_t)st->sm_count * 8) blocks = (int64_t)st->sm_count * 8;
    k_gemm_skinny_reduce<<<(unsigned)blocks, 256, 0, st->stream>>>(P, (int)splits, M * N, N, epilogue, bias, residual, c, drop);
    return after_launch(st, "k_gemm_skinny_reduce");
}

dl4s_status launch_gemm_f32(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                            float alpha, float beta, int trans_a, int trans_b, int epilogue, const float *bias,
                            const float *residual, const DropoutSpec *dropp)
{
    if (M == 0 || N == 0) return DL4S_OK;
    const DropoutSpec drop = dropp ? *dropp : DropoutSpec();
    if (!trans_a && !trans_b && M <= 64 && N >= 512 && K >= 512 && alpha == 1.0f && beta == 0.0f && splits_fit(M, N))
        return launch_gemm_skinny(st, a, b, c, M, N, K, epilogue, bias, residual, drop);
    dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(M, BM));
    DL4S_REQUIRE(ceil_div(M, BM) <= 65535, "M too large for the fp32 gemm grid");
    if (!trans_a && !trans_b) k_gemm_f32<false, false><<<grid, GT, 0, st->stream>>>(a, b, c, M, N, K, alpha, beta, epilogue, bias, residual, drop);
    else if (!trans_a && trans_b) k_gemm_f32<false, true><<<grid, GT, 0, st->stream>>>(a, b, c, M, N, K, alpha, beta, epilogue, bias, residual, drop);
    else if (trans_a && !trans_b) k_gemm_f32<true, false><<<grid, GT, 0, st->stream>>>(a, b, c, M, N, K, alpha, beta, epilogue, bias, residual, drop);
    else k_gemm_f32<true, true><<<grid, GT, 0, st->stream>>>(a, b, c, M, N, K, alpha, beta, epilogue, bias, residual, drop);
    return after_launch(st, "k_gemm_f32");
}

}  // namespace dl4s
