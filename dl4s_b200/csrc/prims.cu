// fp32 EngineType primitives: element-wise, broadcast, reduce, permute, stack,
// band, strided copies. All are HBM-bound grid-stride kernels with 128-bit
// accesses where alignment allows; grids are sized in multiples of the SM count.
#include "common.cuh"

namespace dl4s {

constexpr int kMaxDim = 8;
constexpr int kThreads = 256;

static inline int grid_for(DeviceState *st, int64_t work_items, int per_block)
{
    int64_t blocks = ceil_div(work_items, per_block);
    int64_t cap = (int64_t)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// ---------------------------------------------------------------- element-wise
enum UnaryOp { U_NEG, U_EXP, U_LOG, U_SQRT, U_RELU, U_HEAVISIDE, U_SIN, U_COS, U_TANH };
enum BinaryOp { B_ADD, B_SUB, B_MUL, B_DIV };

template <int OP>
__device__ __forceinline__ float unary(float x)
{
    if (OP == U_NEG) return -x;
    if (OP == U_EXP) return expf(x);
    if (OP == U_LOG) return logf(x);
    if (OP == U_SQRT) return sqrtf(x);
    if (OP == U_RELU) return x > 0.f ? x : 0.f;
    if (OP == U_HEAVISIDE) return x > 0.f ? 1.f : 0.f;
    if (OP == U_SIN) return sinf(x);
    if (OP == U_COS) return cosf(x);
    return tanhf(x);
}

template <int OP>
__device__ __forceinline__ float binary(float a, float b)
{
    if (OP == B_ADD) return a + b;
    if (OP == B_SUB) return a - b;
    if (OP == B_MUL) return a * b;
    return a / b;
}

template <int OP>
__global__ void __launch_bounds__(kThreads) k_unary(const float *__restrict__ x, float *__restrict__ y, int64_t n, int vec)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        float4 *y4 = reinterpret_cast<float4 *>(y);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 v = x4[i];
            v.x = unary<OP>(v.x); v.y = unary<OP>(v.y); v.z = unary<OP>(v.z); v.w = unary<OP>(v.w);
            y4[i] = v;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) y[i] = unary<OP>(x[i]);
    } else {
        for (int64_t i = tid; i < n; i += stride) y[i] = unary<OP>(x[i]);
    }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) k_binary(const float *__restrict__ a, const float *__restrict__ b,
                                                     float *__restrict__ y, int64_t n, int vec)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        const float4 *a4 = reinterpret_cast<const float4 *>(a);
        const float4 *b4 = reinterpret_cast<const float4 *>(b);
        float4 *y4 = reinterpret_cast<float4 *>(y);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 u = a4[i], v = b4[i], r;
            r.x = binary<OP>(u.x, v.x); r.y = binary<OP>(u.y, v.y);
            r.z = binary<OP>(u.z, v.z); r.w = binary<OP>(u.w, v.w);
            y4[i] = r;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) y[i] = binary<OP>(a[i], b[i]);
    } else {
        for (int64_t i = tid; i < n; i += stride) y[i] = binary<OP>(a[i], b[i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) k_fill(T *__restrict__ y, T value, int64_t n)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) y[i] = value;
}

static inline int aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

template <int OP>
static dl4s_status run_unary(const float *x, float *y, int64_t n)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(n >= 0 && (n == 0 || (x && y)), "bad arguments");
    if (n == 0) return DL4S_OK;
    int vec = aligned16(x) && aligned16(y);
    k_unary<OP><<<grid_for(st, n, kThreads * 4), kThreads, 0, st->stream>>>(x, y, n, vec);
    return after_launch(st, "k_unary");
}

template <int OP>
static dl4s_status run_binary(const float *a, const float *b, float *y, int64_t n)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(n >= 0 && (n == 0 || (a && b && y)), "bad arguments");
    if (n == 0) return DL4S_OK;
    int vec = aligned16(a) && aligned16(b) && aligned16(y);
    k_binary<OP><<<grid_for(st, n, kThreads * 4), kThreads, 0, st->stream>>>(a, b, y, n, vec);
    return after_launch(st, "k_binary");
}

// ------------------------------------------------------------------ broadcast
struct BroadcastArgs {
    int dim;
    int64_t shape[kMaxDim];
    int64_t ls[kMaxDim];  // lhs strides, 0 on broadcast axes
    int64_t rs[kMaxDim];
};

// rhs_is_scalar_div: the reference multiplies by the fp32 reciprocal when the
// divisor is broadcast along the innermost varying axis (vector / scalar).
template <int OP>
__global__ void __launch_bounds__(kThreads) k_broadcast(const float *__restrict__ a, const float *__restrict__ b,
                                                        float *__restrict__ y, int64_t n, BroadcastArgs args,
                                                        int recip_div)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t rem = i, lo = 0, ro = 0;
#pragma unroll
        for (int d = kMaxDim - 1; d >= 0; --d) {
            if (d < args.dim) {
                int64_t c = rem % args.shape[d];
                rem /= args.shape[d];
                lo += c * args.ls[d];
                ro += c * args.rs[d];
            }
        }
        float u = a[lo], v = b[ro];
        if (OP == B_DIV && recip_div) y[i] = u * (1.0f / v);
        else if (OP == B_SUB) y[i] = u + (-v);
        else y[i] = binary<OP>(u, v);
    }
}

template <int OP>
static dl4s_status run_broadcast(const float *a, const int64_t *lshape, int ldim, const float *b,
                                 const int64_t *rshape, int rdim, float *y)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(a && b && y, "NULL buffer");
    DL4S_REQUIRE(ldim >= 0 && rdim >= 0 && ldim <= kMaxDim && rdim <= kMaxDim, "at most %d dimensions", kMaxDim);
    BroadcastArgs args;
    args.dim = ldim > rdim ? ldim : rdim;
    int64_t lsh[kMaxDim], rsh[kMaxDim];
    for (int d = 0; d < args.dim; ++d) {
        int li = d - (args.dim - ldim), ri = d - (args.dim - rdim);
        lsh[d] = li >= 0 ? lshape[li] : 1;
        rsh[d] = ri >= 0 ? rshape[ri] : 1;
        DL4S_REQUIRE(lsh[d] == rsh[d] || lsh[d] == 1 || rsh[d] == 1, "shapes are not broadcast-compatible on axis %d", d);
        args.shape[d] = lsh[d] > rsh[d] ? lsh[d] : rsh[d];
    }
    int64_t n = 1, lstr = 1, rstr = 1;
    for (int d = args.dim - 1; d >= 0; --d) {
        args.ls[d] = lsh[d] == 1 ? 0 : lstr;
        args.rs[d] = rsh[d] == 1 ? 0 : rstr;
        lstr *= lsh[d];
        rstr *= rsh[d];
        n *= args.shape[d];
    }
    for (int d = args.dim; d < kMaxDim; ++d) { args.shape[d] = 1; args.ls[d] = args.rs[d] = 0; }
    if (n == 0) return DL4S_OK;
    // Vector / scalar mode of the reference: walking from the last axis, the first
    // axis where the extents differ has the larger extent on the left.
    int recip = 0;
    if (OP == B_DIV) {
        for (int d = args.dim - 1; d >= 0; --d) {
            if (lsh[d] > rsh[d]) { recip = 1; break; }
            if (rsh[d] > lsh[d]) break;
            if (lsh[d] > 1) break;  // equal, non-trivial suffix: vector / vector
        }
    }
    k_broadcast<OP><<<grid_for(st, n, kThreads * 2), kThreads, 0, st->stream>>>(a, b, y, n, args, recip);
    return after_launch(st, "k_broadcast");
}

// --------------------------------------------------------------------- reduce
struct ReduceArgs {
    int nkept, nred;
    int64_t kept_shape[kMaxDim], kept_stride[kMaxDim];
    int64_t red_shape[kMaxDim], red_stride[kMaxDim];
    int64_t red_count;
};

template <int THREADS, bool IS_MAX>
__global__ void __launch_bounds__(THREADS) k_reduce(const float *__restrict__ x, float *__restrict__ y,
                                                    int32_t *__restrict__ ctx, int64_t nout, ReduceArgs args)
{
    __shared__ double s_val[THREADS / 32];
    __shared__ int64_t s_idx[THREADS / 32];
    for (int64_t o = blockIdx.x; o < nout; o += gridDim.x) {
        int64_t rem = o, base = 0;
        for (int d = args.nkept - 1; d >= 0; --d) {
            int64_t c = rem % args.kept_shape[d];
            rem /= args.kept_shape[d];
            base += c * args.kept_stride[d];
        }
        double acc = IS_MAX ? -INFINITY : 0.0;
        int64_t best = 0;
        for (int64_t r = threadIdx.x; r < args.red_count; r += THREADS) {
            int64_t rr = r, off = base;
            for (int d = args.nred - 1; d >= 0; --d) {
                int64_t c = rr % args.red_shape[d];
                rr /= args.red_shape[d];
                off += c * args.red_stride[d];
            }
            float v = x[off];
            if (IS_MAX) { if ((double)v > acc) { acc = v; best = r; } }
            else acc += (double)v;
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            double ov = __shfl_xor_sync(0xffffffffu, acc, s);
            int64_t oi = __shfl_xor_sync(0xffffffffu, best, s);
            if (IS_MAX) { if (ov > acc || (ov == acc && oi < best)) { acc = ov; best = oi; } }
            else acc += ov;
        }
        int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) { s_val[warp] = acc; s_idx[warp] = best; }
        __syncthreads();
        if (threadIdx.x == 0) {
            double a = s_val[0];
            int64_t bi = s_idx[0];
            for (int w = 1; w < THREADS / 32; ++w) {
                if (IS_MAX) { if (s_val[w] > a || (s_val[w] == a && s_idx[w] < bi)) { a = s_val[w]; bi = s_idx[w]; } }
                else a += s_val[w];
            }
            y[o] = (float)a;
            if (IS_MAX && ctx) ctx[o] = (int32_t)bi;
        }
        __syncthreads();
    }
}

template <bool IS_MAX>
static dl4s_status run_reduce(const float *x, const int64_t *shape, int dim, const int32_t *axes, int naxes,
                              float *y, int32_t *ctx)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(x && y && shape, "NULL argument");
    DL4S_REQUIRE(dim >= 1 && dim <= kMaxDim && naxes >= 1 && naxes <= dim, "bad rank");
    DL4S_REQUIRE(!ctx || naxes == 1, "arg-max context needs exactly one reduced axis");
    bool red[kMaxDim] = {false};
    for (int i = 0; i < naxes; ++i) {
        DL4S_REQUIRE(axes[i] >= 0 && axes[i] < dim && !red[axes[i]], "bad axis %d", axes[i]);
        red[axes[i]] = true;
    }
    int64_t strides[kMaxDim], s = 1;
    for (int d = dim - 1; d >= 0; --d) { strides[d] = s; s *= shape[d]; }
    ReduceArgs args;
    args.nkept = args.nred = 0;
    args.red_count = 1;
    int64_t nout = 1;
    for (int d = 0; d < dim; ++d) {
        if (red[d]) { args.red_shape[args.nred] = shape[d]; args.red_stride[args.nred++] = strides[d]; args.red_count *= shape[d]; }
        else { args.kept_shape[args.nkept] = shape[d]; args.kept_stride[args.nkept++] = strides[d]; nout *= shape[d]; }
    }
    if (nout == 0) return DL4S_OK;
    DL4S_REQUIRE(args.red_count > 0, "cannot reduce an empty axis");
    int64_t cap = (int64_t)st->sm_count * 16;
    int grid = (int)(nout < cap ? nout : cap);
    if (args.red_count <= 2048) k_reduce<32, IS_MAX><<<grid, 32, 0, st->stream>>>(x, y, ctx, nout, args);
    else k_reduce<256, IS_MAX><<<grid, 256, 0, st->stream>>>(x, y, ctx, nout, args);
    return after_launch(st, "k_reduce");
}

// -------------------------------------------------- permute / strided copy / band
struct GatherArgs {
    int dim;
    int64_t shape[kMaxDim];       // extents of the iteration space (destination order)
    int64_t src_stride[kMaxDim];  // element stride in the source per iteration axis
    int64_t dst_stride[kMaxDim];
    int64_t src_offset, dst_offset;
};

// T is float, or float4 when the innermost axis is contiguous on both sides and
// everything is 16-byte aligned (extents, strides and offsets are then in float4 units).
template <typename T>
__global__ void __launch_bounds__(kThreads) k_gather(const T *__restrict__ x, T *__restrict__ y, int64_t n, GatherArgs args)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t rem = i, so = args.src_offset, dof = args.dst_offset;
#pragma unroll
        for (int d = kMaxDim - 1; d >= 0; --d) {
            if (d < args.dim) {
                int64_t c = rem % args.shape[d];
                rem /= args.shape[d];
                so += c * args.src_stride[d];
                dof += c * args.dst_stride[d];
            }
        }
        y[dof] = x[so];
    }
}

__global__ void __launch_bounds__(kThreads) k_band(const float *__restrict__ x, float *__restrict__ y, int64_t rows,
                                                   int64_t cols, int64_t below, int64_t above)
{
    int64_t n = rows * cols;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t r = i / cols, c = i % cols;
        bool keep = (c >= r - below) && (c <= r + above);
        y[i] = keep ? x[i] : 0.f;
    }
}

// y = x * bernoulli(1 - rate) with the counter-based mask of common.cuh (Dropout.swift:47-55).
__global__ void __launch_bounds__(kThreads) k_dropout(const float *__restrict__ x, float *__restrict__ y, int64_t n, DropoutSpec drop)
{
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) y[i] = dropout_keep(drop, (uint64_t)i) ? x[i] : 0.f;
}

// result[o, j] = stacked[o * row + j] + add[o, j] for the slab of `inner` columns that starts at `stacked`.
__global__ void __launch_bounds__(kThreads) k_unstack_add(const float *__restrict__ stacked, int64_t row, const float *__restrict__ add,
                                                          float *__restrict__ y, int64_t outer, int64_t inner)
{
    int64_t n = outer * inner;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t o = i / inner, j = i - o * inner;
        y[i] = stacked[o * row + j] + add[i];
    }
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_fill_f32(float value, float *d_result, int64_t count)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(count >= 0 && (count == 0 || d_result), "bad arguments");
    if (count == 0) return DL4S_OK;
    k_fill<float><<<grid_for(st, count, kThreads * 4), kThreads, 0, st->stream>>>(d_result, value, count);
    return after_launch(st, "k_fill");
}

dl4s_status dl4s_cuda_fill_i32(int32_t value, int32_t *d_result, int64_t count)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(count >= 0 && (count == 0 || d_result), "bad arguments");
    if (count == 0) return DL4S_OK;
    k_fill<int32_t><<<grid_for(st, count, kThreads * 4), kThreads, 0, st->stream>>>(d_result, value, count);
    return after_launch(st, "k_fill");
}

dl4s_status dl4s_cuda_vadd(const float *a, const float *b, float *y, int64_t n) { return run_binary<B_ADD>(a, b, y, n); }
dl4s_status dl4s_cuda_vsub(const float *a, const float *b, float *y, int64_t n) { return run_binary<B_SUB>(a, b, y, n); }
dl4s_status dl4s_cuda_vmul(const float *a, const float *b, float *y, int64_t n) { return run_binary<B_MUL>(a, b, y, n); }
dl4s_status dl4s_cuda_vdiv(const float *a, const float *b, float *y, int64_t n) { return run_binary<B_DIV>(a, b, y, n); }
dl4s_status dl4s_cuda_vneg(const float *x, float *y, int64_t n) { return run_unary<U_NEG>(x, y, n); }
dl4s_status dl4s_cuda_exp(const float *x, float *y, int64_t n) { return run_unary<U_EXP>(x, y, n); }
dl4s_status dl4s_cuda_log(const float *x, float *y, int64_t n) { return run_unary<U_LOG>(x, y, n); }
dl4s_status dl4s_cuda_sqrt(const float *x, float *y, int64_t n) { return run_unary<U_SQRT>(x, y, n); }
dl4s_status dl4s_cuda_relu(const float *x, float *y, int64_t n) { return run_unary<U_RELU>(x, y, n); }
dl4s_status dl4s_cuda_heaviside(const float *x, float *y, int64_t n) { return run_unary<U_HEAVISIDE>(x, y, n); }
dl4s_status dl4s_cuda_sin(const float *x, float *y, int64_t n) { return run_unary<U_SIN>(x, y, n); }
dl4s_status dl4s_cuda_cos(const float *x, float *y, int64_t n) { return run_unary<U_COS>(x, y, n); }
dl4s_status dl4s_cuda_tanh(const float *x, float *y, int64_t n) { return run_unary<U_TANH>(x, y, n); }

dl4s_status dl4s_cuda_broadcast_add(const float *a, const int64_t *ls, int32_t ld, const float *b, const int64_t *rs, int32_t rd, float *y)
{ return run_broadcast<B_ADD>(a, ls, ld, b, rs, rd, y); }
dl4s_status dl4s_cuda_broadcast_sub(const float *a, const int64_t *ls, int32_t ld, const float *b, const int64_t *rs, int32_t rd, float *y)
{ return run_broadcast<B_SUB>(a, ls, ld, b, rs, rd, y); }
dl4s_status dl4s_cuda_broadcast_mul(const float *a, const int64_t *ls, int32_t ld, const float *b, const int64_t *rs, int32_t rd, float *y)
{ return run_broadcast<B_MUL>(a, ls, ld, b, rs, rd, y); }
dl4s_status dl4s_cuda_broadcast_div(const float *a, const int64_t *ls, int32_t ld, const float *b, const int64_t *rs, int32_t rd, float *y)
{ return run_broadcast<B_DIV>(a, ls, ld, b, rs, rd, y); }

dl4s_status dl4s_cuda_reduce_sum(const float *x, const int64_t *shape, int32_t dim, const int32_t *axes, int32_t naxes, float *y)
{ return run_reduce<false>(x, shape, dim, axes, naxes, y, nullptr); }
dl4s_status dl4s_cuda_reduce_max(const float *x, const int64_t *shape, int32_t dim, const int32_t *axes, int32_t naxes, float *y, int32_t *ctx)
{ return run_reduce<true>(x, shape, dim, axes, naxes, y, ctx); }

dl4s_status dl4s_cuda_permute_axes(const float *x, const int64_t *shape, int32_t dim, const int32_t *arangement, float *y)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(x && y && shape && arangement, "NULL argument");
    DL4S_REQUIRE(dim >= 1 && dim <= kMaxDim, "bad rank");
    bool seen[kMaxDim] = {false};
    for (int i = 0; i < dim; ++i) {
        DL4S_REQUIRE(arangement[i] >= 0 && arangement[i] < dim && !seen[arangement[i]], "arangement is not a permutation");
        seen[arangement[i]] = true;
    }
    int64_t sstr[kMaxDim], s = 1, n = 1;
    for (int d = dim - 1; d >= 0; --d) { sstr[d] = s; s *= shape[d]; n *= shape[d]; }
    GatherArgs args;
    args.dim = dim;
    args.src_offset = args.dst_offset = 0;
    // Source axis i lands on destination axis arangement[i].
    for (int i = 0; i < dim; ++i) { args.shape[arangement[i]] = shape[i]; args.src_stride[arangement[i]] = sstr[i]; }
    s = 1;
    for (int d = dim - 1; d >= 0; --d) { args.dst_stride[d] = s; s *= args.shape[d]; }
    for (int d = dim; d < kMaxDim; ++d) { args.shape[d] = 1; args.src_stride[d] = args.dst_stride[d] = 0; }
    if (n == 0) return DL4S_OK;
    k_gather<float><<<grid_for(st, n, kThreads * 2), kThreads, 0, st->stream>>>(x, y, n, args);
    return after_launch(st, "k_gather");
}

dl4s_status dl4s_cuda_copy_strided_f32(const float *d_src, const int64_t *src_strides, int64_t src_offset, float *d_dst,
                                       const int64_t *dst_strides, int64_t dst_offset, const int64_t *extent, int32_t dim)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_src && d_dst && src_strides && dst_strides && extent, "NULL argument");
    DL4S_REQUIRE(dim >= 1 && dim <= kMaxDim, "bad rank");
    GatherArgs args;
    args.dim = dim;
    args.src_offset = src_offset;
    args.dst_offset = dst_offset;
    int64_t n = 1;
    for (int d = 0; d < dim; ++d) {
        DL4S_REQUIRE(extent[d] >= 0, "negative extent");
        args.shape[d] = extent[d]; args.src_stride[d] = src_strides[d]; args.dst_stride[d] = dst_strides[d];
        n *= extent[d];
    }
    for (int d = dim; d < kMaxDim; ++d) { args.shape[d] = 1; args.src_stride[d] = args.dst_stride[d] = 0; }
    if (n == 0) return DL4S_OK;
    // 128-bit path: contiguous innermost axis, all offsets and outer strides multiples of 4 floats.
    bool vec = src_strides[dim - 1] == 1 && dst_strides[dim - 1] == 1 && extent[dim - 1] % 4 == 0 && src_offset % 4 == 0 &&
               dst_offset % 4 == 0 && (((uintptr_t)d_src | (uintptr_t)d_dst) & 15) == 0;
    for (int d = 0; d + 1 < dim && vec; ++d) vec = src_strides[d] % 4 == 0 && dst_strides[d] % 4 == 0;
    if (vec) {
        for (int d = 0; d + 1 < dim; ++d) { args.src_stride[d] /= 4; args.dst_stride[d] /= 4; }
        args.shape[dim - 1] /= 4;
        args.src_offset /= 4;
        args.dst_offset /= 4;
        n /= 4;
        k_gather<float4><<<grid_for(st, n, kThreads * 2), kThreads, 0, st->stream>>>(reinterpret_cast<const float4 *>(d_src),
                                                                                   reinterpret_cast<float4 *>(d_dst), n, args);
    } else {
        k_gather<float><<<grid_for(st, n, kThreads * 2), kThreads, 0, st->stream>>>(d_src, d_dst, n, args);
    }
    return after_launch(st, "k_gather");
}

dl4s_status dl4s_cuda_stack(const float *const *d_buffers, const int64_t *shapes, int32_t n, int32_t dim, int32_t axis, float *d_result)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_buffers && shapes && d_result && n >= 1, "bad arguments");
    DL4S_REQUIRE(dim >= 1 && dim <= kMaxDim && axis >= 0 && axis < dim, "bad axis");
    int64_t outer = 1, total_inner = 0;
    for (int d = 0; d < axis; ++d) outer *= shapes[d];
    for (int i = 0; i < n; ++i) {
        const int64_t *sh = shapes + (int64_t)i * dim;
        int64_t inner = 1, o = 1;
        for (int d = 0; d < axis; ++d) o *= sh[d];
        DL4S_REQUIRE(o == outer, "leading extents of buffer %d differ", i);
        for (int d = axis; d < dim; ++d) inner *= sh[d];
        total_inner += inner;
    }
    int64_t off = 0;
    for (int i = 0; i < n; ++i) {
        const int64_t *sh = shapes + (int64_t)i * dim;
        int64_t inner = 1;
        for (int d = axis; d < dim; ++d) inner *= sh[d];
        if (inner == 0 || outer == 0) continue;
        DL4S_CUDA_TRY(cudaMemcpy2DAsync(d_result + off, (size_t)total_inner * sizeof(float), d_buffers[i],
                                        (size_t)inner * sizeof(float), (size_t)inner * sizeof(float), (size_t)outer,
                                        cudaMemcpyDeviceToDevice, st->stream));
        off += inner;
    }
    return DL4S_OK;
}

// unstack / unstackAdd (Engine.swift:543,551; CPUEngine.swift:1025-1085): the inverse of stack. Buffer i receives
// the slab [outer, inner_i] that starts `off` elements into every [total_inner] row of the stacked tensor.
static dl4s_status unstack_impl(const float *d_stacked, const float *const *d_add, float *const *d_results, const int64_t *shapes,
                                int32_t n, int32_t dim, int32_t axis)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_stacked && d_results && shapes && n >= 1, "bad arguments");
    DL4S_REQUIRE(dim >= 1 && dim <= kMaxDim && axis >= 0 && axis < dim, "bad axis");
    int64_t outer = 1, total_inner = 0;
    for (int d = 0; d < axis; ++d) outer *= shapes[d];
    for (int i = 0; i < n; ++i) {
        const int64_t *sh = shapes + (int64_t)i * dim;
        int64_t inner = 1, o = 1;
        for (int d = 0; d < axis; ++d) o *= sh[d];
        DL4S_REQUIRE(o == outer, "leading extents of buffer %d differ", i);
        for (int d = axis; d < dim; ++d) inner *= sh[d];
        total_inner += inner;
    }
    int64_t off = 0;
    for (int i = 0; i < n; ++i) {
        const int64_t *sh = shapes + (int64_t)i * dim;
        int64_t inner = 1;
        for (int d = axis; d < dim; ++d) inner *= sh[d];
        if (inner == 0 || outer == 0) continue;
        DL4S_REQUIRE(d_results[i] && (!d_add || d_add[i]), "buffer %d is NULL", i);
        if (d_add) {
            k_unstack_add<<<grid_for(st, outer * inner, kThreads * 2), kThreads, 0, st->stream>>>(d_stacked + off, total_inner, d_add[i],
                                                                                               d_results[i], outer, inner);
            DL4S_TRY(after_launch(st, "k_unstack_add"));
        } else {
            DL4S_CUDA_TRY(cudaMemcpy2DAsync(d_results[i], (size_t)inner * sizeof(float), d_stacked + off,
                                            (size_t)total_inner * sizeof(float), (size_t)inner * sizeof(float), (size_t)outer,
                                            cudaMemcpyDeviceToDevice, st->stream));
        }
        off += inner;
    }
    return DL4S_OK;
}

dl4s_status dl4s_cuda_unstack(const float *d_stacked, float *const *d_results, const int64_t *shapes, int32_t n, int32_t dim,
                              int32_t axis)
{
    return unstack_impl(d_stacked, nullptr, d_results, shapes, n, dim, axis);
}

dl4s_status dl4s_cuda_unstack_add(const float *d_stacked, const float *const *d_add, float *const *d_results, const int64_t *shapes,
                                  int32_t n, int32_t dim, int32_t axis)
{
    DL4S_REQUIRE(d_add, "add is NULL");
    return unstack_impl(d_stacked, d_add, d_results, shapes, n, dim, axis);
}

dl4s_status dl4s_cuda_set_dropout(float rate, uint64_t seed)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(rate >= 0.f && rate < 1.f, "the dropout rate must lie in [0, 1) (got %g)", (double)rate);
    st->dropout_rate = rate;
    st->dropout_seed = seed;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_dropout_counter(uint32_t *current, const uint32_t *set_to)
{
    DL4S_STATE(st);
    if (set_to) st->dropout_counter = *set_to;
    if (current) *current = st->dropout_counter;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_dropout(const float *d_x, float *d_result, int64_t count, float rate, uint64_t seed, uint32_t counter)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(count >= 0 && (count == 0 || (d_x && d_result)), "bad arguments");
    DL4S_REQUIRE(rate >= 0.f && rate < 1.f, "the dropout rate must lie in [0, 1) (got %g)", (double)rate);
    if (count == 0) return DL4S_OK;
    DropoutSpec d;
    if (rate > 0.f) {
        double keep = (1.0 - (double)rate) * 4294967296.0;
        d.threshold = keep >= 4294967295.0 ? 0xFFFFFFFFu : (keep < 1.0 ? 1u : (uint32_t)keep);
        d.seed_lo = (uint32_t)seed;
        d.seed_hi = (uint32_t)(seed >> 32);
        d.counter = counter;
    }
    k_dropout<<<grid_for(st, count, kThreads * 2), kThreads, 0, st->stream>>>(d_x, d_result, count, d);
    return after_launch(st, "k_dropout");
}

dl4s_status dl4s_cuda_band(const float *d_src, int64_t rows, int64_t cols, int32_t below, int32_t has_below, int32_t above,
                           int32_t has_above, float *d_result)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_src && d_result && rows >= 0 && cols >= 0, "bad arguments");
    if (rows * cols == 0) return DL4S_OK;
    int64_t big = rows > cols ? rows : cols;
    int64_t bd = has_below ? below : big, ad = has_above ? above : big;
    k_band<<<grid_for(st, rows * cols, kThreads * 2), kThreads, 0, st->stream>>>(d_src, d_result, rows, cols, bd, ad);
    return after_launch(st, "k_band");
}

}  // extern "C"
