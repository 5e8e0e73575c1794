// The tensor-core pipeline of MultiHeadAttention, PointwiseFeedForward and
// TransformerEncoder (DL4S_PREC_F16 / DL4S_PREC_F16_SPLIT): the kernel sequence with every
// intermediate that only feeds a tensor-core operand kept in half precision and
// written by the kernel that produces it, so no conversion or permute pass runs
// between kernels.
//
// Per encoder layer (TransformerEncoderBlock.swift:58-65), x fp32 [M,D], M = B*S:
//   1 GEMM   x_h [M,D] x Wqkv_h [D,3*H*d]  -> Qh, Kh, Vh half [B,H,S,d] (q pre-scaled)   MultiHeadAttention.swift:109-115
//   2 attention (tcgen05)                   -> heads_h half [M,H*d]                        :117-119
//   3 GEMM   heads_h x Wo_h + x             -> pr fp32 [M,D]                               :121-123
//   4 LayerNorm over [S,D] per batch elem.  -> y fp32 + y_h half                           :124
//   5 GEMM   y_h x W1_h + b1, GeLU          -> h_h half [M,F]                              PointwiseFeedForward.swift:74-76
//   6 GEMM   h_h x W2_h + b2 + y            -> o fp32 [M,D]                                :77-79
//   7 LayerNorm per row                     -> out fp32 + out_h half (next layer's x_h)   :79
// Weights are converted to half once per call, or once per model when the caller prepares
// them (dl4s_cuda_encoder_prepare); q, k and v matrices are concatenated column-wise into
// one operand. Activations are rounded to half exactly once; products accumulate in fp32.
//
// DL4S_PREC_F16_SPLIT keeps every weight matrix as two halves, W_hi = half(W) and
// W_lo = half(W - W_hi), stacked along k, and the GEMMs accumulate A W_hi + A W_lo: the
// weights enter with ~22 significant bits for twice the MMA work. Rounding the weights is what
// dominates the error of a deep stack: a weight's rounding error is the same for every token
// and adds up layer after layer, the activations' errors do not. On a 6-layer encoder
// (d_model 512, 8 heads, d_ff 2048) single-rounded weights give relative L2 6.7e-4 and
// max-abs 3e-3 against the CPU engine, split weights 2.9e-4 and 1.5e-3.
#include "tc.cuh"

#include <cmath>

namespace dl4s {

// Two-half weights in the q/k/v projection: only the value columns take the remainder W_lo. The rounding of Wq and Wk
// moves the scores before a softmax that averages over hundreds of keys and is not visible in the encoder's output
// (the 6-layer configuration's error is the same with and without their remainders), while Wv's goes straight into
// the residual stream.
constexpr bool kSplitValueOnly = true;

// fp32 [rows, na] | [rows, nb] | [rows, nc] -> half [rows, na+nb+nc] (b, c optional); the first block is multiplied
// by a_scale before it is rounded (Wq carries the log2(e)/temperature factor of the scores, so the projection's
// epilogue has nothing to multiply);
// lo_off != 0: the half-rounded remainders go `lo_off` elements further (the split form).
__global__ void __launch_bounds__(256) k_concat_cols_f16(const float *__restrict__ a, int na, const float *__restrict__ b, int nb,
                                                         const float *__restrict__ c, int nc, int64_t rows, __half *__restrict__ out,
                                                         int64_t lo_off, float a_scale, int32_t *status)
{
    pdl_launch_dependents();
    pdl_wait();
    bool bad = false;
    const int n = na + nb + nc;
    const int64_t total = rows * (n / 4);
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < total; i += stride) {
        int64_t r = i / (n / 4);
        int col = (int)(i % (n / 4)) * 4;
        const float *src;
        if (col < na) src = a + r * na + col;
        else if (col < na + nb) src = b + r * nb + (col - na);
        else src = c + r * nc + (col - na - nb);
        float4 v = *reinterpret_cast<const float4 *>(src);
        if (col < na) { v.x *= a_scale; v.y *= a_scale; v.z *= a_scale; v.w *= a_scale; }
        uint2 hi, lo;
        split_hilo(v, hi, lo);
        bad |= half2_not_finite(hi.x) | half2_not_finite(hi.y);
        *reinterpret_cast<uint2 *>(out + r * n + col) = hi;
        if (lo_off) *reinterpret_cast<uint2 *>(out + lo_off + r * n + col) = lo;
    }
    if (bad) atomicOr(status, kStatusHalfRange);
}

static dl4s_status concat_cols_f16(DeviceState *st, const float *a, int na, const float *b, int nb, const float *c, int nc,
                                   int64_t rows, void *out, int split, float a_scale)
{
    DL4S_REQUIRE(na % 4 == 0 && nb % 4 == 0 && nc % 4 == 0, "column counts must be multiples of 4");
    int64_t total = rows * ((na + nb + nc) / 4);
    int64_t blocks = ceil_div(total, 256 * 4);
    int64_t cap = (int64_t)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const int64_t lo_off = split ? rows * (na + nb + nc) : 0;
    DL4S_CUDA_TRY(launch_pdl(st, k_concat_cols_f16, dim3((unsigned)blocks), dim3(256), 0, 1, a, na, b, nb, c, nc, rows, (__half *)out,
                             lo_off, a_scale, st->status_word));
    return after_launch(st, "k_concat_cols_f16");
}

// One weight matrix to half (split: [hi; lo] stacked along k).
static dl4s_status weight_to_f16(DeviceState *st, const float *w, void *out, int64_t n, int split)
{
    if (split) return launch_f32_to_f16_hilo(st, w, out, (__half *)out + n, n);
    return launch_f32_to_f16(st, w, out, n);
}

// All tensor-core weights of all encoder layers to half in ONE launch (blockIdx.y = layer):
// [Wq|Wk|Wv] concatenated column-wise, then Wo, W1, W2. Source and destination of layer l
// lie at constant strides from those of layer 0. split: every matrix is followed by its remainders.
struct LayerWeightsArgs {
    const float *src;        // layer 0 parameter block
    int64_t src_stride;      // floats per layer
    char *dst;               // layer 0 half weights (wqkv, then wo, w1, w2 at the byte offsets below)
    int64_t dst_stride;      // bytes per layer
    int64_t off_wo, off_w1, off_w2;   // destination byte offsets inside a layer
    int D, Nq, Nv, F;
    int split;
    float q_scale;           // Wq is multiplied by it before rounding (see k_concat_cols_f16)
    int32_t *status;
};

__global__ void __launch_bounds__(256) k_layer_weights_f16(LayerWeightsArgs a)
{
    pdl_launch_dependents();
    pdl_wait();
    const float *src = a.src + (int64_t)blockIdx.y * a.src_stride;
    char *dst = a.dst + (int64_t)blockIdx.y * a.dst_stride;
    const int nqkv = 2 * a.Nq + a.Nv;
    const int64_t g_qkv = (int64_t)a.D * nqkv / 4, g_wo = (int64_t)a.Nv * a.D / 4, g_w1 = (int64_t)a.D * a.F / 4;
    const int64_t total = g_qkv + g_wo + 2 * g_w1;
    // parameter order inside a layer: Wq, Wk [D,Nq], Wv [D,Nv], Wo [Nv,D], ln1 scale, shift [D], W1 [D,F], b1 [F], W2 [F,D]
    const float *wq = src, *wk = wq + (int64_t)a.D * a.Nq, *wv = wk + (int64_t)a.D * a.Nq, *wo = wv + (int64_t)a.D * a.Nv;
    const float *w1 = wo + (int64_t)a.Nv * a.D + 2 * a.D, *w2 = w1 + (int64_t)a.D * a.F + a.F;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float *s;
        __half *d;
        int64_t lo_off;   // elements from a matrix's rounded values to its remainders
        float scale = 1.0f;
        if (i < g_qkv) {
            // 32-bit index arithmetic: the q/k/v block of one layer has far fewer than 2^31 groups
            const unsigned per_row = (unsigned)(nqkv / 4);
            const unsigned r = (unsigned)i / per_row;
            const int col = (int)((unsigned)i - r * per_row) * 4;
            if (col < a.Nq) { s = wq + (int64_t)r * a.Nq + col; scale = a.q_scale; }
            else if (col < 2 * a.Nq) s = wk + (int64_t)r * a.Nq + (col - a.Nq);
            else s = wv + (int64_t)r * a.Nv + (col - 2 * a.Nq);
            d = reinterpret_cast<__half *>(dst) + (int64_t)r * nqkv + col;
            lo_off = (int64_t)a.D * nqkv;
        } else if (i < g_qkv + g_wo) {
            int64_t j = (i - g_qkv) * 4;
            s = wo + j;
            d = reinterpret_cast<__half *>(dst + a.off_wo) + j;
            lo_off = (int64_t)a.Nv * a.D;
        } else if (i < g_qkv + g_wo + g_w1) {
            int64_t j = (i - g_qkv - g_wo) * 4;
            s = w1 + j;
            d = reinterpret_cast<__half *>(dst + a.off_w1) + j;
            lo_off = (int64_t)a.D * a.F;
        } else {
            int64_t j = (i - g_qkv - g_wo - g_w1) * 4;
            s = w2 + j;
            d = reinterpret_cast<__half *>(dst + a.off_w2) + j;
            lo_off = (int64_t)a.D * a.F;
        }
        float4 v = *reinterpret_cast<const float4 *>(s);
        v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
        uint2 hi, lo;
        split_hilo(v, hi, lo);
        bad |= half2_not_finite(hi.x) | half2_not_finite(hi.y);
        *reinterpret_cast<uint2 *>(d) = hi;
        if (a.split) *reinterpret_cast<uint2 *>(d + lo_off) = lo;
    }
    if (bad) atomicOr(a.status, kStatusHalfRange);
}

// Carves 1 KiB-aligned pieces out of one scratch block; with base == nullptr it only adds up sizes.
struct Bump {
    char *base;
    size_t off = 0;
    explicit Bump(void *b) : base(static_cast<char *>(b)) {}
    void *take(size_t bytes)
    {
        void *p = base ? base + off : nullptr;
        off += align_up(bytes ? bytes : 1, 1024);
        return p;
    }
};

bool tc_block_supported(int64_t B, int64_t Sq, int64_t Sk, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F)
{
    if (!(dk == dv && (dk == 64 || dk == 128))) return false;
    if (!attn_prefill_tc_supported(Sq, Sk, dk, dv) || B * H > 65535) return false;
    const int64_t Mq = B * Sq, Mk = B * Sk;
    if (!gemm_tc_supported(Mq, H * dk, D) || !gemm_tc_supported(Mk, H * dk, D) || !gemm_tc_supported(Mq, D, H * dv)) return false;
    if (F > 0 && (!gemm_tc_supported(Mq, F, D) || !gemm_tc_supported(Mq, D, F))) return false;
    return D % 4 == 0;
}

struct MhaTcBuffers {
    void *wqkv_h, *wo_h;           // prepared weights (null: prepare here)
    void *xq_h, *xk_h, *xv_h;      // half copies of the inputs (null: convert here)
    void *qh, *kh, *vh, *heads_h;
    float *pr;
};

// Lays the MHA scratch out (or measures it). `have_w` / `have_xh`: the caller supplies prepared weights / a half copy of x.
static size_t mha_tc_layout(Bump &bp, MhaTcBuffers &m, int64_t B, int64_t Sq, int64_t Sk, int64_t D, int64_t H, int64_t dk,
                            int64_t dv, bool self, bool have_w, bool have_xh, int split)
{
    const size_t wmul = split ? 4 : 2;   // bytes per weight element
    if (!have_w) {
        m.wqkv_h = bp.take((size_t)(D * (2 * H * dk + H * dv)) * wmul);
        m.wo_h = bp.take((size_t)(H * dv * D) * wmul);
    }
    if (!have_xh) {
        m.xq_h = bp.take((size_t)(B * Sq * D) * 2);
        m.xk_h = self ? m.xq_h : bp.take((size_t)(B * Sk * D) * 2);
        m.xv_h = self ? m.xq_h : bp.take((size_t)(B * Sk * D) * 2);
    }
    m.qh = bp.take((size_t)(B * H * Sq * dk) * 2);
    m.kh = bp.take((size_t)(B * H * Sk * dk) * 2);
    m.vh = bp.take((size_t)(B * H * Sk * dv) * 2);
    m.heads_h = bp.take((size_t)(B * Sq * H * dv) * 2);
    m.pr = (float *)bp.take((size_t)(B * Sq * D) * 4);
    return bp.off;
}

// MultiHeadAttention.swift:97-127 on the tensor cores. xq/xk/xv fp32; when `self` they are one tensor.
// out fp32 [B,Sq,D]; out_h (optional) the same values in half.
static dl4s_status mha_tc_run(DeviceState *st, const float *xq, const float *xk, const float *xv, bool self, int64_t B,
                              int64_t Sq, int64_t Sk, int64_t D, int64_t H, int64_t dk, int64_t dv, const float *wq,
                              const float *wk, const float *wv, const float *wo, const float *g, const float *sh,
                              const MaskSpec &mask, float *out, void *out_h, MhaTcBuffers m, bool have_w, bool have_xh, int split)
{
    ScopedGroup group(st, "MultiHeadAttention");
    const int Nq = (int)(H * dk), Nv = (int)(H * dv);
    const float q_scale = attn_prefill_tc_q_scale(1.0f / sqrtf((float)dk));
    if (!have_w) {
        DL4S_TRY(concat_cols_f16(st, wq, Nq, wk, Nq, wv, Nv, D, m.wqkv_h, split, q_scale));
        DL4S_TRY(weight_to_f16(st, wo, m.wo_h, H * dv * D, split));
    }
    if (!have_xh) {
        DL4S_TRY(launch_f32_to_f16(st, xq, m.xq_h, B * Sq * D));
        if (!self) {
            DL4S_TRY(launch_f32_to_f16(st, xk, m.xk_h, B * Sk * D));
            DL4S_TRY(launch_f32_to_f16(st, xv, m.xv_h, B * Sk * D));
        }
    }
    GemmTcOut o;
    o.mode = OUT_HEADS_F16;
    o.H = (int)H;
    if (self) {
        o.nparts = 3; o.S = (int)Sq;
        o.part_ptr[0] = m.qh; o.part_ptr[1] = m.kh; o.part_ptr[2] = m.vh;
        o.part_d[0] = (int)dk; o.part_d[1] = (int)dk; o.part_d[2] = (int)dv;
        DL4S_TRY(launch_gemm_tc_h(st, m.xq_h, m.wqkv_h, B * Sq, 2 * Nq + Nv, D, EPI_NONE, nullptr, nullptr, o, 1, 0, split, nullptr,
                                  kSplitValueOnly ? 2 * Nq : 0));
    } else {
        // Distinct query / key / value inputs: three products against the column blocks of the
        // concatenated weights are not contiguous operands, so the weights are taken apart again.
        return fail(DL4S_ERR_UNSUPPORTED, "internal: cross-attention takes the unfused tensor-core path");
    }
    {
        ScopedGroup sdpa(st, "ScaledDotProductAttention");
        DL4S_TRY(launch_attn_prefill_tc_h(st, m.qh, m.kh, m.vh, m.heads_h, strides_bshd(H, Sq, dv), 1, B, H, Sq, Sk, dk, mask));
    }
    GemmTcOut po;
    po.mode = OUT_F32;
    po.c = m.pr;
    // The Wo epilogue leaves the LayerNorm's partial sums when the block shape allows it: one pass less over pr.
    const int parts = gemm_tc_stats_per_row_block(D);
    const DropoutSpec drop = next_dropout(st);   // MultiHeadAttention.swift:122
    if (layernorm_stats_usable(B, Sq, D, parts)) {
        po.ln_stats = st->ln_partials;
        DL4S_TRY(launch_gemm_tc_h(st, m.heads_h, m.wo_h, B * Sq, D, Nv, EPI_RESIDUAL_STATS, nullptr, xq, po, 1, 0, split, &drop));
        ScopedGroup ln(st, "LayerNorm");
        return launch_layernorm_from_stats(st, m.pr, B, Sq, D, g, sh, out, out_h, st->ln_partials, parts);
    }
    DL4S_TRY(launch_gemm_tc_h(st, m.heads_h, m.wo_h, B * Sq, D, Nv, EPI_RESIDUAL, nullptr, xq, po, 1, 0, split, &drop));
    ScopedGroup ln(st, "LayerNorm");
    return launch_layernorm(st, m.pr, nullptr, B, Sq, D, g, sh, out, out_h);
}

struct FfnTcBuffers {
    void *w1_h, *w2_h, *x_h, *h_h;
    float *o;
};

static size_t ffn_tc_layout(Bump &bp, FfnTcBuffers &f, int64_t M, int64_t D, int64_t F, bool have_w, bool have_xh, int split)
{
    const size_t wmul = split ? 4 : 2;
    if (!have_w) {
        f.w1_h = bp.take((size_t)(D * F) * wmul);
        f.w2_h = bp.take((size_t)(F * D) * wmul);
    }
    if (!have_xh) f.x_h = bp.take((size_t)(M * D) * 2);
    f.h_h = bp.take((size_t)(M * F) * 2);
    f.o = (float *)bp.take((size_t)(M * D) * 4);
    return bp.off;
}

// PointwiseFeedForward.swift:67-82 on the tensor cores.
static dl4s_status ffn_tc_run(DeviceState *st, const float *x, int64_t M, int64_t D, int64_t F, const float *w1, const float *b1,
                              const float *w2, const float *b2, const float *g, const float *sh, int act, float *out,
                              void *out_h, FfnTcBuffers f, bool have_w, bool have_xh, int split)
{
    ScopedGroup group(st, "PointwiseFeedForward");
    if (!have_w) {
        DL4S_TRY(weight_to_f16(st, w1, f.w1_h, D * F, split));
        DL4S_TRY(weight_to_f16(st, w2, f.w2_h, F * D, split));
    }
    if (!have_xh) DL4S_TRY(launch_f32_to_f16(st, x, f.x_h, M * D));
    GemmTcOut ho;
    ho.mode = OUT_F16;
    ho.c = f.h_h;
    {
        ScopedGroup dense(st, "Dense");
        DL4S_TRY(launch_gemm_tc_h(st, f.x_h, f.w1_h, M, F, D, act == DL4S_ACT_RELU ? EPI_BIAS_RELU : EPI_BIAS_GELU, b1, nullptr, ho, 1,
                                  0, split));
    }
    GemmTcOut oo;
    oo.mode = OUT_F32;
    oo.c = f.o;
    {
        ScopedGroup dense(st, "Dense");
        const DropoutSpec drop = next_dropout(st);   // PointwiseFeedForward.swift:78
        DL4S_TRY(launch_gemm_tc_h(st, f.h_h, f.w2_h, M, D, F, EPI_BIAS_RESIDUAL, b2, x, oo, 1, 0, split, &drop));
    }
    ScopedGroup ln(st, "LayerNorm");
    return launch_layernorm(st, f.o, nullptr, M, 1, D, g, sh, out, out_h);
}

dl4s_status mha_self_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                        const float *wq, const float *wk, const float *wv, const float *wo, const float *g, const float *sh,
                        const MaskSpec &mask, float *out, int split)
{
    MhaTcBuffers m{};
    Bump measure(nullptr);
    size_t need = mha_tc_layout(measure, m, B, S, S, D, H, dk, dv, true, false, false, split);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, need, &base));
    Bump bp(base);
    mha_tc_layout(bp, m, B, S, S, D, H, dk, dv, true, false, false, split);
    return mha_tc_run(st, x, x, x, true, B, S, S, D, H, dk, dv, wq, wk, wv, wo, g, sh, mask, out, nullptr, m, false, false, split);
}

// First half of self-attention MultiHeadAttention for the H heads one GPU owns (MultiHeadAttention.swift:109-119):
// one fused q/k/v product into head-major halves, attention, result [B,S,H*dv] as fp32 or half.
dl4s_status mha_heads_self_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk,
                              int64_t dv, const float *wq, const float *wk, const float *wv, const MaskSpec &mask, void *out,
                              int out_half, int split, const void *x_half)
{
    const int Nq = (int)(H * dk), Nv = (int)(H * dv);
    auto layout = [&](Bump &bp, void **w, void **xh, void **qh, void **kh, void **vh) {
        *w = bp.take((size_t)(D * (2 * Nq + Nv)) * (split ? 4 : 2));
        *xh = x_half ? nullptr : bp.take((size_t)(B * S * D) * 2);   // the caller may hold the half copy already
        *qh = bp.take((size_t)(B * H * S * dk) * 2);
        *kh = bp.take((size_t)(B * H * S * dk) * 2);
        *vh = bp.take((size_t)(B * H * S * dv) * 2);
        return bp.off;
    };
    void *w = nullptr, *xh = nullptr, *qh = nullptr, *kh = nullptr, *vh = nullptr;
    Bump measure(nullptr);
    size_t need = layout(measure, &w, &xh, &qh, &kh, &vh);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, need, &base));
    Bump bp(base);
    layout(bp, &w, &xh, &qh, &kh, &vh);
    DL4S_TRY(concat_cols_f16(st, wq, Nq, wk, Nq, wv, Nv, D, w, split, attn_prefill_tc_q_scale(1.0f / sqrtf((float)dk))));
    if (x_half) xh = const_cast<void *>(x_half);
    else DL4S_TRY(launch_f32_to_f16(st, x, xh, B * S * D));
    GemmTcOut o;
    o.mode = OUT_HEADS_F16;
    o.H = (int)H; o.S = (int)S; o.nparts = 3;
    o.part_ptr[0] = qh; o.part_ptr[1] = kh; o.part_ptr[2] = vh;
    o.part_d[0] = (int)dk; o.part_d[1] = (int)dk; o.part_d[2] = (int)dv;
    DL4S_TRY(launch_gemm_tc_h(st, xh, w, B * S, 2 * Nq + Nv, D, EPI_NONE, nullptr, nullptr, o, 1, 0, split, nullptr,
                              kSplitValueOnly ? 2 * Nq : 0));
    return launch_attn_prefill_tc_h(st, qh, kh, vh, out, strides_bshd(H, S, dv), out_half, B, H, S, S, dk, mask);
}

// Second half (MultiHeadAttention.swift:121-124): heads [B*S,HDv] (fp32 or half) x Wo + residual, LayerNorm per batch element.
dl4s_status mha_output_tc(DeviceState *st, const void *heads, int heads_half, const float *residual, int64_t B, int64_t S,
                          int64_t D, int64_t HDv, const float *wo, const float *g, const float *sh, float *out, int64_t groups,
                          int64_t group_stride, int split)
{
    // `heads` may be the rank-major result of an all-gather, [groups][B*S][HDv/groups] with `group_stride`
    // elements between groups: the GEMM's tensor map walks it as it lies, no row rebuild.
    const int64_t M = B * S, C = HDv / groups;
    auto layout = [&](Bump &bp, void **w, void **hh, float **pr) {
        *w = bp.take((size_t)(HDv * D) * (split ? 4 : 2));
        *hh = heads_half ? nullptr : bp.take((size_t)(B * S * HDv) * 2);
        *pr = (float *)bp.take((size_t)(B * S * D) * 4);
        return bp.off;
    };
    void *w = nullptr, *hh = nullptr;
    float *pr = nullptr;
    Bump measure(nullptr);
    size_t need = layout(measure, &w, &hh, &pr);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, need, &base));
    Bump bp(base);
    layout(bp, &w, &hh, &pr);
    DL4S_TRY(weight_to_f16(st, wo, w, HDv * D, split));
    const void *a = heads;
    if (!heads_half) {
        for (int64_t gi = 0; gi < groups; ++gi)
            DL4S_TRY(launch_f32_to_f16(st, static_cast<const float *>(heads) + gi * group_stride, (__half *)hh + gi * M * C, M * C));
        a = hh;
        group_stride = M * C;
    }
    GemmTcOut po;
    po.mode = OUT_F32;
    po.c = pr;
    // As in the whole layer: the epilogue leaves the LayerNorm's partial sums where the block shape allows it.
    const int parts = gemm_tc_stats_per_row_block(D);
    const DropoutSpec drop = next_dropout(st);   // MultiHeadAttention.swift:122
    if (layernorm_stats_usable(B, S, D, parts)) {
        po.ln_stats = st->ln_partials;
        DL4S_TRY(launch_gemm_tc_h(st, a, w, M, D, HDv, EPI_RESIDUAL_STATS, nullptr, residual, po, groups, group_stride, split, &drop));
        return launch_layernorm_from_stats(st, pr, B, S, D, g, sh, out, nullptr, st->ln_partials, parts);
    }
    DL4S_TRY(launch_gemm_tc_h(st, a, w, M, D, HDv, EPI_RESIDUAL, nullptr, residual, po, groups, group_stride, split, &drop));
    return launch_layernorm(st, pr, nullptr, B, S, D, g, sh, out, nullptr);
}

dl4s_status ffn_tc(DeviceState *st, const float *x, int64_t M, int64_t D, int64_t F, const float *w1, const float *b1,
                   const float *w2, const float *b2, const float *g, const float *sh, int act, float *out, int split)
{
    FfnTcBuffers f{};
    Bump measure(nullptr);
    size_t need = ffn_tc_layout(measure, f, M, D, F, false, false, split);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, need, &base));
    Bump bp(base);
    ffn_tc_layout(bp, f, M, D, F, false, false, split);
    return ffn_tc_run(st, x, M, D, F, w1, b1, w2, b2, g, sh, act, out, nullptr, f, false, false, split);
}

// ------------------------------------------------------------------------------------------------ encoder
constexpr int kMaxLayers = 64;

struct LayerW { void *wqkv_h, *wo_h, *w1_h, *w2_h; };
struct LayerP { const float *wq, *wk, *wv, *wo, *g1, *s1, *w1, *b1, *w2, *b2, *g2, *s2; };

// The half weights of a whole encoder, converted once and kept (dl4s_cuda_encoder_prepare). LayerNorm parameters
// and biases are read from the caller's fp32 parameter block on every forward.
struct EncoderPrepared {
    uint32_t magic = 0x454e4350;   // "ENCP"
    int device = -1;
    int64_t D = 0, H = 0, dk = 0, dv = 0, F = 0, layers = 0;
    int split = 0;
    const float *params = nullptr;
    void *block = nullptr;
    size_t bytes = 0;
    LayerW lw[kMaxLayers];
};

static size_t layer_weights_layout(Bump &bp, LayerW *lw, int64_t D, int64_t Nq, int64_t Nv, int64_t F, int64_t layers, int split)
{
    const size_t wmul = split ? 4 : 2;
    for (int64_t l = 0; l < layers; ++l) {
        lw[l].wqkv_h = bp.take((size_t)(D * (2 * Nq + Nv)) * wmul);
        lw[l].wo_h = bp.take((size_t)(Nv * D) * wmul);
        lw[l].w1_h = bp.take((size_t)(D * F) * wmul);
        lw[l].w2_h = bp.take((size_t)(F * D) * wmul);
    }
    return bp.off;
}

static int64_t layer_param_floats(int64_t D, int64_t Nq, int64_t Nv, int64_t F)
{
    return 2 * D * Nq + D * Nv + Nv * D + 2 * D + D * F + F + F * D + D + 2 * D;
}

static void layer_param_pointers(const float *params, LayerP *lp, int64_t D, int64_t Nq, int64_t Nv, int64_t F, int64_t layers)
{
    const float *p = params;
    for (int64_t l = 0; l < layers; ++l) {
        lp[l].wq = p; p += D * Nq;
        lp[l].wk = p; p += D * Nq;
        lp[l].wv = p; p += D * Nv;
        lp[l].wo = p; p += Nv * D;
        lp[l].g1 = p; p += D;
        lp[l].s1 = p; p += D;
        lp[l].w1 = p; p += D * F;
        lp[l].b1 = p; p += F;
        lp[l].w2 = p; p += F * D;
        lp[l].b2 = p; p += D;
        lp[l].g2 = p; p += D;
        lp[l].s2 = p; p += D;
    }
}

// All weights of all layers to half (one launch).
static dl4s_status convert_layer_weights(DeviceState *st, const float *params, const LayerW *lw, int64_t D, int64_t Nq, int64_t Nv,
                                         int64_t F, int64_t layers, int split, float q_scale)
{
    DL4S_REQUIRE(((uintptr_t)params & 15) == 0, "the parameter block must be 16-byte aligned");
    DL4S_REQUIRE(D % 4 == 0 && Nq % 4 == 0 && Nv % 4 == 0 && F % 4 == 0, "weight extents must be multiples of 4");
    LayerWeightsArgs a;
    a.src = params;
    a.src_stride = layer_param_floats(D, Nq, Nv, F);
    a.dst = static_cast<char *>(lw[0].wqkv_h);
    a.dst_stride = layers > 1 ? static_cast<char *>(lw[1].wqkv_h) - static_cast<char *>(lw[0].wqkv_h) : 0;
    a.off_wo = static_cast<char *>(lw[0].wo_h) - a.dst;
    a.off_w1 = static_cast<char *>(lw[0].w1_h) - a.dst;
    a.off_w2 = static_cast<char *>(lw[0].w2_h) - a.dst;
    a.D = (int)D; a.Nq = (int)Nq; a.Nv = (int)Nv; a.F = (int)F;
    a.split = split;
    a.q_scale = q_scale;
    a.status = st->status_word;
    DL4S_REQUIRE(D * (2 * Nq + Nv) / 4 < (1ll << 31), "projection weights too large for the conversion kernel's index arithmetic");
    int64_t groups = (D * (2 * Nq + Nv) + Nv * D + 2 * D * F) / 4;
    int64_t bx = ceil_div(groups, 256 * 4);
    int64_t cap = ceil_div((int64_t)st->sm_count * 8, layers);
    if (bx > cap) bx = cap;
    if (bx < 1) bx = 1;
    dim3 grid((unsigned)bx, (unsigned)layers);
    DL4S_CUDA_TRY(launch_pdl(st, k_layer_weights_f16, grid, dim3(256), 0, 1, a));
    return after_launch(st, "k_layer_weights_f16");
}

// TransformerEncoder.swift:61-71 on the tensor cores; `params` in the order of dl4s_cuda_encoder_forward.
// `prep` (optional): half weights converted earlier; otherwise they are converted here, once per call.
static dl4s_status encoder_tc_run(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk,
                                  int64_t dv, int64_t F, int64_t layers, const float *params, const MaskSpec &mask, int act,
                                  float *out, int split, const EncoderPrepared *prep)
{
    ScopedGroup group(st, "Encoder");
    const int64_t M = B * S;
    const int64_t Nq = H * dk, Nv = H * dv;
    DL4S_REQUIRE(layers <= kMaxLayers, "at most %d layers", kMaxLayers);
    auto layout = [&](Bump &bp, LayerW *lw, MhaTcBuffers &m, FfnTcBuffers &f, void **xh, float **act32, void **acth) {
        if (!prep) layer_weights_layout(bp, lw, D, Nq, Nv, F, layers, split);
        *xh = bp.take((size_t)(M * D) * 2);            // half copy of the layer input
        act32[0] = (float *)bp.take((size_t)(M * D) * 4);   // attention block output y
        acth[0] = bp.take((size_t)(M * D) * 2);
        act32[1] = (float *)bp.take((size_t)(M * D) * 4);   // layer output (all but the last layer)
        mha_tc_layout(bp, m, B, S, S, D, H, dk, dv, true, true, true, split);
        ffn_tc_layout(bp, f, M, D, F, true, true, split);
        return bp.off;
    };
    LayerW lw_local[kMaxLayers];
    MhaTcBuffers m{};
    FfnTcBuffers f{};
    void *xh = nullptr, *acth[1] = {nullptr};
    float *act32[2] = {nullptr, nullptr};
    Bump measure(nullptr);
    size_t need = layout(measure, lw_local, m, f, &xh, act32, acth);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, need, &base));
    Bump bp(base);
    layout(bp, lw_local, m, f, &xh, act32, acth);
    const LayerW *lw = prep ? prep->lw : lw_local;

    LayerP lp[kMaxLayers];
    layer_param_pointers(params, lp, D, Nq, Nv, F, layers);
    if (!prep) DL4S_TRY(convert_layer_weights(st, params, lw, D, Nq, Nv, F, layers, split, attn_prefill_tc_q_scale(1.0f / sqrtf((float)dk))));
    DL4S_TRY(launch_f32_to_f16(st, x, xh, M * D));
    const float *cur = x;
    for (int64_t l = 0; l < layers; ++l) {
        ScopedGroup layer(st, "EncoderLayer");
        m.wqkv_h = lw[l].wqkv_h; m.wo_h = lw[l].wo_h;
        m.xq_h = m.xk_h = m.xv_h = xh;
        DL4S_TRY(mha_tc_run(st, cur, cur, cur, true, B, S, S, D, H, dk, dv, nullptr, nullptr, nullptr, nullptr, lp[l].g1, lp[l].s1,
                            mask, act32[0], acth[0], m, true, true, split));
        f.w1_h = lw[l].w1_h; f.w2_h = lw[l].w2_h; f.x_h = acth[0];
        float *dst = (l == layers - 1) ? out : act32[1];
        // The half copy of the layer output becomes the next layer's x_h.
        DL4S_TRY(ffn_tc_run(st, act32[0], M, D, F, nullptr, lp[l].b1, nullptr, lp[l].b2, lp[l].g2, lp[l].s2, act, dst,
                            (l == layers - 1) ? nullptr : xh, f, true, true, split));
        cur = dst;
    }
    return DL4S_OK;
}

dl4s_status encoder_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                       int64_t F, int64_t layers, const float *params, const MaskSpec &mask, int act, float *out, int split)
{
    return encoder_tc_run(st, x, B, S, D, H, dk, dv, F, layers, params, mask, act, out, split, nullptr);
}

dl4s_status encoder_prepare(DeviceState *st, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int64_t layers,
                            const float *params, int split, void **handle)
{
    DL4S_REQUIRE(layers >= 1 && layers <= kMaxLayers, "between 1 and %d layers", kMaxLayers);
    DL4S_REQUIRE(!st->capturing, "prepare the weights before dl4s_cuda_graph_begin");
    EncoderPrepared *p = new EncoderPrepared();
    p->device = st->ordinal;
    p->D = D; p->H = H; p->dk = dk; p->dv = dv; p->F = F; p->layers = layers;
    p->split = split;
    p->params = params;
    Bump measure(nullptr);
    p->bytes = layer_weights_layout(measure, p->lw, D, H * dk, H * dv, F, layers, split);
    cudaError_t e = cudaMalloc(&p->block, p->bytes);
    if (e != cudaSuccess) {
        delete p;
        return check_cuda(e, "cudaMalloc(prepared encoder weights)");
    }
    Bump bp(p->block);
    layer_weights_layout(bp, p->lw, D, H * dk, H * dv, F, layers, split);
    dl4s_status s = convert_layer_weights(st, params, p->lw, D, H * dk, H * dv, F, layers, split,
                                          attn_prefill_tc_q_scale(1.0f / sqrtf((float)dk)));
    if (s != DL4S_OK) {
        cudaFree(p->block);
        delete p;
        return s;
    }
    *handle = p;
    return DL4S_OK;
}

static EncoderPrepared *as_prepared(DeviceState *st, void *handle)
{
    EncoderPrepared *p = static_cast<EncoderPrepared *>(handle);
    if (!p || p->magic != 0x454e4350) {
        fail(DL4S_ERR_INVALID_ARG, "not a handle of dl4s_cuda_encoder_prepare");
        return nullptr;
    }
    if (p->device != st->ordinal) {
        fail(DL4S_ERR_INVALID_ARG, "the weights were prepared on device %d, the current device is %d", p->device, st->ordinal);
        return nullptr;
    }
    return p;
}

dl4s_status encoder_prepared_refresh(DeviceState *st, void *handle)
{
    EncoderPrepared *p = as_prepared(st, handle);
    if (!p) return DL4S_ERR_INVALID_ARG;
    return convert_layer_weights(st, p->params, p->lw, p->D, p->H * p->dk, p->H * p->dv, p->F, p->layers, p->split,
                                 attn_prefill_tc_q_scale(1.0f / sqrtf((float)p->dk)));
}

dl4s_status encoder_prepared_destroy(DeviceState *st, void *handle)
{
    if (!handle) return DL4S_OK;
    EncoderPrepared *p = as_prepared(st, handle);
    if (!p) return DL4S_ERR_INVALID_ARG;
    DL4S_REQUIRE(!st->capturing, "free prepared weights after dl4s_cuda_graph_end");
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));   // a forward may still read them
    // a recorded graph may still name the block: it goes with the last graph
    DL4S_TRY(release_internal(st, p->block));
    p->magic = 0;
    delete p;
    return DL4S_OK;
}

dl4s_status encoder_tc_prepared(DeviceState *st, void *handle, const float *x, int64_t B, int64_t S, const MaskSpec &mask, int act,
                                float *out)
{
    EncoderPrepared *p = as_prepared(st, handle);
    if (!p) return DL4S_ERR_INVALID_ARG;
    if (!tc_block_supported(B, S, S, p->D, p->H, p->dk, p->dv, p->F))
        return fail(DL4S_ERR_UNSUPPORTED, "batch %lld x sequence %lld is outside the tensor-core pipeline's shapes; use "
                    "dl4s_cuda_encoder_forward", (long long)B, (long long)S);
    return encoder_tc_run(st, x, B, S, p->D, p->H, p->dk, p->dv, p->F, p->layers, p->params, mask, act, out, p->split, p);
}

}  // namespace dl4s
