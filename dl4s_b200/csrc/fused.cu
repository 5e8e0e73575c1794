// Host side of the fused entry points: argument checks, scratch layout and the
// kernel sequence of ScaledDotProductAttention, MultiHeadAttention,
// PointwiseFeedForward and TransformerEncoder. No arithmetic happens on the host.
#include "common.cuh"
#include "tc.cuh"

#include <cmath>

namespace dl4s {

// PE[s, 2i] = sin(s / f_i), PE[s, 2i+1] = cos(s / f_i), f_i = exp(ln(10000) * i / (D/2))
// (PositionalEncoding.swift:52-71). The table depends on (S, D) only, so it is computed once per
// device and kept. exp / sin / cos are evaluated in double and rounded once, which reproduces the
// correctly rounded fp32 results of the host libm the CPU engine calls; an fp32 device exp that is
// one ulp off would move sin(p / f) by p * 1e-7.
__global__ void __launch_bounds__(256) k_positional_table(int64_t S, int64_t D, float *__restrict__ pe)
{
    const int64_t half = D / 2;
    const float ln_base = logf(10000.0f);
    const float inv_half = 1.0f / (float)half;
    for (int64_t pos = blockIdx.x; pos < S; pos += gridDim.x) {
        for (int64_t i = threadIdx.x; i < half; i += blockDim.x) {
            float f = (float)exp((double)(((float)i * inv_half) * ln_base));
            float a = (float)pos / f;
            pe[pos * D + 2 * i] = (float)sin((double)a);
            pe[pos * D + 2 * i + 1] = (float)cos((double)a);
        }
    }
}

// x[b,s,:] = E[ids[b,s]] * sqrt(D) + PE[s,:]   (Transformer.swift:82-88, Embedding.swift:152-165).
// Two elements per thread step (D is even); an id equal to ignore_index or outside the vocabulary
// embeds as zeros.
__global__ void __launch_bounds__(256) k_embed_positional(const int32_t *__restrict__ ids, int64_t BS, int64_t S, int64_t D,
                                                          const float *__restrict__ E, int64_t vocab, int32_t ignore_index,
                                                          float scale, const float *__restrict__ pe, float *__restrict__ out,
                                                          DropoutSpec drop)
{
    const int64_t half = D / 2;
    for (int64_t row = blockIdx.x; row < BS; row += gridDim.x) {
        const int32_t id = ids[row];
        const int64_t pos = row % S;
        const bool zero = (id == ignore_index) || id < 0 || id >= vocab;
        const float2 *e = reinterpret_cast<const float2 *>(E + (zero ? 0 : (int64_t)id * D));
        const float2 *p = reinterpret_cast<const float2 *>(pe + pos * D);
        float2 *o = reinterpret_cast<float2 *>(out + row * D);
        for (int64_t i = threadIdx.x; i < half; i += blockDim.x) {
            float2 ev = zero ? make_float2(0.f, 0.f) : e[i];
            float2 pv = p[i];
            float2 r = make_float2(ev.x * scale + pv.x, ev.y * scale + pv.y);
            if (drop.threshold != 0) {   // dropout(embedded * sqrt(D) + positions), Transformer.swift:87
                const uint64_t e = (uint64_t)(row * D + 2 * i);
                r.x = dropout_keep(drop, e) ? r.x : 0.f;
                r.y = dropout_keep(drop, e + 1) ? r.y : 0.f;
            }
            o[i] = r;
        }
    }
}

// Incremental decoding: the current token's key and value rows go to position lengths[b] of the caches
// [B, H, Lmax, d], and lengths[b] + 1 (the keys the token may see, itself included) is written to len1.
// A full cache (lengths[b] >= Lmax) sets bit 0x200 of the status word and leaves the cache alone.
__global__ void __launch_bounds__(128) k_kv_append(const float *__restrict__ k_new, const float *__restrict__ v_new, int64_t H,
                                                   int64_t dk, int64_t dv, int64_t Lmax, const int32_t *__restrict__ lens,
                                                   float *__restrict__ k_cache, float *__restrict__ v_cache,
                                                   int32_t *__restrict__ len1, int32_t *status)
{
    const int64_t b = blockIdx.y, h = blockIdx.x;
    int len = lens[b];
    if (len < 0) len = 0;
    if (len >= Lmax) {
        if (threadIdx.x == 0) {
            atomicOr(status, kStatusCacheFull);
            if (h == 0) len1[b] = (int32_t)Lmax;
        }
        return;
    }
    if (threadIdx.x == 0 && h == 0) len1[b] = len + 1;
    const float *ks = k_new + (b * H + h) * dk;
    const float *vs = v_new + (b * H + h) * dv;
    float *kd = k_cache + ((b * H + h) * Lmax + len) * dk;
    float *vd = v_cache + ((b * H + h) * Lmax + len) * dv;
    for (int64_t i = threadIdx.x; i < dk; i += blockDim.x) kd[i] = ks[i];
    for (int64_t i = threadIdx.x; i < dv; i += blockDim.x) vd[i] = vs[i];
}

// DL4S_PREC_F16 and DL4S_PREC_F16_SPLIT both run on the tensor cores; the second keeps weights as two halves.
static inline bool prec_known(int p) { return p == DL4S_PREC_FP32 || p == DL4S_PREC_F16 || p == DL4S_PREC_F16_SPLIT; }
static inline bool prec_tc(int p) { return p == DL4S_PREC_F16 || p == DL4S_PREC_F16_SPLIT; }
static inline int prec_split(int p) { return p == DL4S_PREC_F16_SPLIT ? 1 : 0; }

// The sinusoidal table [rows, D] is built on first use and kept; it is rebuilt when D changes or more rows are needed.
dl4s_status ensure_positional_table(DeviceState *st, int64_t rows, int64_t D)
{
    if (st->pe_dim == D && st->pe_rows >= rows) return DL4S_OK;
    if (st->capturing)
        return fail(DL4S_ERR_UNSUPPORTED, "the positional-encoding table has to be built: run the call once before capturing");
    // the old table may still be in use by work queued on the stream
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    DL4S_TRY(release_internal(st, st->pe_table));
    st->pe_table = nullptr;
    st->pe_rows = 0;
    DL4S_CUDA_TRY(cudaMalloc((void **)&st->pe_table, (size_t)(rows * D) * sizeof(float)));
    st->pe_rows = rows;
    st->pe_dim = D;
    int64_t tb = rows < (int64_t)st->sm_count * 8 ? rows : (int64_t)st->sm_count * 8;
    k_positional_table<<<(unsigned)tb, 256, 0, st->stream>>>(rows, D, st->pe_table);
    return after_launch(st, "k_positional_table");
}

static dl4s_status check_mask(const MaskSpec &m, int64_t B, int64_t H, int64_t Sq, int64_t Sk)
{
    if (!m.d_mask) return DL4S_OK;
    const int64_t full[4] = {B, H, Sq, Sk};
    for (int i = 0; i < 4; ++i)
        DL4S_REQUIRE(m.ms[i] == 1 || m.ms[i] == full[i], "mask extent %d is %lld; it must be 1 or %lld", i,
                     (long long)m.ms[i], (long long)full[i]);
    return DL4S_OK;
}

static MaskSpec make_mask(const int32_t *lens, int causal, const float *mask, const int64_t *mshape)
{
    MaskSpec m;
    m.d_key_lengths = lens;
    m.causal = causal;
    m.d_mask = mask;
    if (mask && mshape) for (int i = 0; i < 4; ++i) m.ms[i] = mshape[i];
    return m;
}

// Attention on already projected, possibly strided q/k/v. Chooses the kernel.
static dl4s_status attention(DeviceState *st, const float *q, Strides4 qs, const float *k, Strides4 ks, const float *v,
                             Strides4 vs, float *o, Strides4 os, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk,
                             int64_t dv, float inv_t, const MaskSpec &mask, int precision, void *scratch, size_t scratch_bytes)
{
    ScopedGroup group(st, "ScaledDotProductAttention");
    // The tensor-core kernel covers structural masks and head sizes 64 / 128; everything
    // else (dense masks, odd head sizes) runs on the fp32 kernel, which is the more exact one.
    if (prec_tc(precision) && !mask.d_mask && attn_prefill_tc_supported(Sq, Sk, dk, dv))
        return launch_attn_prefill_tc(st, q, qs, k, ks, v, vs, o, os, B, H, Sq, Sk, dk, dv, inv_t, mask, scratch, scratch_bytes);
    return launch_attn_ref(st, q, qs, k, ks, v, vs, o, os, B, H, Sq, Sk, dk, dv, inv_t, mask);
}

static dl4s_status gemm(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K, int epi,
                        const float *bias, const float *residual, int precision, void *scratch, size_t scratch_bytes,
                        const DropoutSpec *drop = nullptr)
{
    if (prec_tc(precision) && gemm_tc_supported(M, N, K))
        return launch_gemm_tc(st, a, b, c, M, N, K, epi, bias, residual, scratch, scratch_bytes, prec_split(precision), drop);
    return launch_gemm_f32(st, a, b, c, M, N, K, 1.0f, 0.0f, 0, 0, epi, bias, residual, drop);
}

struct MhaShape {
    int64_t B, Sq, Sk, D, H, dk, dv;
};

static size_t mha_scratch_floats(const MhaShape &s)
{
    return (size_t)(s.B * s.Sq * s.H * s.dk + s.B * s.Sk * s.H * s.dk + s.B * s.Sk * s.H * s.dv + s.B * s.Sq * s.H * s.dv +
                    s.B * s.Sq * s.D);
}

static size_t mha_heads_scratch_floats(const MhaShape &s)
{
    return (size_t)(s.B * s.Sq * s.H * s.dk + s.B * s.Sk * s.H * s.dk + s.B * s.Sk * s.H * s.dv);
}

// First half of MultiHeadAttention.swift:97-127 for s.H heads (all of them, or the
// heads one GPU owns): projections without bias (:109-111) and attention (:117),
// result [B, Sq, H*dv] (the layout :119 views before the output projection).
// Projection outputs stay [B,S,H,d]; the attention kernels take strides, so the
// reference's permute copies (:113-115, :119) vanish.
static dl4s_status mha_heads(DeviceState *st, const float *xq, const float *xk, const float *xv, const MhaShape &s,
                             const float *wq, const float *wk, const float *wv, const MaskSpec &mask, float *heads_out,
                             int precision, float *ws, void *extra, size_t extra_bytes)
{
    ScopedGroup group(st, "MultiHeadAttention");
    float *qp = ws;
    float *kp = qp + s.B * s.Sq * s.H * s.dk;
    float *vp = kp + s.B * s.Sk * s.H * s.dk;
    const float inv_t = 1.0f / sqrtf((float)s.dk);
    DL4S_TRY(gemm(st, xq, wq, qp, s.B * s.Sq, s.H * s.dk, s.D, EPI_NONE, nullptr, nullptr, precision, extra, extra_bytes));
    DL4S_TRY(gemm(st, xk, wk, kp, s.B * s.Sk, s.H * s.dk, s.D, EPI_NONE, nullptr, nullptr, precision, extra, extra_bytes));
    DL4S_TRY(gemm(st, xv, wv, vp, s.B * s.Sk, s.H * s.dv, s.D, EPI_NONE, nullptr, nullptr, precision, extra, extra_bytes));
    return attention(st, qp, strides_bshd(s.H, s.Sq, s.dk), kp, strides_bshd(s.H, s.Sk, s.dk), vp,
                     strides_bshd(s.H, s.Sk, s.dv), heads_out, strides_bshd(s.H, s.Sq, s.dv), s.B, s.H, s.Sq, s.Sk, s.dk, s.dv,
                     inv_t, mask, precision, extra, extra_bytes);
}

// Second half (:121-124): heads [B*Sq, HDv] x Wo [HDv, D] + residual, then LayerNorm over
// [Sq, D] per batch element. `pr` holds B*Sq*D floats.
static dl4s_status mha_output(DeviceState *st, const float *heads, const float *residual, int64_t B, int64_t Sq, int64_t D,
                              int64_t HDv, const float *wo, const float *g, const float *sh, float *out, int precision,
                              float *pr, void *extra, size_t extra_bytes)
{
    const DropoutSpec drop = next_dropout(st);   // MultiHeadAttention.swift:122
    DL4S_TRY(gemm(st, heads, wo, pr, B * Sq, D, HDv, EPI_RESIDUAL, nullptr, residual, precision, extra, extra_bytes, &drop));
    return launch_layernorm(st, pr, nullptr, B, Sq, D, g, sh, out);
}

// MultiHeadAttention.swift:97-127. `ws` holds mha_scratch_floats floats followed by
// `extra_bytes` of kernel scratch.
static dl4s_status mha(DeviceState *st, const float *xq, const float *xk, const float *xv, const MhaShape &s, const float *wq,
                       const float *wk, const float *wv, const float *wo, const float *g, const float *sh, const MaskSpec &mask,
                       float *out, int precision, float *ws, void *extra, size_t extra_bytes)
{
    float *ao = ws + mha_heads_scratch_floats(s);
    float *pr = ao + s.B * s.Sq * s.H * s.dv;
    DL4S_TRY(mha_heads(st, xq, xk, xv, s, wq, wk, wv, mask, ao, precision, ws, extra, extra_bytes));
    return mha_output(st, ao, xq, s.B, s.Sq, s.D, s.H * s.dv, wo, g, sh, out, precision, pr, extra, extra_bytes);
}

static size_t ffn_scratch_floats(int64_t M, int64_t D, int64_t F) { return (size_t)(M * F + M * D); }

// PointwiseFeedForward.swift:67-82.
static dl4s_status ffn(DeviceState *st, const float *x, int64_t M, int64_t D, int64_t F, const float *w1, const float *b1,
                       const float *w2, const float *b2, const float *g, const float *sh, int act, float *out, int precision,
                       float *ws, void *extra, size_t extra_bytes)
{
    ScopedGroup group(st, "PointwiseFeedForward");
    float *hbuf = ws;
    float *obuf = hbuf + M * F;
    int epi1 = act == DL4S_ACT_RELU ? EPI_BIAS_RELU : EPI_BIAS_GELU;
    DL4S_TRY(gemm(st, x, w1, hbuf, M, F, D, epi1, b1, nullptr, precision, extra, extra_bytes));
    const DropoutSpec drop = next_dropout(st);   // PointwiseFeedForward.swift:78
    DL4S_TRY(gemm(st, hbuf, w2, obuf, M, D, F, EPI_BIAS_RESIDUAL, b2, x, precision, extra, extra_bytes, &drop));
    return launch_layernorm(st, obuf, nullptr, M, 1, D, g, sh, out);
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_gemm(const float *d_a, const float *d_b, float *d_c, int64_t M, int64_t N, int64_t K, float alpha,
                           float beta, int32_t trans_a, int32_t trans_b, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(M >= 0 && N >= 0 && K >= 0, "negative extent");
    DL4S_REQUIRE(M * N == 0 || (d_c && (K == 0 || (d_a && d_b))), "NULL buffer");
    ScopedTimer timer(st);
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    if (prec_tc(precision) && !trans_a && !trans_b && alpha == 1.0f && beta == 0.0f && gemm_tc_supported(M, N, K)) {
        size_t need = gemm_tc_scratch_bytes(M, N, K, prec_split(precision));
        void *scratch = nullptr;
        DL4S_TRY(arena_reserve(st, need, &scratch));
        return launch_gemm_tc(st, d_a, d_b, d_c, M, N, K, EPI_NONE, nullptr, nullptr, scratch, need, prec_split(precision));
    }
    if (prec_tc(precision) && alpha == 1.0f && beta == 0.0f && gemm_tc_trans_supported(M, N, K, trans_a, trans_b) &&
        (((uintptr_t)d_a | (uintptr_t)d_b | (uintptr_t)d_c) & 15) == 0) {
        // the products of a matmul's backward (dA = dC B^T, dB = A^T dC, Matrix.swift:139-173) on the tensor cores
        size_t need = gemm_tc_scratch_bytes(M, N, K, 0);
        void *scratch = nullptr;
        DL4S_TRY(arena_reserve(st, need, &scratch));
        return launch_gemm_tc_trans(st, d_a, d_b, d_c, M, N, K, trans_a, trans_b, scratch, need);
    }
    return launch_gemm_f32(st, d_a, d_b, d_c, M, N, K, alpha, beta, trans_a, trans_b, EPI_NONE, nullptr, nullptr);
}

dl4s_status dl4s_cuda_sdpa_forward(const float *d_q, const float *d_k, const float *d_v, int64_t B, int64_t H, int64_t Sq,
                                   int64_t Sk, int64_t dk, int64_t dv, float temperature, const int32_t *d_key_lengths,
                                   int32_t causal, const float *d_mask, const int64_t *mask_shape, float *d_out,
                                   int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_q && d_k && d_v && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 0 && H >= 0 && Sq >= 0 && Sk >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(temperature != 0.0f, "temperature must not be zero");
    DL4S_REQUIRE(!d_mask || mask_shape, "a dense mask needs its shape");
    DL4S_REQUIRE(!causal || Sq == Sk, "the causal mask of DL4S is square (TransformerUtil.swift:38-50): Sq must equal Sk");
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    MaskSpec mask = make_mask(d_key_lengths, causal, d_mask, mask_shape);
    DL4S_TRY(check_mask(mask, B, H, Sq, Sk));
    ScopedTimer timer(st);
    void *scratch = nullptr;
    size_t need = 0;
    if (prec_tc(precision)) {
        need = attn_prefill_tc_scratch_bytes(B, H, Sq, Sk, dk, dv);
        DL4S_TRY(arena_reserve(st, need, &scratch));
    }
    return attention(st, d_q, strides_bhsd(H, Sq, dk), d_k, strides_bhsd(H, Sk, dk), d_v, strides_bhsd(H, Sk, dv), d_out,
                     strides_bhsd(H, Sq, dv), B, H, Sq, Sk, dk, dv, 1.0f / temperature, mask, precision, scratch, need);
}

// Decode attention on q [B,H,1,dk] against caches [B,H,Lmax,d]; `scratch` holds the split-K records.
static size_t decode_scratch_bytes(int64_t B, int64_t H, int64_t Lmax, int64_t dv)
{
    return (size_t)(B * H * ceil_div(Lmax, 256) * (dv + 2)) * sizeof(float);
}

static dl4s_status decode_attention(DeviceState *st, const float *q, const float *k, const float *v, int64_t B, int64_t H,
                                    int64_t Lmax, int64_t dk, int64_t dv, float inv_t, const int32_t *lens, float *out,
                                    void *scratch)
{
    bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0;
    if (dk != dv || (dk != 64 && dk != 128) || !aligned || B > 65535 || H > 65535) {
        // Shapes outside the streaming kernel's layout go through the general fp32 kernel.
        MaskSpec mask = make_mask(lens, 0, nullptr, nullptr);
        return launch_attn_ref(st, q, strides_bhsd(H, 1, dk), k, strides_bhsd(H, Lmax, dk), v, strides_bhsd(H, Lmax, dv), out,
                               strides_bhsd(H, 1, dv), B, H, 1, Lmax, dk, dv, inv_t, mask);
    }
    return launch_attn_decode(st, q, k, v, B, H, Lmax, dk, dv, inv_t, lens, out, (float *)scratch, 256, ceil_div(Lmax, 256));
}

dl4s_status dl4s_cuda_sdpa_decode(const float *d_q, const float *d_k, const float *d_v, int64_t B, int64_t H, int64_t Lmax,
                                  int64_t dk, int64_t dv, float temperature, const int32_t *d_key_lengths, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_q && d_k && d_v && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 0 && H >= 0 && Lmax >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(temperature != 0.0f, "temperature must not be zero");
    if (B * H == 0) return DL4S_OK;
    ScopedTimer timer(st);
    const float inv_t = 1.0f / temperature;
    void *scratch = nullptr;
    DL4S_TRY(arena_reserve(st, decode_scratch_bytes(B, H, Lmax, dv), &scratch));
    return decode_attention(st, d_q, d_k, d_v, B, H, Lmax, dk, dv, inv_t, d_key_lengths, d_out, scratch);
}

dl4s_status dl4s_cuda_mha_decode_step(const float *d_x, int64_t B, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                      const float *d_wq, const float *d_wk, const float *d_wv, const float *d_wo,
                                      const float *d_ln_scale, const float *d_ln_shift, float *d_k_cache, float *d_v_cache,
                                      int64_t Lmax, const int32_t *d_lengths, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_wq && d_wk && d_wv && d_wo && d_ln_scale && d_ln_shift && d_k_cache && d_v_cache && d_lengths && d_out,
                 "NULL buffer");
    DL4S_REQUIRE(B >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && Lmax >= 1, "bad extents");
    DL4S_REQUIRE(B <= 65535 && H <= 65535, "B and H must each be at most 65535");
    // scratch: q, k, v of the token, head outputs, pre-norm rows, lengths + 1, split-K records
    const size_t nq = (size_t)(B * H * dk), nv = (size_t)(B * H * dv);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes, 256); return o; };
    const size_t o_q = take(nq * 4), o_k = take(nq * 4), o_v = take(nv * 4), o_heads = take(nv * 4), o_pr = take((size_t)(B * D) * 4);
    const size_t o_len = take((size_t)B * 4), o_rec = take(decode_scratch_bytes(B, H, Lmax, dv));
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, off, &base));
    char *w = (char *)base;
    float *q = (float *)(w + o_q), *k = (float *)(w + o_k), *v = (float *)(w + o_v), *heads = (float *)(w + o_heads);
    float *pr = (float *)(w + o_pr);
    int32_t *len1 = (int32_t *)(w + o_len);
    ScopedTimer timer(st);
    // projections without bias (MultiHeadAttention.swift:109-111), one row per sequence
    DL4S_TRY(launch_gemm_f32(st, d_x, d_wq, q, B, H * dk, D, 1.0f, 0.0f, 0, 0, EPI_NONE, nullptr, nullptr));
    DL4S_TRY(launch_gemm_f32(st, d_x, d_wk, k, B, H * dk, D, 1.0f, 0.0f, 0, 0, EPI_NONE, nullptr, nullptr));
    DL4S_TRY(launch_gemm_f32(st, d_x, d_wv, v, B, H * dv, D, 1.0f, 0.0f, 0, 0, EPI_NONE, nullptr, nullptr));
    k_kv_append<<<dim3((unsigned)H, (unsigned)B), 128, 0, st->stream>>>(k, v, H, dk, dv, Lmax, d_lengths, d_k_cache, d_v_cache, len1,
                                                                       st->status_word);
    DL4S_TRY(after_launch(st, "k_kv_append"));
    // attention of the one query row over the cached keys and itself (:117); [B,H,1,dv] is [B, H*dv] as it lies
    DL4S_TRY(decode_attention(st, q, d_k_cache, d_v_cache, B, H, Lmax, dk, dv, 1.0f / sqrtf((float)dk), len1, heads, w + o_rec));
    // output projection + residual, LayerNorm over the token's [1, D] block (:121-124)
    DL4S_TRY(launch_gemm_f32(st, heads, d_wo, pr, B, D, H * dv, 1.0f, 0.0f, 0, 0, EPI_RESIDUAL, nullptr, d_x));
    return launch_layernorm(st, pr, nullptr, B, 1, D, d_ln_scale, d_ln_shift, d_out);
}

dl4s_status dl4s_cuda_mha_forward(const float *d_xq, const float *d_xk, const float *d_xv, int64_t B, int64_t Sq, int64_t Sk,
                                  int64_t D, int64_t H, int64_t dk, int64_t dv, const float *d_wq, const float *d_wk,
                                  const float *d_wv, const float *d_wo, const float *d_ln_scale, const float *d_ln_shift,
                                  const int32_t *d_key_lengths, int32_t causal, const float *d_mask, const int64_t *mask_shape,
                                  float *d_out, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_xq && d_xk && d_xv && d_wq && d_wk && d_wv && d_wo && d_ln_scale && d_ln_shift && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && Sq >= 1 && Sk >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(!d_mask || mask_shape, "a dense mask needs its shape");
    DL4S_REQUIRE(!causal || Sq == Sk, "the causal mask of DL4S is square: Sq must equal Sk");
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    MaskSpec mask = make_mask(d_key_lengths, causal, d_mask, mask_shape);
    DL4S_TRY(check_mask(mask, B, H, Sq, Sk));
    MhaShape s{B, Sq, Sk, D, H, dk, dv};
    if (prec_tc(precision) && d_xq == d_xk && d_xk == d_xv && !d_mask && tc_block_supported(B, Sq, Sk, D, H, dk, dv, 0)) {
        // Self-attention: the fused tensor-core pipeline (one q/k/v product, half intermediates).
        ScopedTimer timer(st);
        return mha_self_tc(st, d_xq, B, Sq, D, H, dk, dv, d_wq, d_wk, d_wv, d_wo, d_ln_scale, d_ln_shift, mask, d_out,
                           prec_split(precision));
    }
    size_t main_bytes = align_up(mha_scratch_floats(s) * sizeof(float), 1024);
    size_t extra = prec_tc(precision) ? tc_layer_scratch_bytes(B, Sq > Sk ? Sq : Sk, D, H, dk, dv, 0, prec_split(precision)) : 0;
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, main_bytes + extra, &base));
    ScopedTimer timer(st);
    return mha(st, d_xq, d_xk, d_xv, s, d_wq, d_wk, d_wv, d_wo, d_ln_scale, d_ln_shift, mask, d_out, precision, (float *)base,
               (char *)base + main_bytes, extra);
}

}  // extern "C"

namespace dl4s {
// dl4s_cuda_mha_heads_forward with an optional half copy of the (self-attention) input that the caller already holds:
// the layer that spans GPUs rounds its whole replicated input once per call instead of once per batch chunk.
dl4s_status mha_heads_forward_impl(const float *d_xq, const float *d_xk, const float *d_xv, int64_t B, int64_t Sq, int64_t Sk,
                                   int64_t D, int64_t Hl, int64_t dk, int64_t dv, const float *d_wq, const float *d_wk,
                                   const float *d_wv, const int32_t *d_key_lengths, int32_t causal, void *d_heads_out,
                                   int32_t precision, int32_t half_output, const void *d_x_half)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_xq && d_xk && d_xv && d_wq && d_wk && d_wv && d_heads_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && Sq >= 1 && Sk >= 1 && D >= 1 && Hl >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(!causal || Sq == Sk, "the causal mask of DL4S is square: Sq must equal Sk");
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    MaskSpec mask = make_mask(d_key_lengths, causal, nullptr, nullptr);
    const bool fused_tc = prec_tc(precision) && d_xq == d_xk && d_xk == d_xv && tc_block_supported(B, Sq, Sk, D, Hl, dk, dv, 0);
    if (fused_tc) {
        ScopedTimer timer(st);
        return mha_heads_self_tc(st, d_xq, B, Sq, D, Hl, dk, dv, d_wq, d_wk, d_wv, mask, d_heads_out, half_output != 0,
                                 prec_split(precision), d_x_half);
    }
    if (half_output)
        return fail(DL4S_ERR_UNSUPPORTED, "half output needs the fused tensor-core path (see dl4s_cuda_mha_heads_half_supported)");
    MhaShape s{B, Sq, Sk, D, Hl, dk, dv};
    size_t main_bytes = align_up(mha_heads_scratch_floats(s) * sizeof(float), 1024);
    size_t extra = prec_tc(precision) ? tc_layer_scratch_bytes(B, Sq > Sk ? Sq : Sk, D, Hl, dk, dv, 0, prec_split(precision)) : 0;
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, main_bytes + extra, &base));
    ScopedTimer timer(st);
    return mha_heads(st, d_xq, d_xk, d_xv, s, d_wq, d_wk, d_wv, mask, (float *)d_heads_out, precision, (float *)base,
                     (char *)base + main_bytes, extra);
}

}  // namespace dl4s

extern "C" {

dl4s_status dl4s_cuda_mha_heads_forward(const float *d_xq, const float *d_xk, const float *d_xv, int64_t B, int64_t Sq,
                                        int64_t Sk, int64_t D, int64_t Hl, int64_t dk, int64_t dv, const float *d_wq,
                                        const float *d_wk, const float *d_wv, const int32_t *d_key_lengths, int32_t causal,
                                        void *d_heads_out, int32_t precision, int32_t half_output)
{
    return mha_heads_forward_impl(d_xq, d_xk, d_xv, B, Sq, Sk, D, Hl, dk, dv, d_wq, d_wk, d_wv, d_key_lengths, causal, d_heads_out,
                                  precision, half_output, nullptr);
}

dl4s_status dl4s_cuda_mha_heads_half_supported(int64_t B, int64_t S, int64_t D, int64_t Hl, int64_t dk, int64_t dv, int64_t HDv,
                                               int32_t *supported)
{
    DL4S_REQUIRE(supported, "supported is NULL");
    *supported = tc_block_supported(B, S, S, D, Hl, dk, dv, 0) && gemm_tc_supported(B * S, D, HDv) && D % 4 == 0;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_mha_output_forward(const void *d_heads, const float *d_residual, int64_t B, int64_t Sq, int64_t D,
                                         int64_t HDv, const float *d_wo, const float *d_ln_scale, const float *d_ln_shift,
                                         float *d_out, int32_t precision, int32_t half_input, int64_t groups,
                                         int64_t group_stride)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_heads && d_residual && d_wo && d_ln_scale && d_ln_shift && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && Sq >= 1 && D >= 1 && HDv >= 1, "bad extents");
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    DL4S_REQUIRE(groups >= 1 && HDv % groups == 0, "%lld column groups do not divide %lld head columns", (long long)groups,
                 (long long)HDv);
    const int64_t C = HDv / groups, M = B * Sq;
    if (groups == 1) group_stride = M * C;
    DL4S_REQUIRE(group_stride >= M * C, "group stride %lld is smaller than one group (%lld elements)", (long long)group_stride,
                 (long long)(M * C));
    if (prec_tc(precision) && gemm_tc_supported(M, D, HDv) && D % 4 == 0 && C % 64 == 0 && group_stride % 8 == 0) {
        ScopedTimer timer(st);
        return mha_output_tc(st, d_heads, half_input != 0, d_residual, B, Sq, D, HDv, d_wo, d_ln_scale, d_ln_shift, d_out,
                             groups, group_stride, prec_split(precision));
    }
    if (half_input)
        return fail(DL4S_ERR_UNSUPPORTED, "half input needs the tensor-core path (see dl4s_cuda_mha_heads_half_supported)");
    size_t main_bytes = align_up((size_t)(M * D) * sizeof(float), 1024);
    size_t rows_bytes = groups > 1 ? align_up((size_t)(M * HDv) * sizeof(float), 1024) : 0;
    size_t extra = prec_tc(precision) && gemm_tc_supported(M, D, HDv) ? gemm_tc_scratch_bytes(M, D, HDv, prec_split(precision)) : 0;
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, main_bytes + rows_bytes + extra, &base));
    ScopedTimer timer(st);
    const float *heads = (const float *)d_heads;
    if (groups > 1) {
        // rows[m, g, c] = heads[g * group_stride + m * C + c]
        float *rows = (float *)((char *)base + main_bytes);
        const int64_t src_strides[3] = {C, group_stride, 1}, dst_strides[3] = {HDv, C, 1}, extent[3] = {M, groups, C};
        DL4S_TRY(dl4s_cuda_copy_strided_f32(heads, src_strides, 0, rows, dst_strides, 0, extent, 3));
        heads = rows;
    }
    return mha_output(st, heads, d_residual, B, Sq, D, HDv, d_wo, d_ln_scale, d_ln_shift, d_out, precision, (float *)base,
                      (char *)base + main_bytes + rows_bytes, extra);
}

dl4s_status dl4s_cuda_ffn_forward(const float *d_x, int64_t M, int64_t D, int64_t F, const float *d_w1, const float *d_b1,
                                  const float *d_w2, const float *d_b2, const float *d_ln_scale, const float *d_ln_shift,
                                  int32_t act, float *d_out, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_w1 && d_b1 && d_w2 && d_b2 && d_ln_scale && d_ln_shift && d_out, "NULL buffer");
    DL4S_REQUIRE(M >= 1 && D >= 1 && F >= 1, "bad extents");
    DL4S_REQUIRE(act == DL4S_ACT_GELU_SIGMOID || act == DL4S_ACT_RELU, "unknown activation %d", act);
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    if (prec_tc(precision) && gemm_tc_supported(M, F, D) && gemm_tc_supported(M, D, F) && D % 4 == 0) {
        ScopedTimer timer(st);
        return ffn_tc(st, d_x, M, D, F, d_w1, d_b1, d_w2, d_b2, d_ln_scale, d_ln_shift, act, d_out, prec_split(precision));
    }
    size_t main_bytes = align_up(ffn_scratch_floats(M, D, F) * sizeof(float), 1024);
    size_t extra = prec_tc(precision) ? tc_layer_scratch_bytes(1, M, D, 1, 1, 1, F, prec_split(precision)) : 0;
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, main_bytes + extra, &base));
    ScopedTimer timer(st);
    return ffn(st, d_x, M, D, F, d_w1, d_b1, d_w2, d_b2, d_ln_scale, d_ln_shift, act, d_out, precision, (float *)base,
               (char *)base + main_bytes, extra);
}

dl4s_status dl4s_cuda_encoder_forward(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                      int64_t F, int64_t layers, const float *d_params, const int32_t *d_lengths, int32_t act,
                                      float *d_out, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_params && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && S >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && F >= 1 && layers >= 0, "bad extents");
    DL4S_REQUIRE(act == DL4S_ACT_GELU_SIGMOID || act == DL4S_ACT_RELU, "unknown activation %d", act);
    DL4S_REQUIRE(prec_known(precision), "unknown precision %d", precision);
    if (prec_tc(precision) && layers > 0 && tc_block_supported(B, S, S, D, H, dk, dv, F)) {
        ScopedTimer timer(st);
        return encoder_tc(st, d_x, B, S, D, H, dk, dv, F, layers, d_params, make_mask(d_lengths, 0, nullptr, nullptr), act, d_out,
                          prec_split(precision));
    }
    MhaShape s{B, S, S, D, H, dk, dv};
    size_t mf = mha_scratch_floats(s), ff = ffn_scratch_floats(B * S, D, F);
    size_t main_floats = (mf > ff ? mf : ff) + 2 * (size_t)(B * S * D);
    size_t main_bytes = align_up(main_floats * sizeof(float), 1024);
    size_t extra = prec_tc(precision) ? tc_layer_scratch_bytes(B, S, D, H, dk, dv, F, prec_split(precision)) : 0;
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, main_bytes + extra, &base));
    ScopedTimer timer(st);
    float *ping = (float *)base;
    float *pong = ping + B * S * D;
    float *ws = pong + B * S * D;
    void *ex = (char *)base + main_bytes;
    MaskSpec mask = make_mask(d_lengths, 0, nullptr, nullptr);
    if (layers == 0) {
        DL4S_CUDA_TRY(cudaMemcpyAsync(d_out, d_x, sizeof(float) * (size_t)(B * S * D), cudaMemcpyDeviceToDevice, st->stream));
        return DL4S_OK;
    }
    const float *cur = d_x;
    const float *p = d_params;
    ScopedGroup group(st, "Encoder");
    for (int64_t l = 0; l < layers; ++l) {
        ScopedGroup layer(st, "EncoderLayer");
        const float *wq = p; p += D * H * dk;
        const float *wk = p; p += D * H * dk;
        const float *wv = p; p += D * H * dv;
        const float *wo = p; p += H * dv * D;
        const float *g1 = p; p += D;
        const float *s1 = p; p += D;
        const float *w1 = p; p += D * F;
        const float *b1 = p; p += F;
        const float *w2 = p; p += F * D;
        const float *b2 = p; p += D;
        const float *g2 = p; p += D;
        const float *s2 = p; p += D;
        DL4S_TRY(mha(st, cur, cur, cur, s, wq, wk, wv, wo, g1, s1, mask, ping, precision, ws, ex, extra));
        float *dst = (l == layers - 1) ? d_out : pong;
        DL4S_TRY(ffn(st, ping, B * S, D, F, w1, b1, w2, b2, g2, s2, act, dst, precision, ws, ex, extra));
        cur = dst;
    }
    return DL4S_OK;
}

dl4s_status dl4s_cuda_encoder_prepare(int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int64_t layers,
                                      const float *d_params, int32_t precision, void **prepared)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_params && prepared, "NULL argument");
    *prepared = nullptr;
    DL4S_REQUIRE(D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && F >= 1 && layers >= 1, "bad extents");
    DL4S_REQUIRE(prec_tc(precision), "weights are prepared for the tensor-core precisions only (got %d)", precision);
    return encoder_prepare(st, D, H, dk, dv, F, layers, d_params, prec_split(precision), prepared);
}

dl4s_status dl4s_cuda_encoder_prepared_refresh(void *prepared)
{
    DL4S_STATE(st);
    return encoder_prepared_refresh(st, prepared);
}

dl4s_status dl4s_cuda_encoder_prepared_destroy(void *prepared)
{
    DL4S_STATE(st);
    return encoder_prepared_destroy(st, prepared);
}

dl4s_status dl4s_cuda_encoder_forward_prepared(void *prepared, const float *d_x, int64_t B, int64_t S, const int32_t *d_lengths,
                                               int32_t act, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(prepared && d_x && d_out, "NULL argument");
    DL4S_REQUIRE(B >= 1 && S >= 1, "bad extents");
    DL4S_REQUIRE(act == DL4S_ACT_GELU_SIGMOID || act == DL4S_ACT_RELU, "unknown activation %d", act);
    ScopedTimer timer(st);
    return encoder_tc_prepared(st, prepared, d_x, B, S, make_mask(d_lengths, 0, nullptr, nullptr), act, d_out);
}

dl4s_status dl4s_cuda_embed_positional(const int32_t *d_ids, int64_t B, int64_t S, int64_t D, const float *d_embedding,
                                       int64_t vocab, int32_t ignore_index, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_ids && d_embedding && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 0 && S >= 0 && D >= 2 && D % 2 == 0 && vocab >= 1, "bad extents (D must be even)");
    if (B * S == 0) return DL4S_OK;
    DL4S_REQUIRE((((uintptr_t)d_embedding | (uintptr_t)d_out) & 7) == 0, "embedding and output must be 8-byte aligned");
    DL4S_TRY(ensure_positional_table(st, S, D));
    ScopedGroup group(st, "Embedding");
    int64_t blocks = B * S < (int64_t)st->sm_count * 16 ? B * S : (int64_t)st->sm_count * 16;
    k_embed_positional<<<(unsigned)blocks, 256, 0, st->stream>>>(d_ids, B * S, S, D, d_embedding, vocab, ignore_index,
                                                                sqrtf((float)D), st->pe_table, d_out, next_dropout(st));
    return after_launch(st, "k_embed_positional");
}

}  // extern "C"
