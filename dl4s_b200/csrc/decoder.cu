// The decoder side of the Transformer: TransformerDecoderBlock / TransformerDecoder
// (NN/Models/Transformer/TransformerDecoderBlock.swift:61-68, TransformerDecoder.swift:49-62) over whole
// sequences, incremental decoding with key/value caches (the caller of the decode attention kernel), and the
// greedy loop of Transformer.callAsFunction(inputSequence:startToken:endToken:maxLength:)
// (Transformer.swift:118-137).
//
// Parameter block of one decoder layer, in this order (the order of TransformerDecoderBlock.parameters):
//   self-attention     Wq, Wk [D,H*dk], Wv [D,H*dv], Wo [H*dv,D], ln_scale, ln_shift [D]
//   encoder attention  the same six
//   feed-forward       W1 [D,F], b1 [F], W2 [F,D], b2 [D], ln_scale, ln_shift [D]
//
// A note on what a key/value cache can and cannot reproduce. The reference re-runs the whole decoder on the
// growing prefix for every generated token, and its LayerNorm inside MultiHeadAttention normalises the whole
// [prefix, D] block at once (LayerNorm.swift:62-77 reduces over every axis but the first). The statistics
// therefore change with every token and move ALL earlier rows, so no cache of earlier keys and values is exactly
// what the reference would recompute. Greedy decoding exists in both forms here: `cached = 0` follows the
// reference's schedule to the letter (decoder re-run on the prefix, the same kernels as the forward pass);
// `cached = 1` appends one token per step to per-layer caches and normalises each token's own [1, D] block,
// which is the serving formulation and costs one token of work per step.
#include "common.cuh"

#include <cmath>

namespace dl4s {

// x[b,:] = E[ids[b]] * sqrt(D) + PE[pos,:] for one position of every sequence (Transformer.swift:82-88 for the
// token a decoding step feeds back). `ids` lives on the device: the greedy loop never returns to the host.
__global__ void __launch_bounds__(256) k_embed_at(const int32_t *__restrict__ ids, int64_t ids_stride, int64_t D,
                                                  const float *__restrict__ E, int64_t vocab, int32_t ignore_index, float scale,
                                                  const float *__restrict__ pe_row, float *__restrict__ out)
{
    const int64_t b = blockIdx.x;
    const int32_t id = ids[b * ids_stride];
    const bool zero = (id == ignore_index) || id < 0 || id >= vocab;
    for (int64_t i = threadIdx.x; i < D; i += blockDim.x)
        out[b * D + i] = (zero ? 0.f : E[(int64_t)id * D + i] * scale) + pe_row[i];
}

// lengths[b] += 1 (capped at the cache size).
__global__ void k_advance_lengths(int32_t *lengths, int64_t B, int32_t cap)
{
    const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B && lengths[b] < cap) lengths[b] += 1;
}

struct DecLayerP {
    const float *swq, *swk, *swv, *swo, *sg, *ss;   // self-attention
    const float *ewq, *ewk, *ewv, *ewo, *eg, *es;   // encoder attention
    const float *w1, *b1, *w2, *b2, *fg, *fs;       // feed-forward
};

static int64_t dec_layer_floats(int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F)
{
    const int64_t mha = 2 * D * H * dk + D * H * dv + H * dv * D + 2 * D;
    return 2 * mha + D * F + F + F * D + D + 2 * D;
}

static DecLayerP dec_layer_pointers(const float *p, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F)
{
    DecLayerP l;
    const int64_t Nq = H * dk, Nv = H * dv;
    l.swq = p; p += D * Nq; l.swk = p; p += D * Nq; l.swv = p; p += D * Nv; l.swo = p; p += Nv * D; l.sg = p; p += D; l.ss = p; p += D;
    l.ewq = p; p += D * Nq; l.ewk = p; p += D * Nq; l.ewv = p; p += D * Nv; l.ewo = p; p += Nv * D; l.eg = p; p += D; l.es = p; p += D;
    l.w1 = p; p += D * F; l.b1 = p; p += F; l.w2 = p; p += F * D; l.b2 = p; p += D; l.fg = p; p += D; l.fs = p; p += D;
    return l;
}

constexpr int kMaxDecLayers = 64;

// Incremental decoding state of a decoder stack for B sequences.
struct DecoderCache {
    uint32_t magic = 0x44454343;   // "DECC"
    int device = -1;
    int64_t B = 0, Lmax = 0, Ss = 0, D = 0, H = 0, dk = 0, dv = 0, F = 0, layers = 0;
    const float *params = nullptr;
    char *block = nullptr;          // everything below lives in one allocation
    float *self_k[kMaxDecLayers], *self_v[kMaxDecLayers];   // [B,H,Lmax,d]
    float *enc_k[kMaxDecLayers], *enc_v[kMaxDecLayers];     // [B,H,Ss,d]
    int32_t *lengths = nullptr;      // [B] tokens cached so far (the same for every layer)
    int32_t *enc_lengths = nullptr;  // [B]
    float *tmp[3] = {nullptr, nullptr, nullptr};            // [B,D] rows between the sublayers
    float *q = nullptr, *heads = nullptr, *pr = nullptr;    // cross-attention scratch [B,H*dk], [B,H*dv], [B,D]
    bool encoder_set = false;
};

static DecoderCache *as_cache(DeviceState *st, void *h)
{
    DecoderCache *c = static_cast<DecoderCache *>(h);
    if (!c || c->magic != 0x44454343) {
        fail(DL4S_ERR_INVALID_ARG, "not a handle of dl4s_cuda_decoder_cache_create");
        return nullptr;
    }
    if (c->device != st->ordinal) {
        fail(DL4S_ERR_INVALID_ARG, "the cache lives on device %d, the current device is %d", c->device, st->ordinal);
        return nullptr;
    }
    return c;
}

}  // namespace dl4s

using namespace dl4s;

extern "C" {

dl4s_status dl4s_cuda_decoder_forward(const float *d_x, const float *d_enc, int64_t B, int64_t St, int64_t Ss, int64_t D, int64_t H,
                                      int64_t dk, int64_t dv, int64_t F, int64_t layers, const float *d_params,
                                      const int32_t *d_dec_lengths, const int32_t *d_enc_lengths, int32_t act, float *d_out,
                                      int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_enc && d_params && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && St >= 1 && Ss >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && F >= 1 && layers >= 0, "bad extents");
    DL4S_REQUIRE(!st->capturing, "the decoder forward allocates its intermediate rows and cannot be recorded into a graph");
    const size_t bytes = (size_t)(B * St * D) * sizeof(float);
    if (layers == 0) {
        DL4S_CUDA_TRY(cudaMemcpyAsync(d_out, d_x, bytes, cudaMemcpyDeviceToDevice, st->stream));
        return DL4S_OK;
    }
    // three rows of [B,St,D] between the sublayers (the fused calls lay the scratch arena out themselves). A layer
    // reads its input only in the self-attention call, so the feed-forward may write the next input over it.
    float *buf = nullptr;
    DL4S_CUDA_TRY(cudaMallocAsync((void **)&buf, 3 * bytes, st->stream));
    float *y = buf, *z = buf + B * St * D, *nx = buf + 2 * B * St * D;
    ScopedGroup group(st, "Decoder");
    dl4s_status s = DL4S_OK;
    const float *cur = d_x;
    const int64_t per_layer = dec_layer_floats(D, H, dk, dv, F);
    for (int64_t l = 0; l < layers && s == DL4S_OK; ++l) {
        ScopedGroup layer(st, "DecoderLayer");
        const DecLayerP p = dec_layer_pointers(d_params + l * per_layer, D, H, dk, dv, F);
        // decAttn = selfAttention(q: x, k: x, v: x, mask: decoderMask)      (causal OR padding, TransformerUtil.swift:38-50)
        s = dl4s_cuda_mha_forward(cur, cur, cur, B, St, St, D, H, dk, dv, p.swq, p.swk, p.swv, p.swo, p.sg, p.ss, d_dec_lengths, 1,
                                  nullptr, nullptr, y, precision);
        if (s != DL4S_OK) break;
        // encAttn = encoderAttention(q: decAttn, k: encoderOutput, v: encoderOutput, mask: encoderMask)
        s = dl4s_cuda_mha_forward(y, d_enc, d_enc, B, St, Ss, D, H, dk, dv, p.ewq, p.ewk, p.ewv, p.ewo, p.eg, p.es, d_enc_lengths, 0,
                                  nullptr, nullptr, z, precision);
        if (s != DL4S_OK) break;
        float *dst = (l == layers - 1) ? d_out : nx;
        s = dl4s_cuda_ffn_forward(z, B * St, D, F, p.w1, p.b1, p.w2, p.b2, p.fg, p.fs, act, dst, precision);
        cur = dst;
    }
    cudaFreeAsync(buf, st->stream);
    return s;
}

dl4s_status dl4s_cuda_mha_kv_project(const float *d_x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                     const float *d_wk, const float *d_wv, float *d_k_cache, float *d_v_cache, int64_t Lmax)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_x && d_wk && d_wv && d_k_cache && d_v_cache, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && S >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && Lmax >= S, "bad extents (Lmax must hold the S rows)");
    DL4S_REQUIRE(!st->capturing, "the projection allocates a staging buffer and cannot be recorded into a graph");
    const int64_t dmax = dk > dv ? dk : dv;
    float *proj = nullptr;
    DL4S_CUDA_TRY(cudaMallocAsync((void **)&proj, (size_t)(B * S * H * dmax) * sizeof(float), st->stream));
    dl4s_status s = DL4S_OK;
    for (int which = 0; which < 2 && s == DL4S_OK; ++which) {
        const int64_t d = which ? dv : dk;
        s = launch_gemm_f32(st, d_x, which ? d_wv : d_wk, proj, B * S, H * d, D, 1.0f, 0.0f, 0, 0, EPI_NONE, nullptr, nullptr);
        if (s != DL4S_OK) break;
        // [B, S, H, d] -> [B, H, Lmax, d]
        const int64_t src[4] = {S * H * d, d, H * d, 1}, dst[4] = {H * Lmax * d, Lmax * d, d, 1}, ext[4] = {B, H, S, d};
        s = dl4s_cuda_copy_strided_f32(proj, src, 0, which ? d_v_cache : d_k_cache, dst, 0, ext, 4);
    }
    cudaFreeAsync(proj, st->stream);
    return s;
}

dl4s_status dl4s_cuda_decoder_cache_create(int64_t B, int64_t Lmax, int64_t Ss, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F,
                                           int64_t layers, const float *d_params, void **cache)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(cache && d_params, "NULL argument");
    *cache = nullptr;
    DL4S_REQUIRE(B >= 1 && Lmax >= 1 && Ss >= 1 && D >= 1 && H >= 1 && dk >= 1 && dv >= 1 && F >= 1, "bad extents");
    DL4S_REQUIRE(layers >= 1 && layers <= kMaxDecLayers, "between 1 and %d layers", kMaxDecLayers);
    DL4S_REQUIRE(B <= 65535 && H <= 65535, "B and H must each be at most 65535");
    DL4S_REQUIRE(!st->capturing, "create the cache before dl4s_cuda_graph_begin");
    DecoderCache *c = new DecoderCache();
    c->device = st->ordinal;
    c->B = B; c->Lmax = Lmax; c->Ss = Ss; c->D = D; c->H = H; c->dk = dk; c->dv = dv; c->F = F; c->layers = layers;
    c->params = d_params;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes, 256); return o; };
    size_t o_sk[kMaxDecLayers], o_sv[kMaxDecLayers], o_ek[kMaxDecLayers], o_ev[kMaxDecLayers];
    for (int64_t l = 0; l < layers; ++l) {
        o_sk[l] = take((size_t)(B * H * Lmax * dk) * 4);
        o_sv[l] = take((size_t)(B * H * Lmax * dv) * 4);
        o_ek[l] = take((size_t)(B * H * Ss * dk) * 4);
        o_ev[l] = take((size_t)(B * H * Ss * dv) * 4);
    }
    const size_t o_len = take((size_t)B * 4), o_elen = take((size_t)B * 4);
    const size_t o_t0 = take((size_t)(B * D) * 4), o_t1 = take((size_t)(B * D) * 4), o_t2 = take((size_t)(B * D) * 4);
    const size_t o_q = take((size_t)(B * H * dk) * 4), o_h = take((size_t)(B * H * dv) * 4), o_pr = take((size_t)(B * D) * 4);
    cudaError_t e = cudaMalloc((void **)&c->block, off);
    if (e != cudaSuccess) {
        delete c;
        return check_cuda(e, "cudaMalloc(decoder cache)");
    }
    for (int64_t l = 0; l < layers; ++l) {
        c->self_k[l] = (float *)(c->block + o_sk[l]); c->self_v[l] = (float *)(c->block + o_sv[l]);
        c->enc_k[l] = (float *)(c->block + o_ek[l]); c->enc_v[l] = (float *)(c->block + o_ev[l]);
    }
    c->lengths = (int32_t *)(c->block + o_len);
    c->enc_lengths = (int32_t *)(c->block + o_elen);
    c->tmp[0] = (float *)(c->block + o_t0); c->tmp[1] = (float *)(c->block + o_t1); c->tmp[2] = (float *)(c->block + o_t2);
    c->q = (float *)(c->block + o_q); c->heads = (float *)(c->block + o_h); c->pr = (float *)(c->block + o_pr);
    DL4S_CUDA_TRY(cudaMemsetAsync(c->lengths, 0, (size_t)B * 4, st->stream));
    *cache = c;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_decoder_cache_set_encoder(void *cache, const float *d_enc, const int32_t *d_enc_lengths)
{
    DL4S_STATE(st);
    DecoderCache *c = as_cache(st, cache);
    if (!c) return DL4S_ERR_INVALID_ARG;
    DL4S_REQUIRE(d_enc, "NULL buffer");
    // encoder keys and values of every layer, projected once: they do not change while the sequence is decoded
    const int64_t per_layer = dec_layer_floats(c->D, c->H, c->dk, c->dv, c->F);
    for (int64_t l = 0; l < c->layers; ++l) {
        const DecLayerP p = dec_layer_pointers(c->params + l * per_layer, c->D, c->H, c->dk, c->dv, c->F);
        DL4S_TRY(dl4s_cuda_mha_kv_project(d_enc, c->B, c->Ss, c->D, c->H, c->dk, c->dv, p.ewk, p.ewv, c->enc_k[l], c->enc_v[l], c->Ss));
    }
    if (d_enc_lengths)
        DL4S_CUDA_TRY(cudaMemcpyAsync(c->enc_lengths, d_enc_lengths, (size_t)c->B * 4, cudaMemcpyDeviceToDevice, st->stream));
    else
        DL4S_TRY(dl4s_cuda_fill_i32((int32_t)c->Ss, c->enc_lengths, c->B));
    DL4S_CUDA_TRY(cudaMemsetAsync(c->lengths, 0, (size_t)c->B * 4, st->stream));
    c->encoder_set = true;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_decoder_cache_lengths(void *cache, int32_t **d_lengths)
{
    DL4S_STATE(st);
    DecoderCache *c = as_cache(st, cache);
    if (!c) return DL4S_ERR_INVALID_ARG;
    DL4S_REQUIRE(d_lengths, "NULL argument");
    *d_lengths = c->lengths;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_decoder_step(void *cache, const float *d_x, int32_t act, float *d_out)
{
    DL4S_STATE(st);
    DecoderCache *c = as_cache(st, cache);
    if (!c) return DL4S_ERR_INVALID_ARG;
    DL4S_REQUIRE(d_x && d_out, "NULL buffer");
    DL4S_REQUIRE(c->encoder_set, "call dl4s_cuda_decoder_cache_set_encoder first");
    DL4S_REQUIRE(act == DL4S_ACT_GELU_SIGMOID || act == DL4S_ACT_RELU, "unknown activation %d", act);
    const int64_t B = c->B, D = c->D, H = c->H, dk = c->dk, dv = c->dv, F = c->F;
    const int64_t per_layer = dec_layer_floats(D, H, dk, dv, F);
    ScopedGroup group(st, "Decoder");
    const float *cur = d_x;
    for (int64_t l = 0; l < c->layers; ++l) {
        ScopedGroup layer(st, "DecoderLayer");
        const DecLayerP p = dec_layer_pointers(c->params + l * per_layer, D, H, dk, dv, F);
        float *y = c->tmp[0], *z = c->tmp[1];
        float *dst = (l == c->layers - 1) ? d_out : c->tmp[2];
        // self-attention over the cached prefix and the token itself (TransformerDecoderBlock.swift:64)
        DL4S_TRY(dl4s_cuda_mha_decode_step(cur, B, D, H, dk, dv, p.swq, p.swk, p.swv, p.swo, p.sg, p.ss, c->self_k[l], c->self_v[l],
                                           c->Lmax, c->lengths, y));
        // encoder attention: the token's query against the encoder keys/values projected once (:65)
        {
            ScopedGroup mha(st, "MultiHeadAttention");
            DL4S_TRY(launch_gemm_f32(st, y, p.ewq, c->q, B, H * dk, D, 1.0f, 0.0f, 0, 0, EPI_NONE, nullptr, nullptr));
            DL4S_TRY(dl4s_cuda_sdpa_decode(c->q, c->enc_k[l], c->enc_v[l], B, H, c->Ss, dk, dv, sqrtf((float)dk), c->enc_lengths, c->heads));
            DL4S_TRY(launch_gemm_f32(st, c->heads, p.ewo, c->pr, B, D, H * dv, 1.0f, 0.0f, 0, 0, EPI_RESIDUAL, nullptr, y));
            DL4S_TRY(launch_layernorm(st, c->pr, nullptr, B, 1, D, p.eg, p.es, z));
        }
        // feed-forward on the token's row (:66)
        DL4S_TRY(dl4s_cuda_ffn_forward(z, B, D, F, p.w1, p.b1, p.w2, p.b2, p.fg, p.fs, act, dst, DL4S_PREC_FP32));
        cur = dst;   // read by the next layer's self-attention step only, before its feed-forward writes tmp[2] again
    }
    k_advance_lengths<<<(unsigned)ceil_div(B, 128), 128, 0, st->stream>>>(c->lengths, B, (int32_t)c->Lmax);
    return after_launch(st, "k_advance_lengths");
}

dl4s_status dl4s_cuda_decoder_cache_destroy(void *cache)
{
    DL4S_STATE(st);
    if (!cache) return DL4S_OK;
    DecoderCache *c = as_cache(st, cache);
    if (!c) return DL4S_ERR_INVALID_ARG;
    DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
    DL4S_TRY(release_internal(st, c->block));
    c->magic = 0;
    delete c;
    return DL4S_OK;
}

dl4s_status dl4s_cuda_embed_at(const int32_t *d_ids, int64_t ids_stride, int64_t B, int64_t position, int64_t D,
                               const float *d_embedding, int64_t vocab, int32_t ignore_index, float *d_out)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_ids && d_embedding && d_out, "NULL buffer");
    DL4S_REQUIRE(B >= 1 && position >= 0 && D >= 2 && D % 2 == 0 && vocab >= 1 && B <= 65535, "bad extents (D must be even)");
    // the positional table is the one dl4s_cuda_embed_positional keeps; make it cover `position`
    if (st->pe_dim != D || st->pe_rows <= position) {
        int64_t rows = 64;
        while (rows <= position) rows *= 2;
        DL4S_TRY(ensure_positional_table(st, rows, D));
    }
    k_embed_at<<<(unsigned)B, 256, 0, st->stream>>>(d_ids, ids_stride, D, d_embedding, vocab, ignore_index, sqrtf((float)D),
                                                    st->pe_table + position * D, d_out);
    return after_launch(st, "k_embed_at");
}

dl4s_status dl4s_cuda_transformer_greedy_decode(const int32_t *input_ids, int64_t n_in, int32_t start_token, int32_t end_token,
                                                int64_t max_length, int64_t vocab, int64_t D, int64_t H, int64_t dk, int64_t dv,
                                                int64_t F, int64_t enc_layers, int64_t dec_layers, const float *d_embedding,
                                                const float *d_enc_params, const float *d_dec_params, int32_t act, int32_t precision,
                                                int32_t cached, int32_t *tokens, int64_t *n_tokens)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(input_ids && d_embedding && d_enc_params && d_dec_params && tokens && n_tokens, "NULL argument");
    DL4S_REQUIRE(n_in >= 1 && max_length >= 1 && vocab >= 1 && dec_layers >= 1 && enc_layers >= 0, "bad extents");
    DL4S_REQUIRE(!st->capturing, "the greedy loop reads tokens back and cannot be recorded into a graph");
    *n_tokens = 0;
    const int64_t L = max_length;
    // device buffers: input ids, the token row [start, t1, t2, ...], encoder input / states, decoder rows, logits
    char *block = nullptr;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes, 256); return o; };
    const size_t o_ids = take((size_t)n_in * 4), o_tok = take((size_t)(L + 1) * 4), o_len = take(16), o_elen = take(16);
    const size_t o_ex = take((size_t)(n_in * D) * 4), o_enc = take((size_t)(n_in * D) * 4);
    const size_t o_dx = take((size_t)(L * D) * 4), o_dy = take((size_t)(L * D) * 4);
    const size_t o_logits = take((size_t)vocab * 4), o_max = take(16);
    DL4S_CUDA_TRY(cudaMalloc((void **)&block, off));
    int32_t *d_ids = (int32_t *)(block + o_ids), *d_tok = (int32_t *)(block + o_tok);
    int32_t *d_len = (int32_t *)(block + o_len), *d_elen = (int32_t *)(block + o_elen);
    float *ex = (float *)(block + o_ex), *enc = (float *)(block + o_enc), *dx = (float *)(block + o_dx), *dy = (float *)(block + o_dy);
    float *logits = (float *)(block + o_logits), *mx = (float *)(block + o_max);
    void *cache = nullptr;
    dl4s_status s = DL4S_OK;
    auto run = [&]() -> dl4s_status {
        DL4S_TRY(ensure_positional_table(st, L > n_in ? L : n_in, D));
        DL4S_CUDA_TRY(cudaMemcpyAsync(d_ids, input_ids, (size_t)n_in * 4, cudaMemcpyHostToDevice, st->stream));
        DL4S_TRY(dl4s_cuda_fill_i32(start_token, d_tok, 1));
        DL4S_TRY(dl4s_cuda_fill_i32((int32_t)n_in, d_elen, 1));
        // encIn = prepareInputs(input); encoded = encoder(encIn, [n_in])            (Transformer.swift:119-120)
        DL4S_TRY(dl4s_cuda_embed_positional(d_ids, 1, n_in, D, d_embedding, vocab, -1, ex));
        DL4S_TRY(dl4s_cuda_encoder_forward(ex, 1, n_in, D, H, dk, dv, F, enc_layers, d_enc_params, d_elen, act, enc, precision));
        if (cached) {
            DL4S_TRY(dl4s_cuda_decoder_cache_create(1, L, n_in, D, H, dk, dv, F, dec_layers, d_dec_params, &cache));
            DL4S_TRY(dl4s_cuda_decoder_cache_set_encoder(cache, enc, d_elen));
        }
        const int64_t shape[2] = {1, vocab};
        const int32_t axis = 1;
        for (int64_t t = 0; t < L; ++t) {
            const float *last = nullptr;
            if (cached) {
                // the newest token only: its embedding at position t through every layer's caches
                DL4S_TRY(dl4s_cuda_embed_at(d_tok + t, 1, 1, t, D, d_embedding, vocab, -1, dx));
                DL4S_TRY(dl4s_cuda_decoder_step(cache, dx, act, dy));
                last = dy;
            } else {
                // decIn = prepareInputs([start] + tokens); output = decoder(decIn, encoded, [n_in], [t + 1])   (:124-126)
                DL4S_TRY(dl4s_cuda_fill_i32((int32_t)(t + 1), d_len, 1));
                DL4S_TRY(dl4s_cuda_embed_positional(d_tok, 1, t + 1, D, d_embedding, vocab, -1, dx));
                DL4S_TRY(dl4s_cuda_decoder_forward(dx, enc, 1, t + 1, n_in, D, H, dk, dv, F, dec_layers, d_dec_params, d_len, d_elen, act,
                                                   dy, precision));
                last = dy + t * D;
            }
            // deembedded[0, -1].argmax(): the last row against the embedding matrix, no bias, no softmax   (:127-129)
            DL4S_TRY(launch_gemm_f32(st, last, d_embedding, logits, 1, vocab, D, 1.0f, 0.0f, 0, 1, EPI_NONE, nullptr, nullptr));
            DL4S_TRY(dl4s_cuda_reduce_max(logits, shape, 2, &axis, 1, mx, d_tok + t + 1));
            // the host looks at the tokens every 8 steps (the reference reads each one back): stop at the end token
            if ((t & 7) == 7 || t == L - 1) {
                DL4S_CUDA_TRY(cudaMemcpyAsync(tokens, d_tok + 1, (size_t)(t + 1) * 4, cudaMemcpyDeviceToHost, st->stream));
                DL4S_CUDA_TRY(cudaStreamSynchronize(st->stream));
                for (int64_t i = 0; i <= t; ++i) {
                    if (tokens[i] == end_token) { *n_tokens = i + 1; return DL4S_OK; }
                }
                *n_tokens = t + 1;
            }
        }
        return DL4S_OK;
    };
    s = run();
    cudaStreamSynchronize(st->stream);
    if (cache) dl4s_cuda_decoder_cache_destroy(cache);
    cudaFree(block);
    return s;
}

}  // extern "C"
