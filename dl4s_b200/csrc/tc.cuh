// Host-side interface of the tensor-core (tcgen05) kernels.
#pragma once

#include "common.cuh"

namespace dl4s {

// gemm_tc.cu — C[M,N] = A[M,K] B[K,N] (+ epilogue) with half operands, fp32
// accumulation in tensor memory. Needs K % 64 == 0 and N % 64 == 0 (TMA boxes
// of 128 bytes); other shapes use the fp32 kernel.
bool gemm_tc_supported(int64_t M, int64_t N, int64_t K);
size_t gemm_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int split = 0);
dl4s_status launch_gemm_tc(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                           int epilogue, const float *bias, const float *residual, void *scratch, size_t scratch_bytes,
                           int split = 0, const DropoutSpec *drop = nullptr);

// C = op(A) op(B) with A stored [K, M] (trans_a) and/or B stored [N, K] (trans_b): the products of a matmul's backward.
bool gemm_tc_trans_supported(int64_t M, int64_t N, int64_t K, int trans_a, int trans_b);
dl4s_status launch_gemm_tc_trans(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                                 int trans_a, int trans_b, void *scratch, size_t scratch_bytes);

// The same product with operands that are already half ([M,K] and [K,N], 16-byte aligned)
// and a choice of output: fp32 [M,N], half [M,N], or half scattered head-major into up to
// three tensors [B,H,S,d] (rows are m = b*S + s; used by the fused q/k/v projection).
enum GemmOutMode { OUT_F32 = 0, OUT_F16 = 1, OUT_HEADS_F16 = 2 };
// Epilogue flavour beyond those of common.cuh: residual add that also leaves partial sums (sum, sum of squares)
// of the result for a LayerNorm over whole [S, D] blocks. Each epilogue warp writes one pair of doubles per
// tile for its 32 rows and its share of the tile's columns; the pairs of one 32-row block are contiguous
// (gemm_tc_stats_per_row_block of them);
// the 32 rows must lie inside one block (S % 32 == 0). Sums are taken in a fixed order: no atomics.
constexpr int EPI_RESIDUAL_STATS = 6;
struct GemmTcOut {
    int mode = OUT_F32;
    void *c = nullptr;
    int nparts = 0;
    void *part_ptr[3] = {nullptr, nullptr, nullptr};
    int part_d[3] = {0, 0, 0};
    int S = 1, H = 1;
    double *ln_stats = nullptr;   // EPI_RESIDUAL_STATS
};
// Number of (sum, sum of squares) pairs EPI_RESIDUAL_STATS leaves per 32 rows for a product with N columns.
int gemm_tc_stats_per_row_block(int64_t N);
// b_split != 0: `b_half` is [2K, N], the half-rounded matrix on top of the half-rounded remainder (W_hi; W_lo); the
// product is A W_hi + A W_lo in one accumulator, i.e. B enters with ~22 significant bits at twice the MMA work.
// b_split_from_col > 0 (a multiple of the tile width): only the columns from there on take the remainder; the columns
// before it are A W_hi alone at the plain product's cost.
// A may be given as `a_groups` column blocks: element (m, g*K/a_groups + c) lies at
// a_half[g * a_group_stride + m * K/a_groups + c] (the rank-major layout of an all-gather).
dl4s_status launch_gemm_tc_h(DeviceState *st, const void *a_half, const void *b_half, int64_t M, int64_t N, int64_t K,
                             int epilogue, const float *bias, const float *residual, const GemmTcOut &out,
                             int64_t a_groups = 1, int64_t a_group_stride = 0, int b_split = 0,
                             const DropoutSpec *drop = nullptr, int64_t b_split_from_col = 0);
dl4s_status launch_f32_to_f16(DeviceState *st, const float *x, void *y, int64_t n);
// hi = half(x), lo = half(x - hi): the two-half form of a weight matrix (b_split above reads [hi; lo] stacked along k).
dl4s_status launch_f32_to_f16_hilo(DeviceState *st, const float *x, void *hi, void *lo, int64_t n);

// attn_prefill.cu — flash-style attention with tcgen05 MMAs. Masks are
// structural only (key lengths and/or causal).
bool attn_prefill_tc_supported(int64_t Sq, int64_t Sk, int64_t dk, int64_t dv);
size_t attn_prefill_tc_scratch_bytes(int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv);
dl4s_status launch_attn_prefill_tc(DeviceState *st, const float *q, Strides4 qs, const float *k, Strides4 ks, const float *v,
                                   Strides4 vs, float *o, Strides4 os, int64_t B, int64_t H, int64_t Sq, int64_t Sk,
                                   int64_t dk, int64_t dv, float inv_temperature, const MaskSpec &mask, void *scratch,
                                   size_t scratch_bytes);

// The same kernel on operands that are already half and head-major: qh [B*H,Sq,D]
// (pre-multiplied by attn_prefill_tc_q_scale), kh, vh [B*H,Sk,D]. The output goes to
// `o` with (batch, head, row) strides in elements, as fp32 or (o_half != 0) as half.
float attn_prefill_tc_q_scale(float inv_temperature);
// `lse` (optional, [B*H, Sq]): log2 of every row's softmax denominator in base-2 score units (scores = qh . kh), which
// is what the backward kernel needs to recompute the probabilities.
dl4s_status launch_attn_prefill_tc_h(DeviceState *st, const void *qh, const void *kh, const void *vh, void *o, Strides4 os,
                                     int o_half, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t D, const MaskSpec &mask,
                                     float *lse = nullptr);

// Strided fp32 [B,H,S,D] -> contiguous half [B*H,S,D], multiplied by `scale`.
dl4s_status pack_heads_f16(DeviceState *st, const float *src, Strides4 ss, void *dst, int64_t BH, int64_t H, int64_t S, int D,
                           float scale);

// attn_bwd_tc.cu — flash-style backward of the same attention on the tensor cores: dq, dk, dv [B,H,S,D] fp32
// (contiguous) from q, k, v, dout (fp32, contiguous) with structural masks; the probabilities are recomputed.
bool attn_bwd_tc_supported(int64_t Sq, int64_t Sk, int64_t dk, int64_t dv);
dl4s_status launch_attn_bwd_tc(DeviceState *st, const float *q, const float *k, const float *v, const float *dout, int64_t B,
                               int64_t H, int64_t Sq, int64_t Sk, int64_t D, float inv_temperature, const MaskSpec &mask, float *dq,
                               float *dk, float *dv);

// encoder_tc.cu — the fused tensor-core pipelines (intermediates in half, no conversion passes).
// They reserve their own scratch from the device arena.
bool tc_block_supported(int64_t B, int64_t Sq, int64_t Sk, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F);
// `split` != 0: weights as two halves (hi + lo), see encoder_tc.cu.
dl4s_status mha_self_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                        const float *wq, const float *wk, const float *wv, const float *wo, const float *g, const float *sh,
                        const MaskSpec &mask, float *out, int split);
dl4s_status mha_heads_self_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk,
                              int64_t dv, const float *wq, const float *wk, const float *wv, const MaskSpec &mask, void *out,
                              int out_half, int split, const void *x_half = nullptr);
dl4s_status mha_output_tc(DeviceState *st, const void *heads, int heads_half, const float *residual, int64_t B, int64_t S,
                          int64_t D, int64_t HDv, const float *wo, const float *g, const float *sh, float *out,
                          int64_t groups, int64_t group_stride, int split);
dl4s_status ffn_tc(DeviceState *st, const float *x, int64_t M, int64_t D, int64_t F, const float *w1, const float *b1,
                   const float *w2, const float *b2, const float *g, const float *sh, int act, float *out, int split);
dl4s_status encoder_tc(DeviceState *st, const float *x, int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv,
                       int64_t F, int64_t layers, const float *params, const MaskSpec &mask, int act, float *out, int split);
// Half weights of a whole encoder converted once and kept in device memory of their own.
dl4s_status encoder_prepare(DeviceState *st, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int64_t layers,
                            const float *params, int split, void **handle);
dl4s_status encoder_prepared_refresh(DeviceState *st, void *handle);
dl4s_status encoder_prepared_destroy(DeviceState *st, void *handle);
dl4s_status encoder_tc_prepared(DeviceState *st, void *handle, const float *x, int64_t B, int64_t S, const MaskSpec &mask, int act,
                                float *out);

// Scratch one encoder layer's tensor-core kernels need at most (operand copies
// in half precision); F == 0 leaves the feed-forward GEMMs out.
size_t tc_layer_scratch_bytes(int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int split = 0);

}  // namespace dl4s
