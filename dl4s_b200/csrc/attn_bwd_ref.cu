// fp32 backward of scaled-dot-product attention: the gradients DL4S's autograd produces for
// NN/Models/Transformer/ScaledDotProductAttention.swift:43-64 by chaining the backward closures of
// its primitives (mmul: Tensor/Operators/Matrix.swift:139-173; softmax = exp / sum with a detached
// max: Unary.swift:190-194), in one call and without the forward having kept anything:
//   P  = softmax((q / T) k^T - mask * 1e9)        recomputed
//   dP = dout v^T,  dS = P * (dP - rowsum(dP * P))
//   dq = (dS k) / T,  dk = dS^T (q / T),  dv = P^T dout
// Two kernels. The first owns query rows (one warp per row, the row of P in shared memory, like the
// forward check kernel): it writes dq and leaves P and dS in scratch [B*H, Sq, Sk]. The second owns
// key rows (one warp per four keys): it sums the columns of P and dS against dout and q. Both sum
// in a fixed order: the result does not depend on scheduling. This is the fp32 reference path for
// training on the device; it materialises the score matrix like the CPU engine does.
#include "common.cuh"
#include "tc.cuh"

namespace dl4s {

struct AttnBwdParams {
    const float *q, *k, *v, *g;   // contiguous [B,H,S,d]
    float *dq, *dk, *dv;
    float *P, *dS;                // scratch [B*H, Sq, Sk]
    int64_t B, H, Sq, Sk, dkk, dvv;
    float inv_t;
    const int32_t *lens;
    int causal;
    const float *mask;
    int64_t ms[4];
    int warps;
};

__global__ void k_attn_bwd_rows(AttnBwdParams p)
{
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *pr = smem + (int64_t)warp * (2 * p.Sk + p.dkk + p.dvv);   // probabilities of this warp's row
    float *ds = pr + p.Sk;                                            // dP, then dS
    float *qrow = ds + p.Sk;
    float *grow = qrow + p.dkk;
    const int64_t total_rows = p.B * p.H * p.Sq;
    for (int64_t row = (int64_t)blockIdx.x * p.warps + warp; row < total_rows; row += (int64_t)gridDim.x * p.warps) {
        const int64_t i = row % p.Sq, bh = row / p.Sq, h = bh % p.H, b = bh / p.H;
        const float *qp = p.q + row * p.dkk;
        const float *gp = p.g + row * p.dvv;
        const float *kp = p.k + bh * p.Sk * p.dkk;
        const float *vp = p.v + bh * p.Sk * p.dvv;
        __syncwarp();
        for (int64_t d = lane; d < p.dkk; d += 32) qrow[d] = qp[d] * p.inv_t;
        for (int64_t d = lane; d < p.dvv; d += 32) grow[d] = gp[d];
        __syncwarp();
        // The same structure as the forward check kernel: keys behind the length or the causal diagonal have
        // weight exactly 0 (and so no gradient) unless every key is blocked, which leaves the reference's
        // literal `score - 1e9` on all keys.
        int64_t len = p.lens ? p.lens[b] : p.Sk;
        if (len > p.Sk) len = p.Sk;
        const bool all_blocked = len <= 0;
        int64_t kv_end = all_blocked ? p.Sk : len;
        if (p.causal && !all_blocked && i + 1 < kv_end) kv_end = i + 1;
        const float *mrow = nullptr;
        if (p.mask) {
            int64_t mb = p.ms[0] == 1 ? 0 : b, mh = p.ms[1] == 1 ? 0 : h, mr = p.ms[2] == 1 ? 0 : i;
            mrow = p.mask + ((mb * p.ms[1] + mh) * p.ms[2] + mr) * p.ms[3];
        }
        float mx = -INFINITY;
        for (int64_t j = lane; j < kv_end; j += 32) {
            const float *kr = kp + j * p.dkk;
            float s = 0.f;
            for (int64_t d = 0; d < p.dkk; ++d) s = fmaf(qrow[d], kr[d], s);
            if (mrow) s = s - mrow[p.ms[3] == 1 ? 0 : j] * 1e9f;
            if (all_blocked) s = s - 1e9f;
            pr[j] = s;
            mx = fmaxf(mx, s);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int64_t j = lane; j < kv_end; j += 32) {
            float e = expf(pr[j] - mx);
            pr[j] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
        // dP_j = dout_i . v_j, delta = sum_j dP_j P_j
        float delta = 0.f;
        for (int64_t j = lane; j < kv_end; j += 32) {
            const float *vr = vp + j * p.dvv;
            float t = 0.f;
            for (int64_t d = 0; d < p.dvv; ++d) t = fmaf(grow[d], vr[d], t);
            const float pj = pr[j] * inv;
            pr[j] = pj;
            ds[j] = t;
            delta = fmaf(t, pj, delta);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) delta += __shfl_xor_sync(0xffffffffu, delta, o);
        float *Pg = p.P + row * p.Sk, *Sg = p.dS + row * p.Sk;
        for (int64_t j = lane; j < p.Sk; j += 32) {
            float pj = 0.f, sj = 0.f;
            if (j < kv_end) {
                pj = pr[j];
                sj = pj * (ds[j] - delta);
                ds[j] = sj;
            }
            Pg[j] = pj;
            Sg[j] = sj;
        }
        __syncwarp();
        // dq_i = (sum_j dS_j k_j) / T
        float *dqp = p.dq + row * p.dkk;
        for (int64_t c = lane; c < p.dkk; c += 32) {
            float acc = 0.f;
            for (int64_t j = 0; j < kv_end; ++j) acc = fmaf(ds[j], kp[j * p.dkk + c], acc);
            dqp[c] = acc * p.inv_t;
        }
    }
}

constexpr int BW_KEYS = 4;    // keys per warp in the column kernel
constexpr int BW_MAXD = 8;    // head size up to 32 * BW_MAXD

__global__ void __launch_bounds__(256) k_attn_bwd_cols(AttnBwdParams p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t groups_per_bh = (p.Sk + BW_KEYS - 1) / BW_KEYS;
    const int64_t total = p.B * p.H * groups_per_bh;
    const int nk = (int)((p.dkk + 31) / 32), nv = (int)((p.dvv + 31) / 32);
    for (int64_t grp = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp; grp < total; grp += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int64_t bh = grp / groups_per_bh, j0 = (grp % groups_per_bh) * BW_KEYS;
        const float *qp = p.q + bh * p.Sq * p.dkk;
        const float *gp = p.g + bh * p.Sq * p.dvv;
        const float *Pg = p.P + bh * p.Sq * p.Sk, *Sg = p.dS + bh * p.Sq * p.Sk;
        float acc_k[BW_KEYS][BW_MAXD], acc_v[BW_KEYS][BW_MAXD];
#pragma unroll
        for (int a = 0; a < BW_KEYS; ++a)
#pragma unroll
            for (int c = 0; c < BW_MAXD; ++c) { acc_k[a][c] = 0.f; acc_v[a][c] = 0.f; }
        for (int64_t i = 0; i < p.Sq; ++i) {
            float pj[BW_KEYS], sj[BW_KEYS];
            bool any = false;
#pragma unroll
            for (int a = 0; a < BW_KEYS; ++a) {
                const int64_t j = j0 + a;
                pj[a] = j < p.Sk ? Pg[i * p.Sk + j] : 0.f;
                sj[a] = j < p.Sk ? Sg[i * p.Sk + j] : 0.f;
                any = any || pj[a] != 0.f || sj[a] != 0.f;
            }
            if (!any) continue;     // rows that cannot see these keys (same for all lanes)
#pragma unroll
            for (int c = 0; c < BW_MAXD; ++c) {
                if (c < nv) {
                    const int64_t d = c * 32 + lane;
                    const float gv = d < p.dvv ? gp[i * p.dvv + d] : 0.f;
#pragma unroll
                    for (int a = 0; a < BW_KEYS; ++a) acc_v[a][c] = fmaf(pj[a], gv, acc_v[a][c]);
                }
                if (c < nk) {
                    const int64_t d = c * 32 + lane;
                    const float qv = d < p.dkk ? qp[i * p.dkk + d] * p.inv_t : 0.f;
#pragma unroll
                    for (int a = 0; a < BW_KEYS; ++a) acc_k[a][c] = fmaf(sj[a], qv, acc_k[a][c]);
                }
            }
        }
#pragma unroll
        for (int a = 0; a < BW_KEYS; ++a) {
            const int64_t j = j0 + a;
            if (j >= p.Sk) continue;
#pragma unroll
            for (int c = 0; c < BW_MAXD; ++c) {
                const int64_t d = c * 32 + lane;
                if (c < nv && d < p.dvv) p.dv[(bh * p.Sk + j) * p.dvv + d] = acc_v[a][c];
                if (c < nk && d < p.dkk) p.dk[(bh * p.Sk + j) * p.dkk + d] = acc_k[a][c];
            }
        }
    }
}

dl4s_status launch_attn_bwd_ref(DeviceState *st, const float *q, const float *k, const float *v, const float *dout, int64_t B,
                                int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, float inv_temperature,
                                const MaskSpec &mask, float *dq, float *dkk, float *dvv)
{
    if (B * H == 0) return DL4S_OK;
    DL4S_REQUIRE(Sq >= 1 && Sk >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(dk <= 32 * BW_MAXD && dv <= 32 * BW_MAXD, "the fp32 backward handles head sizes up to %d", 32 * BW_MAXD);
    const size_t mat = align_up((size_t)(B * H * Sq * Sk) * sizeof(float), 1024);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, 2 * mat, &base));
    AttnBwdParams p;
    p.q = q; p.k = k; p.v = v; p.g = dout;
    p.dq = dq; p.dk = dkk; p.dv = dvv;
    p.P = (float *)base;
    p.dS = (float *)((char *)base + mat);
    p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.dkk = dk; p.dvv = dv;
    p.inv_t = inv_temperature;
    p.lens = mask.d_key_lengths;
    p.causal = mask.causal;
    p.mask = mask.d_mask;
    for (int i = 0; i < 4; ++i) p.ms[i] = mask.ms[i];
    const size_t budget = 200 * 1024;
    const size_t per_warp = (size_t)(2 * Sk + dk + dv) * sizeof(float);
    int warps = 8;
    while (warps > 1 && (size_t)warps * per_warp > budget) warps >>= 1;
    if ((size_t)warps * per_warp > budget)
        return fail(DL4S_ERR_UNSUPPORTED, "the fp32 backward keeps two rows of Sk floats on chip: Sk = %lld is too long", (long long)Sk);
    p.warps = warps;
    static bool attr_set[kMaxDevices] = {false};
    if (!attr_set[st->ordinal]) {
        DL4S_CUDA_TRY(cudaFuncSetAttribute(k_attn_bwd_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
        attr_set[st->ordinal] = true;
    }
    int64_t blocks = ceil_div(B * H * Sq, warps);
    int64_t cap = (int64_t)st->sm_count * 16;
    if (blocks > cap) blocks = cap;
    k_attn_bwd_rows<<<(unsigned)blocks, warps * 32, (size_t)warps * per_warp, st->stream>>>(p);
    DL4S_TRY(after_launch(st, "k_attn_bwd_rows"));
    int64_t groups = B * H * ceil_div(Sk, BW_KEYS);
    blocks = ceil_div(groups, 8);
    if (blocks > cap) blocks = cap;
    k_attn_bwd_cols<<<(unsigned)blocks, 256, 0, st->stream>>>(p);
    return after_launch(st, "k_attn_bwd_cols");
}

}  // namespace dl4s

using namespace dl4s;

extern "C" dl4s_status dl4s_cuda_sdpa_backward(const float *d_q, const float *d_k, const float *d_v, const float *d_dout, int64_t B,
                                               int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv, float temperature,
                                               const int32_t *d_key_lengths, int32_t causal, const float *d_mask,
                                               const int64_t *mask_shape, float *d_dq, float *d_dk, float *d_dv, int32_t precision)
{
    DL4S_STATE(st);
    DL4S_REQUIRE(d_q && d_k && d_v && d_dout && d_dq && d_dk && d_dv, "NULL buffer");
    DL4S_REQUIRE(B >= 0 && H >= 0 && Sq >= 1 && Sk >= 1 && dk >= 1 && dv >= 1, "bad extents");
    DL4S_REQUIRE(temperature != 0.0f, "temperature must not be zero");
    DL4S_REQUIRE(!d_mask || mask_shape, "a dense mask needs its shape");
    DL4S_REQUIRE(!causal || Sq == Sk, "the causal mask of DL4S is square: Sq must equal Sk");
    MaskSpec mask;
    mask.d_key_lengths = d_key_lengths;
    mask.causal = causal;
    mask.d_mask = d_mask;
    if (d_mask) {
        const int64_t full[4] = {B, H, Sq, Sk};
        for (int i = 0; i < 4; ++i) {
            DL4S_REQUIRE(mask_shape[i] == 1 || mask_shape[i] == full[i], "mask extent %d is %lld; it must be 1 or %lld", i,
                         (long long)mask_shape[i], (long long)full[i]);
            mask.ms[i] = mask_shape[i];
        }
    }
    DL4S_REQUIRE(precision == DL4S_PREC_FP32 || precision == DL4S_PREC_F16 || precision == DL4S_PREC_F16_SPLIT,
                 "unknown precision %d", precision);
    ScopedTimer timer(st);
    // Tensor-core path: structural masks, head sizes 64 / 128 (no weights are involved, so the two tensor-core
    // precisions are the same here); everything else runs on the fp32 kernels.
    if (precision != DL4S_PREC_FP32 && !d_mask && dk == dv && attn_bwd_tc_supported(Sq, Sk, dk, dv) && B * H <= 65535 &&
        (((uintptr_t)d_q | (uintptr_t)d_k | (uintptr_t)d_v | (uintptr_t)d_dout | (uintptr_t)d_dq | (uintptr_t)d_dk | (uintptr_t)d_dv) & 15) == 0)
        return launch_attn_bwd_tc(st, d_q, d_k, d_v, d_dout, B, H, Sq, Sk, dk, 1.0f / temperature, mask, d_dq, d_dk, d_dv);
    return launch_attn_bwd_ref(st, d_q, d_k, d_v, d_dout, B, H, Sq, Sk, dk, dv, 1.0f / temperature, mask, d_dq, d_dk, d_dv);
}
