// Flash-style scaled-dot-product attention on the sm_100a tensor cores.
// Computes ScaledDotProductAttention.swift:43-64 without ever forming the
// [Sq,Sk] score matrix: softmax((q/temperature) k^T - mask*1e9) v with the mask
// given structurally (key lengths of makeEncoderMasks and/or the causal band of
// makeDecoderMasks, TransformerUtil.swift:29-50).
//
// A conversion pass writes q (pre-multiplied by log2(e)/temperature), k and v
// as half tensors [B*H, S, D]. The main kernel gives one CTA a block of 256
// query rows of one (batch, head) pair, as two 128-row tiles A and B:
//   warps 0-3 / 4-7  softmax of tile A / B: one thread per query row reads its
//                    128 scores from tensor memory (tcgen05.ld), keeps the running
//                    max and sum, writes the probabilities back as halves over the
//                    scores (tcgen05.st) and, when the running max has moved by
//                    more than 2^8, rescales the output accumulator;
//   warp 8           TMA producer: Q once, then K and V tiles of 128 keys through
//                    separate rings (128-byte swizzle);
//   warp 9           MMA issuer: S = Q K^T (both operands K-major from shared
//                    memory) and O += P V (P from tensor memory, V as an MN-major
//                    shared-memory operand), fp32 accumulation in tensor memory,
//                    ordered S_A S_B | PV_A S_A' PV_B S_B' | ... so that one tile's
//                    softmax overlaps the other tile's MMAs.
// Tensor memory: S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [384,384+D).
// 64-wide heads use a second form of the same kernel: ONE 128-row tile per CTA (warps 0-3 softmax, 4 TMA,
// 5 MMA; S [0,128) O [128,192) of 256 tensor-memory columns; 80 KB of shared memory) and two CTAs per SM.
// There the exp2 unit (16 results per clock per SM) needs twice the time of the MMAs, so nothing is lost by
// letting the two tiles of an SM belong to different CTAs, and each CTA's start (barriers, tensor-memory
// allocation, first loads: ~5600 cycles measured) and output pass (~2200) run under the other's softmax.
// Measured against the two-tile form: B 32, H 8, S 512 (encoder) 45 vs 49 us; causal S 1024 / 4096 / 8192:
// 324 / 571 / 638 vs 297 / 544 / 617 TFLOP/s.
// Key tiles beyond the causal diagonal or beyond the sequence length are never
// loaded; the diagonal / tail tile is masked in registers. A sequence of length
// 0 follows the reference's finite -1e9: uniform weights over all Sk keys.
// Every mbarrier wait is bounded (status word + common exit on expiry).
#include "tc.cuh"
#include "tc_device.cuh"

namespace dl4s {

using namespace tc;

// NT query tiles of 128 rows per CTA. NT = 2: 384 threads (warps 0-7 softmax, 8 TMA, 9 MMA, 10-11 only complete the
// third warpgroup), one CTA per SM. NT = 1: 256 threads (warps 0-3 softmax, 4 TMA, 5 MMA), two CTAs per SM.
__host__ __device__ constexpr int at_threads(int nt) { return nt == 2 ? 384 : 256; }
__host__ __device__ constexpr int at_stages(int d, int nt) { return (d == 128 || nt == 1) ? 2 : 3; }
constexpr int AT_TILE = 128;       // rows per query tile and keys per key tile
constexpr int AT_HEAD_GROUP = 8;   // (batch, head) pairs whose blocks are handed out together
constexpr float kLog2e = 1.4426950408889634f;

dl4s_status launch_f32_to_f16(DeviceState *st, const float *x, void *y, int64_t n);

// Strided fp32 [B,H,S,D] -> contiguous half [B*H,S,D], scaled.
__global__ void __launch_bounds__(256) k_pack_heads_f16(const float *__restrict__ x, Strides4 xs, __half *__restrict__ y,
                                                        int64_t H, int64_t S, int D, float scale, int64_t total_vec)
{
    const int vec_per_row = D / 8;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < total_vec; i += stride) {
        int64_t row = i / vec_per_row;
        int c = (int)(i % vec_per_row) * 8;
        int64_t s = row % S, bh = row / S, h = bh % H, b = bh / H;
        const float4 *src = reinterpret_cast<const float4 *>(x + b * xs.b + h * xs.h + s * xs.s + c);
        float4 a0 = src[0], a1 = src[1];
        __half2 h0 = __floats2half2_rn(a0.x * scale, a0.y * scale), h1 = __floats2half2_rn(a0.z * scale, a0.w * scale);
        __half2 h2 = __floats2half2_rn(a1.x * scale, a1.y * scale), h3 = __floats2half2_rn(a1.z * scale, a1.w * scale);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t *>(&h0);
        o.y = *reinterpret_cast<uint32_t *>(&h1);
        o.z = *reinterpret_cast<uint32_t *>(&h2);
        o.w = *reinterpret_cast<uint32_t *>(&h3);
        *reinterpret_cast<uint4 *>(y + row * D + c) = o;
    }
}

dl4s_status pack_heads_f16(DeviceState *st, const float *src, Strides4 ss, void *dst, int64_t BH, int64_t H, int64_t S, int D,
                           float scale)
{
    int64_t total_vec = BH * S * (D / 8);
    if (total_vec == 0) return DL4S_OK;
    int64_t blocks = ceil_div(total_vec, 256 * 4);
    int64_t cap = (int64_t)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    k_pack_heads_f16<<<(unsigned)blocks, 256, 0, st->stream>>>(src, ss, (__half *)dst, H, S, D, scale, total_vec);
    return after_launch(st, "k_pack_heads_f16");
}

struct AttnTcParams {
    void *o;                 // float (o_half == 0) or half (o_half == 1), strides in elements
    int o_half;
    Strides4 os;
    int64_t H;
    int Sq, Sk;
    const int32_t *lens;
    int causal;
    int nqb;                 // blocks of NT x 128 query rows
    int BH;                  // batch * heads
    int32_t *status;
    float *lse;              // optional [B*H, Sq]: log2 of each row's softmax denominator, in the kernel's base-2 score units
};

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Two fp32 values in one 64-bit register for the packed fp32x2 instructions of sm_100.
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);   // a in the low half: element 2c of the row
    return *reinterpret_cast<uint32_t *>(&h);
}

template <int D, int NT>
__global__ void __launch_bounds__(at_threads(NT), NT == 2 ? 1 : 2) k_attn_prefill_tc(const __grid_constant__ CUtensorMap tmap_q,
                                                                   const __grid_constant__ CUtensorMap tmap_k,
                                                                   const __grid_constant__ CUtensorMap tmap_v, AttnTcParams p)
{
    constexpr int NBLK = D / 64;                        // 64-column blocks of a tile
    constexpr uint32_t BLK_BYTES = AT_TILE * 128;       // 128 rows x 128 bytes = 16 KB
    constexpr uint32_t TILE_BYTES = BLK_BYTES * NBLK;
    constexpr int KSTAGES = at_stages(D, NT);
    constexpr int VSTAGES = at_stages(D, NT);
    constexpr int W_TMA = 4 * NT, W_MMA = 4 * NT + 1;   // the warps after the softmax warps
    constexpr uint32_t TMEM_COLS = NT == 2 ? 512 : 256;
    constexpr uint32_t IDESC_S = idesc_f16(128, 128, 0, 0);   // Q K^T: both K-major
    constexpr uint32_t IDESC_O = idesc_f16(128, D, 0, 1);     // P V: V is MN-major
    constexpr uint32_t TM_S0 = 0, TM_S1 = 128, TM_O0 = NT * 128, TM_O1 = TM_O0 + 128;   // NT = 1: S [0,128) O [128,128+D)

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem;                                  // NT tiles
    uint8_t *sK = sQ + NT * TILE_BYTES;
    uint8_t *sV = sK + KSTAGES * TILE_BYTES;
    __shared__ uint64_t q_full, k_full[KSTAGES], k_empty[KSTAGES], v_full[VSTAGES], v_empty[VSTAGES];
    __shared__ uint64_t s_full[2], p_ready[2], o_done[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Work order. With a causal mask the last query block of a head visits the most key tiles, so
    // blocks are handed out heaviest first — not head by head (the last head's heavy blocks would
    // start when everything else is finishing) and not across all heads at once (the CTAs running
    // together would share no K/V in L2), but in groups of AT_HEAD_GROUP heads: within a group all
    // heads' heaviest blocks, then the next lighter ones, and so on.
    const int per_group = p.nqb * AT_HEAD_GROUP;
    const int group = (int)blockIdx.x / per_group;
    const int r = (int)blockIdx.x - group * per_group;
    const int gsize = min(AT_HEAD_GROUP, p.BH - group * AT_HEAD_GROUP);
    const int qb = p.nqb - 1 - r / gsize;
    const int bh = group * AT_HEAD_GROUP + r % gsize;
    const int b = bh / (int)p.H, h = bh % (int)p.H;

    int len = p.lens ? p.lens[b] : p.Sk;
    if (len > p.Sk) len = p.Sk;
    const bool uniform = len <= 0;            // every key blocked: equal weights over all Sk keys
    const int kv_limit = uniform ? p.Sk : len;
    const int n_len = (kv_limit + AT_TILE - 1) / AT_TILE;
    const int row0 = qb * NT * AT_TILE;
    int n_tile[2];
    n_tile[0] = (row0 < p.Sq) ? n_len : 0;
    n_tile[1] = (NT == 2 && row0 + AT_TILE < p.Sq) ? n_len : 0;
    if (p.causal && !uniform) {
        n_tile[0] = min(n_tile[0], NT * qb + 1);
        n_tile[1] = min(n_tile[1], NT * qb + 2);
    }
    const int n_max = max(n_tile[0], n_tile[1]);

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < KSTAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VSTAGES; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_ready[t], 128); mbar_init(&o_done[t], 1); }
        abort_s = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA) { tmem_alloc(&tmem_base_s, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    // Register budget: the two softmax warpgroups keep 128 scores per thread live, the
    // producer warpgroup needs very little. 256*200 + 128*96 <= 384*168 registers.
    // (The instruction sits inside the role branches, which do not rejoin before the exit,
    // so the compiler knows which budget holds where.)
    if (warp >= 4 * NT) {
    if (NT == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == W_TMA) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            mbar_expect_tx(&q_full, NT * TILE_BYTES);
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk)
                    tma_load_3d(sQ + t * TILE_BYTES + blk * BLK_BYTES, &tmap_q, &q_full, blk * 64, row0 + t * AT_TILE, bh);
            uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
            for (int j = 0; j < n_max; ++j) {
                if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag)) break;
                mbar_expect_tx(&k_full[ks], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk)
                    tma_load_3d(sK + ks * TILE_BYTES + blk * BLK_BYTES, &tmap_k, &k_full[ks], blk * 64, j * AT_TILE, bh);
                if (++ks == KSTAGES) { ks = 0; kph ^= 1; }
                if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag)) break;
                mbar_expect_tx(&v_full[vs], TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk)
                    tma_load_3d(sV + vs * TILE_BYTES + blk * BLK_BYTES, &tmap_v, &v_full[vs], blk * 64, j * AT_TILE, bh);
                if (++vs == VSTAGES) { vs = 0; vph ^= 1; }
            }
        }
    } else if (warp == W_MMA) {
        // -------------------------------------------------------------- MMA issuer
        if (elect_one() && n_max > 0) {
            uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
            bool ok = true;
            const uint32_t sq = smem_u32(sQ);
            auto issue_qk = [&](int t, uint32_t kbase) {
                const uint32_t d_tmem = tmem_base + (t ? TM_S1 : TM_S0);
                const uint32_t qbase = sq + t * TILE_BYTES;
#pragma unroll
                for (int k16 = 0; k16 < D / 16; ++k16) {
                    const uint32_t off = (k16 / 4) * BLK_BYTES + (k16 % 4) * 32;
                    umma_ss(d_tmem, smem_desc_sw128(qbase + off, 16, 1024), smem_desc_sw128(kbase + off, 16, 1024), IDESC_S,
                            k16 != 0);
                }
                umma_commit(&s_full[t]);
            };
            auto issue_pv = [&](int t, uint32_t vbase, int j) {
                const uint32_t d_tmem = tmem_base + (t ? TM_O1 : TM_O0);
                const uint32_t p_tmem = tmem_base + (t ? TM_S1 : TM_S0);
#pragma unroll
                for (int k16 = 0; k16 < AT_TILE / 16; ++k16)
                    umma_ts(d_tmem, p_tmem + k16 * 8, smem_desc_mn_sw128(vbase + k16 * 2048, BLK_BYTES, 1024), IDESC_O,
                            (j | k16) != 0);
                umma_commit(&o_done[t]);
            };
            ok = mbar_wait(&q_full, 0, abort_flag);
            // Prologue: scores of key tile 0 for both query tiles.
            if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                const uint32_t kbase = smem_u32(sK);
                if (n_tile[0] > 0) issue_qk(0, kbase);
                if (n_tile[1] > 0) issue_qk(1, kbase);
                umma_commit(&k_empty[0]);
                ks = 1; if (ks == KSTAGES) { ks = 0; kph ^= 1; }
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const bool more = (j + 1 < n_max);
                if (!(ok = mbar_wait(&v_full[vs], vph, abort_flag))) break;
                const uint32_t vbase = smem_u32(sV + vs * TILE_BYTES);
                uint32_t kbase = 0;
                // O_A += P_A V_j, then the next scores of tile A.
                if (j < n_tile[0]) {
                    if (!(ok = mbar_wait(&p_ready[0], j & 1, abort_flag))) break;
                    tc_fence_after();
                    issue_pv(0, vbase, j);
                }
                if (more) {
                    if (!(ok = mbar_wait(&k_full[ks], kph, abort_flag))) break;
                    tc_fence_after();
                    kbase = smem_u32(sK + ks * TILE_BYTES);
                    if (j + 1 < n_tile[0]) issue_qk(0, kbase);
                }
                if (j < n_tile[1]) {
                    if (!(ok = mbar_wait(&p_ready[1], j & 1, abort_flag))) break;
                    tc_fence_after();
                    issue_pv(1, vbase, j);
                }
                umma_commit(&v_empty[vs]);
                if (++vs == VSTAGES) { vs = 0; vph ^= 1; }
                if (more) {
                    if (j + 1 < n_tile[1]) issue_qk(1, kbase);
                    umma_commit(&k_empty[ks]);
                    if (++ks == KSTAGES) { ks = 0; kph ^= 1; }
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        // ------------------------------------------------- softmax of tile t, one row per thread
        const int t = warp >> 2;
        const int quarter = warp & 3;
        const int n_t = n_tile[t];
        const int r_local = quarter * 32 + lane;
        const int row = row0 + t * AT_TILE + r_local;            // query index of this thread
        const uint32_t tm_s = tmem_addr(tmem_base, quarter * 32, t ? TM_S1 : TM_S0);
        const uint32_t tm_o = tmem_addr(tmem_base, quarter * 32, t ? TM_O1 : TM_O0);
        float m_used = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            if (!(ok = mbar_wait(&s_full[t], j & 1, abort_flag))) break;
            tc_fence_after();
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, r[c]);
            tmem_wait_ld();
            const int col0 = j * AT_TILE;
            // Columns at or beyond `limit` are blocked in this tile.
            int limit = kv_limit - col0;
            if (p.causal && !uniform) limit = min(limit, row - col0 + 1);
            if (uniform) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[c][i] = 0u;   // all scores equal
            }
            if (limit < AT_TILE) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i >= limit) r[c][i] = 0xff800000u;   // -inf
            }
            // Row max: four independent chains of 3-input max.
            float mc[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                mc[c] = fmaxf(__uint_as_float(r[c][0]), __uint_as_float(r[c][1]));
#pragma unroll
                for (int i = 2; i < 32; i += 2) mc[c] = max3(mc[c], __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
            }
            const float mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
            // Lazy rescale: keep the reference max m_used until the row max has grown by more than 2^8.
            float alpha = 1.0f;
            const bool need = mx > m_used + 8.0f;
            if (need) {
                alpha = fast_exp2(m_used - mx);     // 0 on the first tile (m_used = -inf)
                m_used = mx;
                l_sum *= alpha;
            }
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                // The accumulator must be complete through key tile j-1 before it is rescaled.
                if (!(ok = mbar_wait(&o_done[t], (j - 1) & 1, abort_flag))) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(tm_o + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tm_o + c * 32, o);
                }
            }
            // p = 2^(s - m_used), packed as halves over the first 64 columns of the score tile.
            // Pairs of columns go through packed fp32x2 arithmetic.
            const uint64_t negm2 = pack2(-m_used, -m_used);
            uint64_t acc0 = pack2(0.f, 0.f), acc1 = acc0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    uint64_t x2 = add2(pack2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), negm2);
                    float p0, p1, x0, x1;
                    unpack2(x2, x0, x1);
                    p0 = fast_exp2(x0);
                    p1 = fast_exp2(x1);
                    if (i & 1) acc1 = add2(acc1, pack2(p0, p1));
                    else acc0 = add2(acc0, pack2(p0, p1));
                    pk[i] = pack_half2(p0, p1);
                }
                tmem_st16(tm_s + c * 16, pk);
            }
            float part;
            {
                float a, b2;
                unpack2(add2(acc0, acc1), a, b2);
                part = a + b2;
            }
            l_sum += part;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_ready[t]);
        }
        // Epilogue: O / l, one output row per thread.
        if (ok && n_t > 0) ok = mbar_wait(&o_done[t], (n_t - 1) & 1, abort_flag);
        if (ok && n_t > 0) {
            tc_fence_after();
            const float inv_l = 1.0f / l_sum;
            // what the backward pass needs to recompute the probabilities: p = 2^(s - lse)
            if (p.lse && row < p.Sq) p.lse[(int64_t)bh * p.Sq + row] = m_used + log2f(l_sum);
            const int64_t ooff = (int64_t)b * p.os.b + (int64_t)h * p.os.h + (int64_t)row * p.os.s;
            float *orow = reinterpret_cast<float *>(p.o) + ooff;
            __half *hrow = reinterpret_cast<__half *>(p.o) + ooff;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tm_o + c * 32, o);
                tmem_wait_ld();
                if (row < p.Sq) {
                    if (p.o_half) {
                        // half output: the operand of the output projection that follows
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 pk;
                            pk.x = pack_half2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
                            pk.y = pack_half2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                            pk.z = pack_half2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
                            pk.w = pack_half2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
                            *reinterpret_cast<uint4 *>(hrow + c * 32 + i) = pk;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4 *>(orow + c * 32 + i) =
                                make_float4(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l,
                                            __uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                    }
                }
            }
        }
    }

    // Common exit, also reached after a wait that gave up.
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_s) atomicOr(p.status, kStatusAttnTimeout);
    if (warp == W_MMA) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Persistent form of the one-tile kernel for 64-wide heads without a causal mask (the encoder's attention): at most
// two CTAs per SM stay resident and work through the (query block, batch x head) items i, i + gridDim.x, ... .
// With sequences of a few hundred keys an item is 2-4 key tiles, and a CTA that lives for one item spends about as
// long on its start (barriers, tensor-memory allocation, first loads), on the wait for the first scores and on the
// output pass as on the key tiles themselves. Here the barriers and the tensor memory are set up once, Q has two
// buffers, and the producer loads the next item's Q, K and V while the current item is still being worked on.
// The probabilities have their own tensor-memory columns (S [0,128) P [128,192) O [192,256)) instead of lying over
// the scores, so the MMA thread issues the scores of key tile g+1 as soon as the softmax warps have READ tile g
// (s_free), in front of P_g V_g: the softmax warps find the next scores ready when they finish a tile, across item
// boundaries as well, and a key tile costs one softmax pass (bound by the exp2 unit) instead of softmax + MMAs +
// hand-offs in series. Barrier phases continue across items (g counts this CTA's key tiles).
template <int D>
__global__ void __launch_bounds__(256, 2) k_attn_prefill_tc_loop(const __grid_constant__ CUtensorMap tmap_q,
                                                                 const __grid_constant__ CUtensorMap tmap_k,
                                                                 const __grid_constant__ CUtensorMap tmap_v, AttnTcParams p)
{
    static_assert(D == 64, "the persistent form is written for 64-wide heads");
    constexpr uint32_t TILE_BYTES = AT_TILE * 128;      // 128 rows x 64 halves
    constexpr int STAGES = 2;
    constexpr int W_TMA = 4, W_MMA = 5;
    constexpr uint32_t TMEM_COLS = 256;
    constexpr uint32_t IDESC_S = idesc_f16(128, 128, 0, 0);
    constexpr uint32_t IDESC_O = idesc_f16(128, D, 0, 1);
    constexpr uint32_t TM_S = 0, TM_P = 128, TM_O = 192;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem;                                  // two buffers
    uint8_t *sK = sQ + 2 * TILE_BYTES;
    uint8_t *sV = sK + STAGES * TILE_BYTES;
    __shared__ uint64_t q_full[2], q_empty[2], k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
    __shared__ uint64_t s_full, s_free, p_ready, o_done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = p.nqb * p.BH;

    // One item: query block qb of (batch, head) pair bh, in the same order as the one-item-per-CTA form.
    struct Item { int bh, b, h, row0, n_t, kv_limit; bool uniform; };
    auto decode = [&](int item) -> Item {
        Item w;
        const int per_group = p.nqb * AT_HEAD_GROUP;
        const int group = item / per_group;
        const int r = item - group * per_group;
        const int gsize = min(AT_HEAD_GROUP, p.BH - group * AT_HEAD_GROUP);
        const int qb = p.nqb - 1 - r / gsize;
        w.bh = group * AT_HEAD_GROUP + r % gsize;
        w.b = w.bh / (int)p.H;
        w.h = w.bh % (int)p.H;
        int len = p.lens ? p.lens[w.b] : p.Sk;
        if (len > p.Sk) len = p.Sk;
        w.uniform = len <= 0;                    // every key blocked: equal weights over all Sk keys
        w.kv_limit = w.uniform ? p.Sk : len;
        w.row0 = qb * AT_TILE;
        w.n_t = (w.kv_limit + AT_TILE - 1) / AT_TILE;   // >= 1: Sk >= 1 and row0 < Sq by construction of the grid
        return w;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        mbar_init(&s_full, 1); mbar_init(&s_free, 128); mbar_init(&p_ready, 128); mbar_init(&o_done, 1);
        abort_s = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA) { tmem_alloc(&tmem_base_s, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    if (warp >= 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == W_TMA) {
            // ------------------------------------------------------------ TMA producer
            if (elect_one()) {
                tma_prefetch_desc(&tmap_q);
                tma_prefetch_desc(&tmap_k);
                tma_prefetch_desc(&tmap_v);
                uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
                bool ok = true;
                for (int it = 0, item = blockIdx.x; ok && item < total; ++it, item += gridDim.x) {
                    const Item w = decode(item);
                    const int qbuf = it & 1;
                    // the buffer's previous user (item it-2) has issued its last Q K^T
                    if (!(ok = mbar_wait(&q_empty[qbuf], ((it >> 1) & 1) ^ 1, abort_flag))) break;
                    mbar_expect_tx(&q_full[qbuf], TILE_BYTES);
                    tma_load_3d(sQ + qbuf * TILE_BYTES, &tmap_q, &q_full[qbuf], 0, w.row0, w.bh);
                    for (int j = 0; j < w.n_t; ++j) {
                        if (!(ok = mbar_wait(&k_empty[ks], kph ^ 1, abort_flag))) break;
                        mbar_expect_tx(&k_full[ks], TILE_BYTES);
                        tma_load_3d(sK + ks * TILE_BYTES, &tmap_k, &k_full[ks], 0, j * AT_TILE, w.bh);
                        if (++ks == STAGES) { ks = 0; kph ^= 1; }
                        if (!(ok = mbar_wait(&v_empty[vs], vph ^ 1, abort_flag))) break;
                        mbar_expect_tx(&v_full[vs], TILE_BYTES);
                        tma_load_3d(sV + vs * TILE_BYTES, &tmap_v, &v_full[vs], 0, j * AT_TILE, w.bh);
                        if (++vs == STAGES) { vs = 0; vph ^= 1; }
                    }
                }
            }
        } else if (warp == W_MMA) {
            // -------------------------------------------------------------- MMA issuer
            if (elect_one()) {
                uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
                bool ok = true;
                // Two walks over this CTA's key tiles: `sc` is the tile whose scores are issued next (one ahead),
                // `pv` the tile whose P V is issued next.
                struct Walk { int it, item, j, n_t; };
                Walk sc{0, (int)blockIdx.x, 0, 0}, pv{0, (int)blockIdx.x, 0, 0};
                if (sc.item < total) sc.n_t = pv.n_t = decode(sc.item).n_t;
                auto advance = [&](Walk &w) {
                    if (++w.j == w.n_t) {
                        w.j = 0;
                        ++w.it;
                        w.item += (int)gridDim.x;
                        w.n_t = w.item < total ? decode(w.item).n_t : 0;
                    }
                };
                // Scores of tile `sc` (its K tile is next in the ring); false after a wait that gave up.
                auto issue_scores = [&]() -> bool {
                    const int qbuf = sc.it & 1;
                    if (sc.j == 0 && !mbar_wait(&q_full[qbuf], (sc.it >> 1) & 1, abort_flag)) return false;
                    if (!mbar_wait(&k_full[ks], kph, abort_flag)) return false;
                    tc_fence_after();
                    const uint32_t qbase = smem_u32(sQ + qbuf * TILE_BYTES), kbase = smem_u32(sK + ks * TILE_BYTES);
#pragma unroll
                    for (int k16 = 0; k16 < D / 16; ++k16)
                        umma_ss(tmem_base + TM_S, smem_desc_sw128(qbase + k16 * 32, 16, 1024),
                                smem_desc_sw128(kbase + k16 * 32, 16, 1024), IDESC_S, k16 != 0);
                    umma_commit(&s_full);
                    umma_commit(&k_empty[ks]);
                    if (++ks == STAGES) { ks = 0; kph ^= 1; }
                    if (sc.j == sc.n_t - 1) umma_commit(&q_empty[qbuf]);   // the item's last use of Q
                    advance(sc);
                    return true;
                };
                if (sc.item < total) ok = issue_scores();
                for (uint32_t g = 0; ok && pv.item < total; ++g) {
                    // the next tile's scores go in front of this tile's P V, once the softmax warps have read S_g
                    if (sc.item < total) {
                        if (!(ok = mbar_wait(&s_free, g & 1, abort_flag))) break;
                        if (!(ok = issue_scores())) break;
                    }
                    if (!(ok = mbar_wait(&v_full[vs], vph, abort_flag))) break;
                    const uint32_t vbase = smem_u32(sV + vs * TILE_BYTES);
                    if (!(ok = mbar_wait(&p_ready, g & 1, abort_flag))) break;
                    tc_fence_after();
#pragma unroll
                    for (int k16 = 0; k16 < AT_TILE / 16; ++k16)
                        umma_ts(tmem_base + TM_O, tmem_base + TM_P + k16 * 8, smem_desc_mn_sw128(vbase + k16 * 2048, TILE_BYTES, 1024),
                                IDESC_O, (pv.j | k16) != 0);
                    umma_commit(&o_done);
                    umma_commit(&v_empty[vs]);
                    if (++vs == STAGES) { vs = 0; vph ^= 1; }
                    advance(pv);
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        // ------------------------------------------------- softmax, one query row per thread
        const int quarter = warp & 3;
        const int r_local = quarter * 32 + lane;
        const uint32_t tm_s = tmem_addr(tmem_base, quarter * 32, TM_S);
        const uint32_t tm_p = tmem_addr(tmem_base, quarter * 32, TM_P);
        const uint32_t tm_o = tmem_addr(tmem_base, quarter * 32, TM_O);
        uint32_t g = 0;          // this CTA's key tiles so far: phase of s_full / s_free / p_ready, and of o_done one behind
        bool ok = true;
        for (int it = 0, item = blockIdx.x; ok && item < total; ++it, item += gridDim.x) {
            const Item w = decode(item);
            const int row = w.row0 + r_local;
            float m_used = -INFINITY, l_sum = 0.f;
            for (int j = 0; j < w.n_t; ++j, ++g) {
                if (!(ok = mbar_wait(&s_full, g & 1, abort_flag))) break;
                tc_fence_after();
                uint32_t r[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, r[c]);
                tmem_wait_ld();
                // the scores are in registers: the next tile's may be written
                tc_fence_before();
                mbar_arrive(&s_free);
                const int limit = w.kv_limit - j * AT_TILE;   // columns at or beyond it are blocked in this tile
                if (w.uniform) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[c][i] = 0u;   // all scores equal
                }
                if (limit < AT_TILE) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i >= limit) r[c][i] = 0xff800000u;   // -inf
                }
                float mc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    mc[c] = fmaxf(__uint_as_float(r[c][0]), __uint_as_float(r[c][1]));
#pragma unroll
                    for (int i = 2; i < 32; i += 2) mc[c] = max3(mc[c], __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                }
                const float mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
                // Lazy rescale, as in the one-item form: only when the row max has grown by more than 2^8.
                float alpha = 1.0f;
                const bool need = mx > m_used + 8.0f;
                if (need) {
                    alpha = fast_exp2(m_used - mx);
                    m_used = mx;
                    l_sum *= alpha;
                }
                const uint64_t negm2 = pack2(-m_used, -m_used);
                uint64_t acc0 = pack2(0.f, 0.f), acc1 = acc0;
                uint32_t pk[4][16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        uint64_t x2 = add2(pack2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), negm2);
                        float p0, p1, x0, x1;
                        unpack2(x2, x0, x1);
                        p0 = fast_exp2(x0);
                        p1 = fast_exp2(x1);
                        if (i & 1) acc1 = add2(acc1, pack2(p0, p1));
                        else acc0 = add2(acc0, pack2(p0, p1));
                        pk[c][i] = pack_half2(p0, p1);
                    }
                }
                {
                    float a, b2;
                    unpack2(add2(acc0, acc1), a, b2);
                    l_sum += a + b2;
                }
                // P_{g-1} V_{g-1} must have finished with the P columns (and with O, if it is rescaled) before they
                // are written again. Within an item that is o_done of the tile before; across items the previous
                // item's output pass has already waited for it.
                if (j > 0) {
                    if (!(ok = mbar_wait(&o_done, (g - 1) & 1, abort_flag))) break;
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld32(tm_o + c * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tm_o + c * 32, o);
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_st16(tm_p + c * 16, pk[c]);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&p_ready);
            }
            if (!ok) break;
            // O / l for this item; the next item's first scores are already in tensor memory or on their way.
            if (!(ok = mbar_wait(&o_done, (g - 1) & 1, abort_flag))) break;
            tc_fence_after();
            const float inv_l = 1.0f / l_sum;
            if (p.lse && row < p.Sq) p.lse[(int64_t)w.bh * p.Sq + row] = m_used + log2f(l_sum);
            const int64_t ooff = (int64_t)w.b * p.os.b + (int64_t)w.h * p.os.h + (int64_t)row * p.os.s;
            float *orow = reinterpret_cast<float *>(p.o) + ooff;
            __half *hrow = reinterpret_cast<__half *>(p.o) + ooff;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tm_o + c * 32, o);
                tmem_wait_ld();
                if (row < p.Sq) {
                    if (p.o_half) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 pk4;
                            pk4.x = pack_half2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
                            pk4.y = pack_half2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                            pk4.z = pack_half2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
                            pk4.w = pack_half2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
                            *reinterpret_cast<uint4 *>(hrow + c * 32 + i) = pk4;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4 *>(orow + c * 32 + i) =
                                make_float4(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l,
                                            __uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                    }
                }
            }
            // O is written again by the next item's first P V, which waits for this thread's next p_ready.
            tc_fence_before();
        }
    }

    // Common exit, also reached after a wait that gave up.
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_s) atomicOr(p.status, kStatusAttnTimeout);
    if (warp == W_MMA) tmem_dealloc(tmem_base, TMEM_COLS);
}

bool attn_prefill_tc_supported(int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    return dk == dv && (dk == 64 || dk == 128) && Sq >= 1 && Sk >= 1 && Sq < (1 << 30) && Sk < (1 << 30);
}

size_t attn_prefill_tc_scratch_bytes(int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    return align_up((size_t)(B * H * Sq * dk) * 2, 1024) + align_up((size_t)(B * H * Sk * dk) * 2, 1024) +
           align_up((size_t)(B * H * Sk * dv) * 2, 1024);
}

template <int D, int NT>
static dl4s_status run_attn_tc(DeviceState *st, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                               const AttnTcParams &p, int64_t BH)
{
    constexpr int stages = at_stages(D, NT);
    constexpr size_t tile = (size_t)AT_TILE * D * 2;
    constexpr size_t smem = NT * tile + 2 * stages * tile + 1024;
    static bool attr_set[kMaxDevices] = {false};
    if (!attr_set[st->ordinal]) {
        DL4S_CUDA_TRY(cudaFuncSetAttribute(k_attn_prefill_tc<D, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[st->ordinal] = true;
    }
    DL4S_REQUIRE((int64_t)p.nqb * BH < (1ll << 31), "too many query blocks for one grid");
    AttnTcParams pp = p;
    pp.BH = (int)BH;
    DL4S_CUDA_TRY(launch_pdl(st, k_attn_prefill_tc<D, NT>, dim3((unsigned)(p.nqb * BH)), dim3(at_threads(NT)), smem, 1, tq, tk, tv, pp));
    return after_launch(st, "k_attn_prefill_tc");
}

dl4s_status launch_attn_prefill_tc(DeviceState *st, const float *q, Strides4 qs, const float *k, Strides4 ks, const float *v,
                                   Strides4 vs, float *o, Strides4 os, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t dk,
                                   int64_t dv, float inv_temperature, const MaskSpec &mask, void *scratch, size_t scratch_bytes)
{
    DL4S_REQUIRE(attn_prefill_tc_supported(Sq, Sk, dk, dv), "shape not supported by the tensor-core attention");
    DL4S_REQUIRE(!mask.d_mask, "dense masks are not supported by the tensor-core attention");
    DL4S_REQUIRE(scratch && scratch_bytes >= attn_prefill_tc_scratch_bytes(B, H, Sq, Sk, dk, dv), "scratch too small");
    DL4S_REQUIRE(B * H <= 65535, "B*H exceeds the grid limit");
    const int64_t BH = B * H;
    if (BH == 0 || Sq == 0) return DL4S_OK;
    auto ok16 = [](const float *ptr, Strides4 s) {
        return (((uintptr_t)ptr & 15) == 0) && s.b % 4 == 0 && s.h % 4 == 0 && s.s % 4 == 0;
    };
    DL4S_REQUIRE(ok16(q, qs) && ok16(k, ks) && ok16(v, vs) && ok16(o, os), "attention operands must be 16-byte aligned");
    const int D = (int)dk;
    __half *qh = (__half *)scratch;
    __half *kh = (__half *)((char *)qh + align_up((size_t)(BH * Sq * D) * 2, 1024));
    __half *vh = (__half *)((char *)kh + align_up((size_t)(BH * Sk * D) * 2, 1024));
    auto pack = [&](const float *src, Strides4 ss, __half *dst, int64_t S, float scale) -> dl4s_status {
        return pack_heads_f16(st, src, ss, dst, BH, H, S, D, scale);
    };
    DL4S_TRY(pack(q, qs, qh, Sq, inv_temperature * kLog2e));
    DL4S_TRY(pack(k, ks, kh, Sk, 1.0f));
    DL4S_TRY(pack(v, vs, vh, Sk, 1.0f));
    return launch_attn_prefill_tc_h(st, qh, kh, vh, o, os, 0, B, H, Sq, Sk, D, mask);
}

float attn_prefill_tc_q_scale(float inv_temperature) { return inv_temperature * kLog2e; }

dl4s_status launch_attn_prefill_tc_h(DeviceState *st, const void *qh, const void *kh, const void *vh, void *o, Strides4 os,
                                     int o_half, int64_t B, int64_t H, int64_t Sq, int64_t Sk, int64_t D, const MaskSpec &mask,
                                     float *lse)
{
    DL4S_REQUIRE(attn_prefill_tc_supported(Sq, Sk, D, D), "shape not supported by the tensor-core attention");
    DL4S_REQUIRE(!mask.d_mask, "dense masks are not supported by the tensor-core attention");
    DL4S_REQUIRE(B * H <= 65535, "B*H exceeds the grid limit");
    const int64_t BH = B * H;
    if (BH == 0 || Sq == 0) return DL4S_OK;
    const int64_t oal = o_half ? 8 : 4;   // elements per 16 bytes
    DL4S_REQUIRE(((uintptr_t)o & 15) == 0 && os.b % oal == 0 && os.h % oal == 0 && os.s % oal == 0,
                 "attention output must be 16-byte aligned");
    CUtensorMap tq, tk, tv;
    DL4S_TRY(make_tmap_f16(&tq, qh, (uint64_t)D, (uint64_t)Sq, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sq * D * 2, 64, AT_TILE));
    DL4S_TRY(make_tmap_f16(&tk, kh, (uint64_t)D, (uint64_t)Sk, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sk * D * 2, 64, AT_TILE));
    DL4S_TRY(make_tmap_f16(&tv, vh, (uint64_t)D, (uint64_t)Sk, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sk * D * 2, 64, AT_TILE));
    AttnTcParams p;
    p.o = o; p.o_half = o_half; p.os = os; p.H = H;
    p.Sq = (int)Sq; p.Sk = (int)Sk;
    p.lens = mask.d_key_lengths;
    p.causal = mask.causal;
    p.status = st->status_word;
    p.lse = lse;
    if (D == 128) {
        p.nqb = (int)ceil_div(Sq, 2 * AT_TILE);
        return run_attn_tc<128, 2>(st, tq, tk, tv, p, BH);
    }
    // 64-wide heads: the softmax is bound by the exp2 unit (16 per clock per SM against 128 x 128 per key tile),
    // the MMAs take half that time, and a short sequence leaves a CTA few key tiles to hide its start and its
    // output pass behind. One query tile per CTA and two CTAs per SM: each CTA's serial parts run under the
    // other's softmax.
    p.nqb = (int)ceil_div(Sq, AT_TILE);
    if (!mask.causal) {
        // every item of a (batch, head) pair costs the same: resident CTAs with a fixed round-robin share
        constexpr size_t smem = (size_t)6 * AT_TILE * 128 + 1024;
        static bool attr_set[kMaxDevices] = {false};
        if (!attr_set[st->ordinal]) {
            DL4S_CUDA_TRY(cudaFuncSetAttribute(k_attn_prefill_tc_loop<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set[st->ordinal] = true;
        }
        DL4S_REQUIRE((int64_t)p.nqb * BH < (1ll << 31), "too many query blocks for one grid");
        p.BH = (int)BH;
        const int64_t items = (int64_t)p.nqb * BH, resident = 2 * (int64_t)st->sm_count;
        DL4S_CUDA_TRY(launch_pdl(st, k_attn_prefill_tc_loop<64>, dim3((unsigned)(items < resident ? items : resident)), dim3(256), smem, 1,
                                 tq, tk, tv, p));
        return after_launch(st, "k_attn_prefill_tc_loop");
    }
    return run_attn_tc<64, 1>(st, tq, tk, tv, p, BH);
}

size_t tc_layer_scratch_bytes(int64_t B, int64_t S, int64_t D, int64_t H, int64_t dk, int64_t dv, int64_t F, int split)
{
    size_t m = 0;
    auto upd = [&](size_t v) { if (v > m) m = v; };
    int64_t M = B * S;
    upd(gemm_tc_scratch_bytes(M, H * dk, D, split));
    upd(gemm_tc_scratch_bytes(M, H * dv, D, split));
    upd(gemm_tc_scratch_bytes(M, D, H * dv, split));
    upd(attn_prefill_tc_scratch_bytes(B, H, S, S, dk, dv));
    if (F > 0) { upd(gemm_tc_scratch_bytes(M, F, D, split)); upd(gemm_tc_scratch_bytes(M, D, F, split)); }
    return m;
}

}  // namespace dl4s
