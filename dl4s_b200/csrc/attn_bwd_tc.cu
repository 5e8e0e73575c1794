// Flash-style backward of scaled-dot-product attention on the sm_100a tensor cores: the gradients DL4S's
// autograd obtains by chaining the backward closures of mmul (Tensor/Operators/Matrix.swift:139-173), of the
// softmax composition (Unary.swift:190-194) and of the division by the temperature
// (ScaledDotProductAttention.swift:53-63), without ever forming the [Sq,Sk] matrices:
//   P  = softmax((q / T) k^T - mask * 1e9)          recomputed tile by tile
//   dP = dout v^T,   dS = P * (dP - delta),  delta_i = sum_j P_ij dP_ij = dout_i . out_i
//   dv = P^T dout,   dk = dS^T (q / T),      dq = (dS k) / T
// Preparation (host side of this file): q (pre-multiplied by log2(e)/T), k, v and dout are packed as half
// [B*H, S, D]; the forward kernel runs once for out and for the log2 of every row's softmax denominator;
// k_attn_bwd_delta forms delta. The main kernel gives one CTA one tile of 128 KEYS of one (batch, head) pair
// and walks the query tiles that see it (with the causal mask: from the diagonal on):
//   warp 4    TMA producer: K_j and V_j once, then Q_i and dout_i per query tile (128-byte swizzle);
//   warp 5    MMA issuer, five products per query tile, fp32 accumulation in tensor memory:
//               S  = Q_i K_j^T          (both K-major)            columns [0,128)
//               dP = dout_i V_j^T       (both K-major)            columns [128,256)
//               dV += P^T dout_i        (A = P as MN-major, B = dout MN-major)     [256, 256+D)
//               dK += dS^T Q_i          (A = dS as MN-major, B = Q MN-major)       [256+D, 256+2D)
//               dQ  = dS K_j            (A = dS K-major, B = K_j MN-major)         D = 64: [384,448); D = 128: [0,128)
//             (with 128-wide heads dQ takes the columns of S, which the softmax warps have consumed by then);
//   warps 0-3 one thread per query row: reads S and dP 32 columns at a time (tcgen05.ld), forms
//             p = 2^(s - lse) (0 where the mask blocks) and dS = p (dP - delta), writes both as halves into two
//             swizzled shared-memory tiles [128 queries x 128 keys] that serve as the A operands above in both
//             orientations; afterwards drains dQ and adds it into global memory (red.global.add.v4.f32: the
//             key tiles of a head contribute to the same dq rows). dV and dK are owned by the CTA and stored
//             once at the end.
// The sum of a dq row over the key tiles is taken by atomic adds, so its rounding can differ from run to run in
// the last bits; dk and dv are summed in a fixed order. One tile pair runs as a dependent chain (scores, softmax,
// three products, dQ drain): the kernel is a first tensor-core form (about a third of the MMA rate is used);
// Q/dout of the next query tile are prefetched under it.
// A sequence of length 0 follows the reference's finite -1e9 (uniform weights over all keys, gradients flow).
// Every mbarrier wait is bounded (status word + common exit on expiry).
#include "tc.cuh"
#include "tc_device.cuh"

namespace dl4s {

using namespace tc;

constexpr int BW_TILE = 128;
constexpr int BW_THREADS = 192;   // warps 0-3 softmax, 4 TMA, 5 MMA
constexpr float kBwLog2e = 1.4426950408889634f;
constexpr float kBwLn2 = 0.6931471805599453f;

struct AttnBwdTcParams {
    const float *lse;      // [BH, Sq] log2 of the softmax denominator (base-2 score units)
    const float *delta;    // [BH, Sq]
    float *dq, *dk, *dv;   // [BH, S, D] fp32; dq zero-filled before the launch
    int64_t H;
    int Sq, Sk;
    const int32_t *lens;
    int causal;
    int nkb;               // key tiles
    float inv_t;
    int32_t *status;
    uint32_t wait_polls;   // poll limit of every bounded wait
};

// Where a bounded wait gave up (bits 16-19 of the status word, beside the time-out bit): the first role to give up records it.
enum { BW_SITE_TMA_STAGE = 1, BW_SITE_MMA_KV = 2, BW_SITE_MMA_QG = 3, BW_SITE_MMA_DQFREE = 4, BW_SITE_MMA_PDS = 5, BW_SITE_SM_SDP = 6,
       BW_SITE_SM_MMDONE = 7 };

__device__ __forceinline__ float bw_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t bw_pack_half2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int D>
__global__ void __launch_bounds__(BW_THREADS, 1) k_attn_bwd_tc(const __grid_constant__ CUtensorMap tmap_q,
                                                               const __grid_constant__ CUtensorMap tmap_k,
                                                               const __grid_constant__ CUtensorMap tmap_v,
                                                               const __grid_constant__ CUtensorMap tmap_g, AttnBwdTcParams p)
{
    constexpr int NBLK = D / 64;
    constexpr uint32_t BLK_BYTES = BW_TILE * 128;          // 128 rows x 128 bytes
    constexpr uint32_t TILE_BYTES = BLK_BYTES * NBLK;      // a [128, D] half tile
    constexpr uint32_t PS_BYTES = BLK_BYTES * 2;           // a [128, 128] half tile (P or dS)
    constexpr int QSTAGES = D == 64 ? 2 : 1;
    constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + D, TM_DQ = D == 64 ? 384 : 0;
    constexpr uint32_t IDESC_S = idesc_f16(128, 128, 0, 0);    // Q K^T, dout V^T: both K-major
    constexpr uint32_t IDESC_T = idesc_f16(128, D, 1, 1);      // P^T dout, dS^T Q: A and B MN-major
    constexpr uint32_t IDESC_Q = idesc_f16(128, D, 0, 1);      // dS K: A K-major, B MN-major
    constexpr int W_TMA = 4, W_MMA = 5;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + TILE_BYTES;
    uint8_t *sQ = sV + TILE_BYTES;                       // QSTAGES tiles
    uint8_t *sG = sQ + QSTAGES * TILE_BYTES;             // QSTAGES tiles of dout
    uint8_t *sP = sG + QSTAGES * TILE_BYTES;
    uint8_t *sS = sP + PS_BYTES;                         // dS
    __shared__ uint64_t kv_full, qg_full[QSTAGES], qg_empty[QSTAGES], sdp_full, pds_ready, mm_done, dq_free;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, abort_site;

    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heaviest key tiles first: with the causal mask key tile 0 is seen by every query tile
    const int kb = (int)blockIdx.x % p.nkb;
    const int bh = (int)blockIdx.x / p.nkb;
    const int b = bh / (int)p.H;
    int len = p.lens ? p.lens[b] : p.Sk;
    if (len > p.Sk) len = p.Sk;
    const bool uniform = len <= 0;
    const int kv_limit = uniform ? p.Sk : len;
    const int key0 = kb * BW_TILE;
    const int n_qt = (p.Sq + BW_TILE - 1) / BW_TILE;
    const int i_begin = (p.causal && !uniform) ? kb : 0;
    // a key tile at or beyond the length has no weight anywhere: its gradients are zero
    const int n_iter = key0 < kv_limit ? max(n_qt - i_begin, 0) : 0;

    if (threadIdx.x == 0) {
        mbar_init(&kv_full, 1);
        for (int s = 0; s < QSTAGES; ++s) { mbar_init(&qg_full[s], 1); mbar_init(&qg_empty[s], 1); }
        mbar_init(&sdp_full, 1);
        mbar_init(&pds_ready, 128);
        mbar_init(&mm_done, 1);
        mbar_init(&dq_free, 128);
        abort_s = 0;
        abort_site = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    volatile int *abort_flag = &abort_s;
    // a wait that gives up notes where (first one wins)
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) -> bool {
        if (mbar_wait(bar, parity, abort_flag, p.wait_polls)) return true;
        atomicCAS(&abort_site, 0, site);
        return false;
    };

    if (warp == W_TMA) {
        if (elect_one() && n_iter > 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            tma_prefetch_desc(&tmap_g);
            mbar_expect_tx(&kv_full, 2 * TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                tma_load_3d(sK + blk * BLK_BYTES, &tmap_k, &kv_full, blk * 64, key0, bh);
                tma_load_3d(sV + blk * BLK_BYTES, &tmap_v, &kv_full, blk * 64, key0, bh);
            }
            uint32_t st = 0, ph = 0;
            for (int it = 0; it < n_iter; ++it) {
                const int row0 = (i_begin + it) * BW_TILE;
                if (!wait(&qg_empty[st], ph ^ 1, BW_SITE_TMA_STAGE)) break;
                mbar_expect_tx(&qg_full[st], 2 * TILE_BYTES);
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk) {
                    tma_load_3d(sQ + st * TILE_BYTES + blk * BLK_BYTES, &tmap_q, &qg_full[st], blk * 64, row0, bh);
                    tma_load_3d(sG + st * TILE_BYTES + blk * BLK_BYTES, &tmap_g, &qg_full[st], blk * 64, row0, bh);
                }
                if (++st == QSTAGES) { st = 0; ph ^= 1; }
            }
        }
    } else if (warp == W_MMA) {
        if (elect_one() && n_iter > 0) {
            const uint32_t kbase = smem_u32(sK), vbase = smem_u32(sV), pbase = smem_u32(sP), sbase = smem_u32(sS);
            bool ok = wait(&kv_full, 0, BW_SITE_MMA_KV);
            uint32_t st = 0, ph = 0;
            for (int it = 0; it < n_iter && ok; ++it) {
                if (!(ok = wait(&qg_full[st], ph, BW_SITE_MMA_QG))) break;
                // the softmax warps have consumed the previous S, dP and dQ
                if (it > 0 && !(ok = wait(&dq_free, (it - 1) & 1, BW_SITE_MMA_DQFREE))) break;
                tc_fence_after();
                const uint32_t qbase = smem_u32(sQ + st * TILE_BYTES), gbase = smem_u32(sG + st * TILE_BYTES);
#pragma unroll
                for (int k16 = 0; k16 < D / 16; ++k16) {
                    const uint32_t off = (k16 / 4) * BLK_BYTES + (k16 % 4) * 32;
                    umma_ss(tmem_base + TM_S, smem_desc_sw128(qbase + off, 16, 1024), smem_desc_sw128(kbase + off, 16, 1024), IDESC_S,
                            k16 != 0);
                }
#pragma unroll
                for (int k16 = 0; k16 < D / 16; ++k16) {
                    const uint32_t off = (k16 / 4) * BLK_BYTES + (k16 % 4) * 32;
                    umma_ss(tmem_base + TM_DP, smem_desc_sw128(gbase + off, 16, 1024), smem_desc_sw128(vbase + off, 16, 1024), IDESC_S,
                            k16 != 0);
                }
                umma_commit(&sdp_full);
                // P and dS of this tile pair are in shared memory
                if (!(ok = wait(&pds_ready, it & 1, BW_SITE_MMA_PDS))) break;
                tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < BW_TILE / 16; ++k16) {   // k runs over the 128 queries
                    umma_ss(tmem_base + TM_DV, smem_desc_mn_sw128(pbase + k16 * 2048, BLK_BYTES, 1024),
                            smem_desc_mn_sw128(gbase + k16 * 2048, BLK_BYTES, 1024), IDESC_T, (it | k16) != 0);
                }
#pragma unroll
                for (int k16 = 0; k16 < BW_TILE / 16; ++k16) {
                    umma_ss(tmem_base + TM_DK, smem_desc_mn_sw128(sbase + k16 * 2048, BLK_BYTES, 1024),
                            smem_desc_mn_sw128(qbase + k16 * 2048, BLK_BYTES, 1024), IDESC_T, (it | k16) != 0);
                }
#pragma unroll
                for (int k16 = 0; k16 < BW_TILE / 16; ++k16) {   // k runs over the 128 keys
                    const uint32_t off = (k16 / 4) * BLK_BYTES + (k16 % 4) * 32;
                    umma_ss(tmem_base + TM_DQ, smem_desc_sw128(sbase + off, 16, 1024),
                            smem_desc_mn_sw128(kbase + k16 * 2048, BLK_BYTES, 1024), IDESC_Q, k16 != 0);
                }
                umma_commit(&qg_empty[st]);   // Q_i and dout_i are no longer read
                umma_commit(&mm_done);
                if (++st == QSTAGES) { st = 0; ph ^= 1; }
            }
        }
    } else {
        // ---------------------------------------------------------------- one query row per thread
        const int quarter = warp;                       // warps 0-3: tensor-memory lanes 32 w .. 32 w + 31
        const int r_local = quarter * 32 + lane;
        const uint32_t tm_row = tmem_addr(tmem_base, quarter * 32, 0);
        bool ok = true;
        for (int it = 0; it < n_iter; ++it) {
            const int qrow = (i_begin + it) * BW_TILE + r_local;
            const bool row_ok = qrow < p.Sq;
            // rows past the end carry lse = +inf: their probabilities are exactly zero
            const float lse = row_ok ? p.lse[(int64_t)bh * p.Sq + qrow] : INFINITY;
            const float delta = row_ok ? p.delta[(int64_t)bh * p.Sq + qrow] : 0.f;
            // keys at or beyond `limit` (relative to this key tile) are blocked for this row
            int limit = kv_limit - key0;
            if (p.causal && !uniform) limit = min(limit, qrow - key0 + 1);
            // (the tensor-memory loads below are warp-collective: the whole warp leaves the loop together)
            ok = __all_sync(0xffffffffu, wait(&sdp_full, it & 1, BW_SITE_SM_SDP));
            if (!ok) break;
            // P/dS tiles of the previous pair are no longer read by the tensor core (the same wait that lets dQ be drained)
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t s[32], g[32];
                tmem_ld32(tm_row + TM_S + c * 32, s);
                tmem_ld32(tm_row + TM_DP + c * 32, g);
                tmem_wait_ld();
                uint32_t pk[16], dk2[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float pv[2], dv2[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = c * 32 + 2 * i + e;
                        const float sc = uniform ? 0.f : __uint_as_float(s[2 * i + e]);
                        const float pe = col < limit ? bw_exp2(sc - lse) : 0.f;
                        pv[e] = pe;
                        dv2[e] = pe * (__uint_as_float(g[2 * i + e]) - delta);
                    }
                    pk[i] = bw_pack_half2(pv[0], pv[1]);
                    dk2[i] = bw_pack_half2(dv2[0], dv2[1]);
                }
                // 32 columns = 64 bytes of this row in each tile: four 16-byte units, xor-swizzled with the row
                const uint32_t rowoff = (uint32_t)(c >> 1) * BLK_BYTES + (uint32_t)r_local * 128u;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t unit = ((uint32_t)((c & 1) * 4 + u) ^ ((uint32_t)r_local & 7u)) << 4;
                    *reinterpret_cast<uint4 *>(sP + rowoff + unit) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
                    *reinterpret_cast<uint4 *>(sS + rowoff + unit) = make_uint4(dk2[4 * u], dk2[4 * u + 1], dk2[4 * u + 2], dk2[4 * u + 3]);
                }
            }
            fence_proxy_async();     // the tensor core reads these tiles through the async proxy
            tc_fence_before();
            mbar_arrive(&pds_ready);
            // dQ of this pair: add into the rows of dq (other key tiles of the head add to the same rows)
            ok = __all_sync(0xffffffffu, wait(&mm_done, it & 1, BW_SITE_SM_MMDONE));
            if (!ok) break;
            tc_fence_after();
            float *dqrow = p.dq + ((int64_t)bh * p.Sq + qrow) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tm_row + TM_DQ + c * 32, o);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        red_add_v4(dqrow + c * 32 + i, __uint_as_float(o[i]) * p.inv_t, __uint_as_float(o[i + 1]) * p.inv_t,
                                   __uint_as_float(o[i + 2]) * p.inv_t, __uint_as_float(o[i + 3]) * p.inv_t);
                }
            }
            tc_fence_before();
            mbar_arrive(&dq_free);
        }
        // dV and dK of this key tile: one key row per thread. tcgen05.ld is warp-collective, so every lane of a warp
        // takes part in the loads and only the stores depend on whether the lane's key exists.
        const int key = key0 + r_local;
        const bool key_ok = key < p.Sk;
        float *dvrow = p.dv + ((int64_t)bh * p.Sk + key) * D;
        float *dkrow = p.dk + ((int64_t)bh * p.Sk + key) * D;
        if (n_iter == 0) {
            if (key_ok) {
                for (int i = 0; i < D; i += 4) {
                    *reinterpret_cast<float4 *>(dvrow + i) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4 *>(dkrow + i) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        } else if (ok) {   // warp-uniform: n_iter is per CTA, ok was agreed on by the warp
            // the last mm_done wait above covers the final accumulation
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tm_row + TM_DV + c * 32, o);
                tmem_wait_ld();
                if (key_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(dvrow + c * 32 + i) =
                            make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
                }
                tmem_ld32(tm_row + TM_DK + c * 32, o);
                tmem_wait_ld();
                // the query operand carried log2(e)/T: dk = dS^T (q / T) = (dS^T qh) * ln 2
                if (key_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(dkrow + c * 32 + i) =
                            make_float4(__uint_as_float(o[i]) * kBwLn2, __uint_as_float(o[i + 1]) * kBwLn2,
                                        __uint_as_float(o[i + 2]) * kBwLn2, __uint_as_float(o[i + 3]) * kBwLn2);
                }
            }
        }
    }

    // Common exit, also reached after a wait that gave up.
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && abort_s) atomicOr(p.status, kStatusAttnTimeout | (abort_site << 16));
    if (warp == W_MMA) tmem_dealloc(tmem_base, 512);
}

// delta[bh, row] = dout_row . out_row (one warp per row), D = 64 or 128.
__global__ void __launch_bounds__(256) k_attn_bwd_delta(const float *__restrict__ g, const float *__restrict__ o, float *__restrict__ delta,
                                                        int64_t rows, int D)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t row = (int64_t)blockIdx.x * 8 + warp; row < rows; row += (int64_t)gridDim.x * 8) {
        const float4 *gp = reinterpret_cast<const float4 *>(g + row * D);
        const float4 *op = reinterpret_cast<const float4 *>(o + row * D);
        float s = 0.f;
        for (int i = lane; i < D / 4; i += 32) {
            const float4 a = gp[i], b2 = op[i];
            s = fmaf(a.x, b2.x, s); s = fmaf(a.y, b2.y, s); s = fmaf(a.z, b2.z, s); s = fmaf(a.w, b2.w, s);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) delta[row] = s;
    }
}

bool attn_bwd_tc_supported(int64_t Sq, int64_t Sk, int64_t dk, int64_t dv)
{
    return attn_prefill_tc_supported(Sq, Sk, dk, dv);
}

template <int D>
static dl4s_status run_attn_bwd_tc(DeviceState *st, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                                   const CUtensorMap &tg, const AttnBwdTcParams &p, int64_t BH)
{
    constexpr size_t tile = (size_t)BW_TILE * D * 2;
    constexpr int qstages = D == 64 ? 2 : 1;
    constexpr size_t smem = 2 * tile + 2 * qstages * tile + 2 * (size_t)BW_TILE * 128 * 2 + 1024;
    static bool attr_set[kMaxDevices] = {false};
    if (!attr_set[st->ordinal]) {
        DL4S_CUDA_TRY(cudaFuncSetAttribute(k_attn_bwd_tc<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[st->ordinal] = true;
    }
    DL4S_REQUIRE((int64_t)p.nkb * BH < (1ll << 31), "too many key tiles for one grid");
    DL4S_CUDA_TRY(launch_pdl(st, k_attn_bwd_tc<D>, dim3((unsigned)(p.nkb * BH)), dim3(BW_THREADS), smem, 1, tq, tk, tv, tg, p));
    return after_launch(st, "k_attn_bwd_tc");
}

dl4s_status launch_attn_bwd_tc(DeviceState *st, const float *q, const float *k, const float *v, const float *dout, int64_t B, int64_t H,
                               int64_t Sq, int64_t Sk, int64_t D, float inv_temperature, const MaskSpec &mask, float *dq, float *dk,
                               float *dv)
{
    DL4S_REQUIRE(attn_bwd_tc_supported(Sq, Sk, D, D), "shape not supported by the tensor-core attention backward");
    DL4S_REQUIRE(!mask.d_mask, "dense masks are not supported by the tensor-core attention backward");
    const int64_t BH = B * H;
    if (BH == 0) return DL4S_OK;
    DL4S_REQUIRE(BH <= 65535, "B*H exceeds the grid limit");
    DL4S_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 15) == 0,
                 "attention operands must be 16-byte aligned");
    // scratch: half q, k, v, dout; fp32 out; lse and delta per row
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes, 1024); return o; };
    const size_t o_q = take((size_t)(BH * Sq * D) * 2), o_k = take((size_t)(BH * Sk * D) * 2), o_v = take((size_t)(BH * Sk * D) * 2);
    const size_t o_g = take((size_t)(BH * Sq * D) * 2), o_o = take((size_t)(BH * Sq * D) * 4);
    const size_t o_lse = take((size_t)(BH * Sq) * 4), o_delta = take((size_t)(BH * Sq) * 4);
    void *base = nullptr;
    DL4S_TRY(arena_reserve(st, off, &base));
    char *w = static_cast<char *>(base);
    void *qh = w + o_q, *kh = w + o_k, *vh = w + o_v, *gh = w + o_g;
    float *out = (float *)(w + o_o), *lse = (float *)(w + o_lse), *delta = (float *)(w + o_delta);
    DL4S_TRY(pack_heads_f16(st, q, strides_bhsd(H, Sq, D), qh, BH, H, Sq, (int)D, inv_temperature * kBwLog2e));
    DL4S_TRY(pack_heads_f16(st, k, strides_bhsd(H, Sk, D), kh, BH, H, Sk, (int)D, 1.0f));
    DL4S_TRY(pack_heads_f16(st, v, strides_bhsd(H, Sk, D), vh, BH, H, Sk, (int)D, 1.0f));
    DL4S_TRY(pack_heads_f16(st, dout, strides_bhsd(H, Sq, D), gh, BH, H, Sq, (int)D, 1.0f));
    // the forward once more: out (for delta) and the softmax denominators
    DL4S_TRY(launch_attn_prefill_tc_h(st, qh, kh, vh, out, strides_bhsd(H, Sq, D), 0, B, H, Sq, Sk, D, mask, lse));
    {
        const int64_t rows = BH * Sq;
        int64_t blocks = ceil_div(rows, 8);
        const int64_t cap = (int64_t)st->sm_count * 16;
        if (blocks > cap) blocks = cap;
        k_attn_bwd_delta<<<(unsigned)blocks, 256, 0, st->stream>>>(dout, out, delta, rows, (int)D);
        DL4S_TRY(after_launch(st, "k_attn_bwd_delta"));
    }
    DL4S_CUDA_TRY(cudaMemsetAsync(dq, 0, (size_t)(BH * Sq * D) * sizeof(float), st->stream));
    CUtensorMap tq, tk, tv, tg;
    DL4S_TRY(make_tmap_f16(&tq, qh, (uint64_t)D, (uint64_t)Sq, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sq * D * 2, 64, BW_TILE));
    DL4S_TRY(make_tmap_f16(&tk, kh, (uint64_t)D, (uint64_t)Sk, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sk * D * 2, 64, BW_TILE));
    DL4S_TRY(make_tmap_f16(&tv, vh, (uint64_t)D, (uint64_t)Sk, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sk * D * 2, 64, BW_TILE));
    DL4S_TRY(make_tmap_f16(&tg, gh, (uint64_t)D, (uint64_t)Sq, (uint64_t)BH, (uint64_t)D * 2, (uint64_t)Sq * D * 2, 64, BW_TILE));
    AttnBwdTcParams p;
    p.lse = lse; p.delta = delta;
    p.dq = dq; p.dk = dk; p.dv = dv;
    p.H = H;
    p.Sq = (int)Sq; p.Sk = (int)Sk;
    p.lens = mask.d_key_lengths;
    p.causal = mask.causal;
    p.nkb = (int)ceil_div(Sk, BW_TILE);
    p.inv_t = inv_temperature;
    p.status = st->status_word;
    // The longest legitimate wait is a few tile loads and MMAs (microseconds); the limit is generous by orders of
    // magnitude and still ends a stuck launch within seconds.
    p.wait_polls = 1u << 18;
    if (D == 128) return run_attn_bwd_tc<128>(st, tq, tk, tv, tg, p, BH);
    return run_attn_bwd_tc<64>(st, tq, tk, tv, tg, p, BH);
}

}  // namespace dl4s
