// Tensor-core GEMM for the projections and the feed-forward block:
//   C[M,N] = A[M,K] B[K,N]  (+ bias / activation / residual epilogue), fp32 in and out.
// Used for Wq/Wk/Wv/Wo (MultiHeadAttention.swift:109-121) and the two Dense
// layers of PointwiseFeedForward.swift:74-78.
//
// Operands are rounded to half once by a conversion pass (A [M,K], B [K,N]); the
// MMA is tcgen05.mma kind::f16 with fp32 accumulation in tensor memory.
// One persistent CTA per SM works through 128 x BN output tiles:
//   warp 0    TMA producer: loads A [128 rows x 64 k] (K-major) and B
//             [64 k-rows x BN] (N contiguous = MN-major, BN/64 boxes) into a
//             ring of 192 KB (4 stages of 48 KB for 256-column tiles, 6 of 32 KB for
//             128-column tiles and for each CTA of a pair), 128-byte swizzle;
//   warp 1    MMA issuer: 4 MMAs (K = 16) per stage, commit frees the stage;
//             two accumulators in tensor memory so the next tile's main loop
//             overlaps the epilogue of the previous one;
//   warps 2.. epilogue (8 or 16 warps by flavour): 16-lane x 256-bit tensor-memory
//             loads, 32 columns at a time, whose register layout lets four lanes
//             store whole sectors of a row straight from registers; fused bias /
//             GeLU / residual / LayerNorm sums.
// Tile schedule. In short launches worker w (a CTA, or a pair) takes tiles w, w + workers, ...: every role works the
// sequence out by itself and nothing is handed around. In long launches (more than 16 tiles per worker), and while a
// collective's kernel shares the SMs (DeviceState::dynamic_tiles), the tiles after the first come from a device-wide
// counter instead, so a CTA that starts late or falls behind simply takes fewer; the producer then publishes each
// tile to the other warps (and the other CTA of a pair) through a small ring, one tile ahead of its loads.
// Tiles are numbered so that the ~148 tiles in flight form a block of 16 tile rows
// x ~9 tile columns: their A and B panels (tens of MB) stay in L2, where a
// column-major walk would stream all of A from HBM once per tile column.
// What bounds the single-CTA main loop: shared-memory bandwidth. Per k-block TMA writes 48 KB of operands and
// the tensor core reads them once (A 16 KB + B 32 KB): 96 KB against 128 bytes per clock = 750 cycles where the
// MMAs alone need 512; clock64 stamps show 750 cycles per k-block in the steady state. The two-CTA tiles below
// need 64 KB per k-block and CTA and run at 520-580.
// What bounds a tile at K = 512 (8 k-blocks) is not the main loop alone. With two accumulators the MMAs of tile
// i+2 wait for the drain of tile i, so a tile costs (main loop + hand-offs + time the accumulator is held) / 2.
// Three things shortened that chain (clock64 stamps per role, first pair of CTAs):
//   * hand-offs that publish no memory are relaxed arrives: a release arrive after the epilogue's global stores
//     (or after the producer's counter atomic) waits until those have been performed, 1000-3400 cycles that the
//     MMA thread then spent waiting for an accumulator or for a tile's first operands;
//   * the half-output flavours read their whole share of the accumulator into registers, hand it back, and only
//     then convert and store (the accumulator is held ~1000 cycles instead of ~5000);
//   * the first tile's loads are issued before anything else the producer does.
// After that the half-output flavours at K = 512 run their epilogue in ~5000-5500 cycles per tile against a
// 4300-cycle pair main loop (issue slots 46 % busy with 4 warps per scheduler, ~1000 instructions per warp and
// tile). Making the epilogue lighter (the score scale folded into Wq when it is rounded, the half-range check as a
// running maximum, fewer shuffles) moved the step by < 1 %, and two-CTA tiles at K = 512 by another 1 % in one mode
// and nothing in the other: single-CTA and two-CTA tiles run at practically the same rate there, and short
// products keep the single-CTA kernel.
// Every mbarrier wait is bounded; on expiry the kernel sets the device status
// word and unwinds through the common exit, which frees the tensor memory.
#include "tc.cuh"
#include "tc_device.cuh"


namespace dl4s {

using namespace tc;

constexpr int GM = 128;          // tile rows
constexpr int GK = 64;           // k per stage (one 128-byte swizzle row of halves)
// Epilogue warps: `parts` warps per tensor-memory lane quarter, each taking BN / parts columns of its 32 rows.
// Measured on the encoder's K = 512 products (per step): 16 warps (96 registers each) against 8 for
// feed-forward 1 (bias + GeLU, 2 MUFU per element) 0.269 vs 0.310 ms, for the q/k/v projection 0.210 either
// way, for the flavours that add a residual 0.448 vs 0.444 ms: those keep 8 warps, whose registers hold the
// prefetched residual values. Single-CTA and two-CTA tiles use the same count.
__host__ __device__ constexpr bool epi_has_residual(int epi) { return epi == EPI_BIAS_RESIDUAL || epi == EPI_RESIDUAL || epi == EPI_RESIDUAL_STATS; }
__host__ __device__ constexpr int epi_parts(int epi, int pair) { return epi_has_residual(epi) ? 2 : 4; }
__host__ __device__ constexpr int gemm_threads(int epi, int pair) { return 64 + 32 * 4 * epi_parts(epi, pair); }   // warp 0 TMA, warp 1 MMA, then the epilogue warps

// DL4S's GeLU, t * sigmoid(1.702 t) with sigmoid(y) = 0.5 tanh(y/2) + 0.5 (Unary.swift:184-186,
// 245-247), evaluated as t / (1 + 2^(-1.702 log2(e) t)): the same function, two fast-math
// instructions (ex2, rcp; relative error ~3e-7) instead of a tanhf call per element. The result is
// rounded to half (4.9e-4) right after, so the epilogue stays shorter than the tile's main loop.
__device__ __forceinline__ float gelu_sigmoid_tc(float t)
{
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t * -2.4554669595930157f));
    return __fdividef(t, 1.0f + e);
}

// max(m, |a|, |b|) in one instruction.
__device__ __forceinline__ float max3_abs(float m, float a, float b)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(m), "f"(fabsf(a)), "f"(fabsf(b)));
    return d;
}

// fp32 -> half, 8 elements per thread per step.
__global__ void __launch_bounds__(256) k_f32_to_f16(const float *__restrict__ x, __half *__restrict__ y, int64_t n, int32_t *status)
{
    pdl_launch_dependents();
    pdl_wait();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t n8 = n >> 3;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    uint4 *y8 = reinterpret_cast<uint4 *>(y);
    bool bad = false;   // a value outside the half range
    for (int64_t i = tid; i < n8; i += stride) {
        float4 a = x4[2 * i], b = x4[2 * i + 1];
        __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
        __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
        uint4 o;
        o.x = *reinterpret_cast<uint32_t *>(&h0);
        o.y = *reinterpret_cast<uint32_t *>(&h1);
        o.z = *reinterpret_cast<uint32_t *>(&h2);
        o.w = *reinterpret_cast<uint32_t *>(&h3);
        bad |= half2_not_finite(o.x) | half2_not_finite(o.y) | half2_not_finite(o.z) | half2_not_finite(o.w);
        y8[i] = o;
    }
    for (int64_t i = (n8 << 3) + tid; i < n; i += stride) {
        const __half hv = __float2half_rn(x[i]);
        bad |= half2_not_finite((uint32_t)__half_as_ushort(hv));
        y[i] = hv;
    }
    if (bad) atomicOr(status, kStatusHalfRange);
}

// fp32 -> two halves: hi = half(x), lo = half(x - hi), so that hi + lo carries 22 significant bits of x.
__global__ void __launch_bounds__(256) k_f32_to_f16_hilo(const float *__restrict__ x, __half *__restrict__ hi, __half *__restrict__ lo,
                                                         int64_t n, int32_t *status)
{
    pdl_launch_dependents();
    pdl_wait();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t n4 = n >> 2;
    bool bad = false;
    for (int64_t i = tid; i < n4; i += stride) {
        const float4 v = reinterpret_cast<const float4 *>(x)[i];
        uint2 ph, pl;
        split_hilo(v, ph, pl);
        bad |= half2_not_finite(ph.x) | half2_not_finite(ph.y);
        reinterpret_cast<uint2 *>(hi)[i] = ph;
        reinterpret_cast<uint2 *>(lo)[i] = pl;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
        const __half h = __float2half_rn(x[i]);
        bad |= half2_not_finite((uint32_t)__half_as_ushort(h));
        hi[i] = h;
        lo[i] = __float2half_rn(x[i] - __half2float(h));
    }
    if (bad) atomicOr(status, kStatusHalfRange);
}

dl4s_status launch_f32_to_f16_hilo(DeviceState *st, const float *x, void *hi, void *lo, int64_t n)
{
    if (n == 0) return DL4S_OK;
    DL4S_REQUIRE((((uintptr_t)x | (uintptr_t)hi | (uintptr_t)lo) & 15) == 0, "conversion buffers must be 16-byte aligned");
    int64_t blocks = ceil_div(n, 256 * 4 * 4);
    int64_t cap = (int64_t)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    DL4S_CUDA_TRY(launch_pdl(st, k_f32_to_f16_hilo, dim3((unsigned)blocks), dim3(256), 0, 1, x, (__half *)hi, (__half *)lo, n, st->status_word));
    return after_launch(st, "k_f32_to_f16_hilo");
}

dl4s_status launch_f32_to_f16(DeviceState *st, const float *x, void *y, int64_t n)
{
    if (n == 0) return DL4S_OK;
    DL4S_REQUIRE((((uintptr_t)x | (uintptr_t)y) & 15) == 0, "conversion buffers must be 16-byte aligned");
    int64_t blocks = ceil_div(n, 256 * 8 * 4);
    int64_t cap = (int64_t)st->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    DL4S_CUDA_TRY(launch_pdl(st, k_f32_to_f16, dim3((unsigned)blocks), dim3(256), 0, 1, x, (__half *)y, n, st->status_word));
    return after_launch(st, "k_f32_to_f16");
}

struct GemmTcParams {
    void *c;                 // OUT_F32: float [M,N]; OUT_F16: half [M,N]; OUT_HEADS_F16: unused
    const float *bias;
    const float *residual;
    int64_t M, N, K;
    int epilogue, out_mode;
    int tiles_m, tiles_n;
    int32_t *status;
    double *ln_stats;        // EPI_RESIDUAL_STATS: partial sums per (32 rows, half tile), see tc.cuh
    int32_t *tile_counter;   // {tiles handed out beyond the first gridDim.x, CTAs done}
    int dynamic_tiles;       // 0: worker w takes tiles w, w + workers, ... ; 1: tiles after the first come from the counter
    int lo_from_tn;          // split B: tile columns below this one use W_hi alone (kblocks_hi k-blocks), the others hi + lo
    int kblocks_hi;
    int a_kc;                // A's k extent per column group (K when A is one plain matrix)
    DropoutSpec drop;        // residual flavours: dropout of the product (+ bias) before the residual is added
    int test_skip_kb;        // -1; test only: the k-block of a CTA's first tile whose loads are left out
    uint32_t wait_polls;     // poll limit of every bounded wait (kWaitPolls; short under an injected fault)
    int a_groups;            // column groups of A; the k walk wraps to group 0 after the last one (split B: K = 2 x A's width)
    // OUT_HEADS_F16: columns [part_begin[p], part_begin[p+1]) go to part_ptr[p], a half tensor
    // [B, H, S, part_d[p]] (row m = b*S + s).
    __half *part_ptr[3];
    int part_begin[4];
    int part_d[3];
    int S, H;
};

constexpr int G_GROUP_M = 16;    // tile rows per block of the tile numbering
constexpr int G_TILE_RING = 4;   // tiles the producer may publish ahead of the slowest consumer

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn)
{
    const int per_group = G_GROUP_M * tiles_n;
    const int group = tile / per_group;
    const int first = group * G_GROUP_M;
    const int gm = min(G_GROUP_M, tiles_m - first);
    const int within = tile - group * per_group;
    tm = first + within % gm;
    tn = within / gm;
}

// Stages of the operand ring: 192 KB of shared memory (48 KB per stage for a single CTA's 128 x 256 tile, 32 KB
// for 128-column tiles and for each CTA of a pair).
__host__ __device__ constexpr int gemm_stages(int BN, int PAIR) { return (PAIR || BN == 128) ? 6 : 4; }   // 192 KB

// PAIR = 1: the tile is 256 x BN, worked on by the two CTAs of a cluster with ONE MMA stream
// (cta_group::2) issued by the leader (cluster rank 0). Each CTA loads its 128 rows of A and
// its half of B's columns — per CTA 32 KB per k-block for a 128 x 256 result instead of 48 KB,
// which is what the L2 -> SM path has to deliver — and drains its own 128 accumulator rows.
//
// TA / TB = 1 (single-CTA tiles only): the operand is stored transposed, as the backward of a product needs it
// (Matrix.swift:139-173: dA = dC B^T, dB = A^T dC). A stored [K, M] arrives as 64 x 64 boxes with m contiguous
// (an MN-major operand, like B in the plain form); B stored [N, K] arrives as one box of BN rows of 64 k (a K-major
// operand, like A in the plain form). Only the tensor maps, the tile loads and the descriptors differ.
template <int BN, int EPI, int OUT, int PAIR, int TA = 0, int TB = 0>
__global__ void __launch_bounds__(gemm_threads(EPI, PAIR), 1) k_gemm_tc(const __grid_constant__ CUtensorMap tmap_a,
                                                          const __grid_constant__ CUtensorMap tmap_b, GemmTcParams p)
{
    static_assert(!(TA || TB) || !PAIR, "transposed operands are served by single-CTA tiles");
    constexpr int CTAS = PAIR ? 2 : 1;
    constexpr int G_EPI_PARTS = epi_parts(EPI, PAIR);
    constexpr int G_EPI_WARPS = 4 * G_EPI_PARTS;
    constexpr int BN_CTA = BN / CTAS;                     // B columns this CTA loads
    constexpr uint32_t A_BYTES = GM * GK * 2;             // 16 KB
    constexpr uint32_t B_BLOCK = GK * 64 * 2;             // 8 KB: 64 k-rows x 64 n
    constexpr uint32_t B_BYTES = B_BLOCK * (BN_CTA / 64);
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;                // two accumulators
    constexpr uint32_t A_BLOCK = GK * 64 * 2;             // TA: 64 k-rows x 64 m
    constexpr uint32_t IDESC = idesc_f16(GM * CTAS, BN, TA, TB ? 0 : 1);   // plain form: A K-major, B MN-major

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int G_STAGES = gemm_stages(BN, PAIR);
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader
    const bool leader = rank == 0;
    __shared__ uint64_t full_bar[G_STAGES], empty_bar[G_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint64_t tile_full[G_TILE_RING], tile_empty[G_TILE_RING];
    __shared__ int tile_ring[G_TILE_RING];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < G_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        // the leader's accumulator is released by the epilogue warps of every CTA of the tile
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], G_EPI_WARPS * CTAS); }
        // a tile slot is read by the MMA thread and the eight epilogue warps, and in a pair also by the
        // other CTA's producer and epilogue warps
        for (int t = 0; t < G_TILE_RING; ++t) { mbar_init(&tile_full[t], 1); mbar_init(&tile_empty[t], PAIR ? 2 * (G_EPI_WARPS + 1) : G_EPI_WARPS + 1); }
        abort_s = 0;
        fence_mbar_init();
    }
    if (PAIR) {
        // barriers of both CTAs exist before anything arrives on them from the other CTA
        cluster_sync_all();
        if (warp == 1) { tmem_alloc_pair(&tmem_base_s, TMEM_COLS); tmem_relinquish_pair(); }
    } else if (warp == 1) {
        tmem_alloc(&tmem_base_s, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    volatile int *abort_flag = &abort_s;
    // Everything above touched no global memory: it may run while the previous kernel drains.
    pdl_launch_dependents();
    pdl_wait();

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (int)(p.K / GK);
    // k-blocks of one tile: all of them, or the first half (W_hi alone) for the columns that do not take the remainder
    auto tile_kblocks = [&](int tile) -> int {
        if (p.lo_from_tn == 0) return kblocks;
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        return tn < p.lo_from_tn ? p.kblocks_hi : kblocks;
    };

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // The first tile is the CTA's (the pair's) own index; later ones come from the counter. The
            // leader runs one tile ahead of its own loads: tile it+1 is published (to both CTAs of a
            // pair) before tile it is loaded, and the counter is asked one tile earlier still, so neither
            // the counter's round trip nor the hand-off to the other CTA sits between two tiles' loads.
            const int workers = (int)(gridDim.x / CTAS);
            auto publish = [&](int idx, int t) -> bool {
                const int s = idx % G_TILE_RING;
                if (!mbar_wait(&tile_empty[s], ((idx / G_TILE_RING) & 1) ^ 1, abort_flag, p.wait_polls)) return false;
                tile_ring[s] = t;
                mbar_arrive(&tile_full[s]);
                if (PAIR) {   // the same slot of the other CTA's ring
                    st_remote_u32(&tile_ring[s], 1, (uint32_t)t);
                    mbar_arrive_remote(&tile_full[s], 1);
                }
                return true;
            };
            int kx = 0, kz = 0;   // A is [groups][rows][a_kc]: k = kz * a_kc + kx
            // Loads of k-blocks [kb0, kb1) of one tile; false after a wait that gave up.
            auto load_kblocks = [&](int this_tile, int it, int kb0, int kb1) -> bool {
                int tm, tn;
                tile_coords(this_tile, p.tiles_m, p.tiles_n, tm, tn);
                const int row0 = (tm * CTAS + (int)rank) * GM, col0 = tn * BN + (int)rank * BN_CTA;
                if (kb0 == 0) { kx = 0; kz = 0; }
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.wait_polls)) return false;
                    uint8_t *sa = smem + stage * STAGE_BYTES;
                    if (!PAIR && it == 0 && kb == p.test_skip_kb) {
                        // Injected fault (dl4s_cuda_inject_failure): this stage is never filled, so the MMA thread's
                        // bounded wait on it runs out and the CTA unwinds through the common exit.
                    } else if (PAIR) {
                        // both CTAs' bytes are counted on the leader's barrier
                        if (leader) mbar_expect_tx_relaxed(&full_bar[stage], STAGE_BYTES * CTAS);
                        tma_load_3d_pair(sa, &tmap_a, &full_bar[stage], kx, row0, kz);
#pragma unroll
                        for (int nb = 0; nb < BN_CTA / 64; ++nb)
                            tma_load_2d_pair(sa + A_BYTES + nb * B_BLOCK, &tmap_b, &full_bar[stage], col0 + nb * 64, kb * GK);
                    } else {
                        mbar_expect_tx_relaxed(&full_bar[stage], STAGE_BYTES);
                        if (TA) {
#pragma unroll
                            for (int mb = 0; mb < GM / 64; ++mb)
                                tma_load_2d(sa + mb * A_BLOCK, &tmap_a, &full_bar[stage], row0 + mb * 64, kb * GK);
                        } else {
                            tma_load_3d(sa, &tmap_a, &full_bar[stage], kx, row0, kz);
                        }
                        if (TB) {
                            tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[stage], kb * GK, col0);
                        } else {
#pragma unroll
                            for (int nb = 0; nb < BN_CTA / 64; ++nb)
                                tma_load_2d(sa + A_BYTES + nb * B_BLOCK, &tmap_b, &full_bar[stage], col0 + nb * 64, kb * GK);
                        }
                    }
                    if (++stage == G_STAGES) { stage = 0; phase ^= 1; }
                    kx += GK;
                    if (kx == p.a_kc) { kx = 0; if (++kz == p.a_groups) kz = 0; }
                }
                return true;
            };
            // Order within a tile: publish the next tile (a release arrive), THEN ask the counter for the one after
            // it, then load. A release arrive waits for the thread's outstanding atomic, so an atomic issued before
            // the publish would put its whole round trip (~1000-3000 cycles) between two tiles' loads; issued after
            // it, the round trip runs under this tile's loads, whose barrier operations are relaxed.
            int cur = blockIdx.x / CTAS, nxt = 0;
            int it_begin = 0;
            if (!p.dynamic_tiles) {
                // Fixed schedule: every role of every CTA works the tile sequence out by itself.
                for (int it = 0, t = cur; ok && t < num_tiles; ++it, t += workers) ok = load_kblocks(t, it, 0, tile_kblocks(t));
                ok = false;   // done: skip the counter-driven loop below
            } else if (leader) {
                const int a1 = atomicAdd(p.tile_counter, 1);      // tile 1 of this CTA (pair)
                ok = publish(0, cur);                             // waits for a1: nothing else to do yet
                if (ok) {
                    // the ring is empty: its first stages are requested before the counter's answer is needed
                    const int kbt = tile_kblocks(cur);
                    const int first = kbt < G_STAGES ? kbt : G_STAGES;
                    ok = load_kblocks(cur, 0, 0, first);
                    nxt = workers + a1;
                    if (ok) ok = publish(1, nxt);
                    const int a2 = atomicAdd(p.tile_counter, 1);  // tile 2, needed when tile 1's loads begin
                    if (ok) ok = load_kblocks(cur, 0, first, kbt);
                    cur = nxt;
                    nxt = workers + a2;
                    it_begin = 1;
                }
            }
            for (int it = it_begin; ok; ++it) {
                const int slot = it % G_TILE_RING;
                int this_tile;
                if (leader) {
                    if (cur >= num_tiles) break;   // the end marker has been published
                    if (!publish(it + 1, nxt)) break;
                    const int nxt2 = workers + atomicAdd(p.tile_counter, 1);
                    this_tile = cur;
                    cur = nxt;
                    ok = load_kblocks(this_tile, it, 0, tile_kblocks(this_tile));
                    nxt = nxt2;
                } else {
                    if (!mbar_wait_cluster(&tile_full[slot], (it / G_TILE_RING) & 1, abort_flag, p.wait_polls)) break;
                    this_tile = tile_ring[slot];
                    if (this_tile >= num_tiles) break;             // the end marker's slot is never reused
                    mbar_arrive_remote_relaxed(&tile_empty[slot], 0);   // issued after the branch on the value read
                    ok = load_kblocks(this_tile, it, 0, tile_kblocks(this_tile));
                }
            }
        }
    } else if (warp == 1) {
        if (leader && elect_one()) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            const int workers = (int)(gridDim.x / CTAS);
            for (int it = 0; ok; ++it) {
                const int slot = it % G_TILE_RING;
                int tile;
                if (!p.dynamic_tiles) {
                    tile = (int)(blockIdx.x / CTAS) + it * workers;
                } else {
                    if (!mbar_wait(&tile_full[slot], (it / G_TILE_RING) & 1, abort_flag, p.wait_polls)) break;
                    tile = tile_ring[slot];
                    mbar_arrive(&tile_empty[slot]);
                }
                if (tile >= num_tiles) break;
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.wait_polls)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int kbt = tile_kblocks(tile);
                for (int kb = 0; kb < kbt; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.wait_polls)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < GK / 16; ++k16) {
                        uint64_t adesc = TA ? smem_desc_mn_sw128(sa + k16 * 2048, A_BLOCK, 1024) : smem_desc_sw128(sa + k16 * 32, 16, 1024);
                        uint64_t bdesc = TB ? smem_desc_sw128(sb + k16 * 32, 16, 1024) : smem_desc_mn_sw128(sb + k16 * 2048, B_BLOCK, 1024);
                        if (PAIR) umma_ss_pair(d_tmem, adesc, bdesc, IDESC, (kb | k16) != 0);
                        else umma_ss(d_tmem, adesc, bdesc, IDESC, (kb | k16) != 0);
                    }
                    // frees the stage in both CTAs / tells both CTAs' epilogue warps
                    if (PAIR) umma_commit_pair(&empty_bar[stage], 3);
                    else umma_commit(&empty_bar[stage]);
                    if (++stage == G_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (PAIR) umma_commit_pair(&acc_full[acc], 3);
                else umma_commit(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        const int quarter = warp & 3;   // tensor-memory lanes this warp may read
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int slot = it % G_TILE_RING;
            int tile;
            if (!p.dynamic_tiles) {
                tile = (int)(blockIdx.x / CTAS) + it * (int)(gridDim.x / CTAS);
                if (tile >= num_tiles) break;
            } else {
                if (PAIR && !leader) {
                    if (!mbar_wait_cluster(&tile_full[slot], (it / G_TILE_RING) & 1, abort_flag, p.wait_polls)) break;
                } else {
                    if (!mbar_wait(&tile_full[slot], (it / G_TILE_RING) & 1, abort_flag, p.wait_polls)) break;
                }
                tile = tile_ring[slot];
                if (tile >= num_tiles) break;   // the end marker's slot is never reused: no arrival needed
                // Relaxed: the slot's value has been read (the branch above depends on it) and nothing this warp
                // wrote is handed over; a release arrive here would wait for the previous tile's global stores.
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && !leader) mbar_arrive_remote_relaxed(&tile_empty[slot], 0);
                    else mbar_arrive_relaxed(&tile_empty[slot]);
                }
            }
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.wait_polls)) { ok = false; break; }
            tc_fence_after();
            // Each warp drains its 32 accumulator rows 32 columns at a time with two 16-lane x 256-bit
            // tensor-memory loads: thread `lane` then holds, for rows lane/4 + {0, 8, 16, 24} of the warp's
            // 32, the column pairs 8p + 2(lane%4) + {0,1}, p = 0..3 (see tmem_ld16x256b_x4). Four lanes own 8
            // consecutive columns of a row, so a warp store of one pair covers 8 rows x 32 bytes (fp32) or
            // 8 rows x 16 bytes (half) and nothing goes through shared memory: the operand ring and the
            // tensor core's operand reads already use the whole shared-memory bandwidth (48 KB written and
            // 48 KB read per k-block against 128 bytes per clock), and a turn of the accumulators through it
            // took ~2400 cycles per 32 x 32 block under that load (clock64 stamps), four times the main
            // loop's share of the tile.
            const int64_t row_base = ((int64_t)tm * CTAS + rank) * GM + quarter * 32;
            const int rsub = lane >> 2, cg = (lane & 3) * 2;
            const int c_begin = ((warp - 2) >> 2) * (BN / G_EPI_PARTS), c_end = c_begin + BN / G_EPI_PARTS;
            // Head-major output: (batch, position) of row row_base + lane, worked out once per tile and
            // handed to the lanes that store the row by shuffle (no division per stored segment).
            int my_bb = 0, my_ss = 0;
            if (OUT == OUT_HEADS_F16) {
                const uint32_t my_row = (uint32_t)(row_base + lane);
                my_bb = (int)(my_row / (uint32_t)p.S);
                my_ss = (int)(my_row - (uint32_t)my_bb * (uint32_t)p.S);
            }
            float stat1 = 0.f, stat2 = 0.f;   // EPI_RESIDUAL_STATS: this lane's share of the warp's block
            float amax = 0.f;                 // half outputs: largest magnitude this lane converts (range check at the end)
            constexpr bool kHasResidual = (EPI == EPI_BIAS_RESIDUAL || EPI == EPI_RESIDUAL || EPI == EPI_RESIDUAL_STATS);
            // Head-major output, common case: the warp's 32 rows lie in one batch element, so the rows a lane
            // stores (rsub, rsub + 8, ...) are part_d * 8 elements apart and one address per group is enough.
            int bb_first = 0, ss_first = 0;
            bool one_batch = true;
            if (OUT == OUT_HEADS_F16) {
                bb_first = __shfl_sync(0xffffffffu, my_bb, 0);
                ss_first = __shfl_sync(0xffffffffu, my_ss, 0);
                one_batch = __shfl_sync(0xffffffffu, my_bb, 31) == bb_first;
            }
            const int64_t first_row = row_base + rsub;            // the first of the 4 rows this lane stores
            const int64_t row_off0 = first_row * p.N;             // plain row-major outputs and the residual
            auto load_group = [&](uint32_t (&r)[32], int c0) {
                tmem_ld16x256b_x4(tmem_addr(tmem_base, quarter * 32, acc * BN + c0), r, 0);
                tmem_ld16x256b_x4(tmem_addr(tmem_base, quarter * 32 + 16, acc * BN + c0), r, 16);
            };
            // One 32-column group: `rc` holds it, `rnx` receives the next one while this one is written out.
            // rc[16h + 4p + 2q + e] = row 16h + 8q + rsub of the warp, column 8p + cg + e of the group.
            auto group = [&](uint32_t (&rc)[32], uint32_t (&rnx)[32], int c0, bool has_next) {
                const int64_t col0 = (int64_t)tn * BN + c0;
                // The residual values of this group are requested before the wait on tensor memory, so
                // their latency hides behind it. (With many epilogue warps the other warps cover that
                // latency and the registers are needed elsewhere: the residual is then read where it is used.)
                constexpr bool kPrefetchResidual = kHasResidual && G_EPI_PARTS == 2;
                float2 res[kPrefetchResidual ? 16 : 1];
                const float *rp = kHasResidual ? p.residual + row_off0 + col0 + cg : nullptr;
                if (kPrefetchResidual && col0 < p.N) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int rq = i >> 2, pp = i & 3;    // row rsub + 8 rq, column pair pp
                        res[i] = first_row + rq * 8 < p.M ? *reinterpret_cast<const float2 *>(rp + (int64_t)rq * 8 * p.N + pp * 8)
                                                          : make_float2(0.f, 0.f);
                    }
                }
                tmem_wait_ld();
                // The next 32 columns travel from tensor memory while this group is written out.
                if (has_next) load_group(rnx, c0 + 32);
                if (col0 >= p.N) return;   // N is a multiple of 64: a 32-column group is all in or all out
                // Half outputs: two lanes that hold neighbouring column pairs swap one pair each, so that every lane
                // stores 4 consecutive halves (8 bytes) and the four lanes of a row 32 contiguous bytes: whole
                // sectors. (A 4 x 4 transpose to one 16-byte store per lane halves the store count but costs more
                // shuffles and selects than it saves; the epilogue is bound by its instruction count.)
                // ch = first of the 4 columns (within 8) this lane then stores.
                const int ch = ((lane >> 1) & 1) * 4;
                // Head-major output: the 32-column group lies inside one head of one part.
                __half *part_base = nullptr;
                int part_d = 1, head = 0, dcol = 0;
                __half *hdst = nullptr;       // half outputs: address of this lane's first row, then a constant step
                int64_t hstep = 0;
                if (OUT == OUT_HEADS_F16) {
                    int part = (col0 >= p.part_begin[1]) + (col0 >= p.part_begin[2]);
                    int rel = (int)col0 - p.part_begin[part];
                    part_d = p.part_d[part];
                    head = rel / part_d;
                    dcol = rel - head * part_d + ch;
                    part_base = p.part_ptr[part];
                    hdst = part_base + (((int64_t)bb_first * p.H + head) * p.S + ss_first + rsub) * part_d + dcol;
                    hstep = (int64_t)8 * part_d;
                } else if (OUT == OUT_F16) {
                    hdst = reinterpret_cast<__half *>(p.c) + row_off0 + col0 + ch;
                    hstep = (int64_t)8 * p.N;
                }
                float *fdst = OUT == OUT_F32 ? reinterpret_cast<float *>(p.c) + row_off0 + col0 + cg : nullptr;
                float2 bias2[4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp)
                    bias2[pp] = (EPI != EPI_NONE && EPI != EPI_RESIDUAL && EPI != EPI_RESIDUAL_STATS)
                                    ? *reinterpret_cast<const float2 *>(p.bias + col0 + cg + pp * 8)
                                    : make_float2(0.f, 0.f);
#pragma unroll
                for (int rq = 0; rq < 4; ++rq) {
                    const int rr = rq * 8 + rsub;
                    int bb = 0, ss = 0;
                    if (OUT == OUT_HEADS_F16 && !one_batch) {     // rare: the 32 rows straddle two batch elements
                        bb = __shfl_sync(0xffffffffu, my_bb, rr);
                        ss = __shfl_sync(0xffffffffu, my_ss, rr);
                    }
                    const bool row_ok = first_row + rq * 8 < p.M;
                    __half *hrow = hdst + rq * hstep;
                    if (OUT == OUT_HEADS_F16 && !one_batch)
                        hrow = part_base + (((int64_t)bb * p.H + head) * p.S + ss) * part_d + dcol;
                    uint32_t h2[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) {
                        const int ri = (rq >> 1) * 16 + pp * 4 + (rq & 1) * 2;
                        float2 t = make_float2(__uint_as_float(rc[ri]), __uint_as_float(rc[ri + 1]));
                        switch (EPI) {
                            case EPI_BIAS:
                            case EPI_BIAS_RESIDUAL:
                                t.x += bias2[pp].x; t.y += bias2[pp].y;
                                break;
                            case EPI_BIAS_GELU:
                                t.x = gelu_sigmoid_tc(t.x + bias2[pp].x); t.y = gelu_sigmoid_tc(t.y + bias2[pp].y);
                                break;
                            case EPI_BIAS_RELU:
                                t.x = fmaxf(t.x + bias2[pp].x, 0.f); t.y = fmaxf(t.y + bias2[pp].y, 0.f);
                                break;
                            default: break;
                        }
                        if (kHasResidual && p.drop.threshold != 0) {
                            // Dropout.swift:47-55 on the projection's output (MultiHeadAttention.swift:122,
                            // PointwiseFeedForward.swift:78): element (row, column) of the [M, N] result
                            const uint64_t e = (uint64_t)((first_row + rq * 8) * p.N + col0 + cg + pp * 8);
                            t.x = dropout_keep(p.drop, e) ? t.x : 0.f;
                            t.y = dropout_keep(p.drop, e + 1) ? t.y : 0.f;
                        }
                        if (kHasResidual) {
                            const float2 q = kPrefetchResidual ? res[kPrefetchResidual ? rq * 4 + pp : 0]
                                             : row_ok      ? *reinterpret_cast<const float2 *>(rp + (int64_t)rq * 8 * p.N + pp * 8)
                                                           : make_float2(0.f, 0.f);
                            t.x += q.x; t.y += q.y;
                        }
                        if (EPI == EPI_RESIDUAL_STATS && row_ok) {
                            stat1 += t.x + t.y;
                            stat2 = fmaf(t.x, t.x, stat2); stat2 = fmaf(t.y, t.y, stat2);
                        }
                        if (OUT == OUT_F32) {
                            if (row_ok) *reinterpret_cast<float2 *>(fdst + (int64_t)rq * 8 * p.N + pp * 8) = t;
                        } else {
                            __half2 h = __floats2half2_rn(t.x, t.y);
                            h2[pp] = *reinterpret_cast<uint32_t *>(&h);
                            amax = max3_abs(amax, t.x, t.y);
                        }
                    }
                    if (OUT != OUT_F32) {
#pragma unroll
                        for (int p2 = 0; p2 < 4; p2 += 2) {
                            const uint32_t send = (lane & 1) ? h2[p2] : h2[p2 + 1];
                            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
                            uint2 o;
                            o.x = (lane & 1) ? recv : h2[p2];
                            o.y = (lane & 1) ? h2[p2 + 1] : recv;
                            if (row_ok) *reinterpret_cast<uint2 *>(hrow + (p2 + (lane & 1)) * 8) = o;
                        }
                    }
                }
            };
            uint32_t ra[32], rb[32];
            constexpr int NG = BN / G_EPI_PARTS / 32;          // 32-column groups per warp
            constexpr bool kEarlyRelease = !kHasResidual && NG <= 2;
            auto release_acc = [&]() {
                // The accumulator goes back to the MMA thread. Every tensor-memory load of this warp has completed
                // (tcgen05.wait::ld) and is ordered before the arrive by the fence; the tile's global stores are
                // nobody's business here, so the arrive is relaxed and does not wait for them.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && !leader) mbar_arrive_remote_relaxed(&acc_empty[acc], 0);
                    else mbar_arrive_relaxed(&acc_empty[acc]);
                }
            };
            if constexpr (kEarlyRelease) {
                // The warp's whole share of the accumulator (64 columns of 32 rows = 64 registers per lane) is read
                // first and the accumulator handed back before anything is converted or stored: with two
                // accumulators the MMAs of tile i+2 wait for the drain of tile i, so the time an accumulator is held
                // (not the length of the epilogue) is what the tile rate sees.
                load_group(ra, c_begin);
                if (NG == 2) load_group(rb, c_begin + 32);
                tmem_wait_ld();
                release_acc();
                group(ra, rb, c_begin, false);
                if (NG == 2) group(rb, ra, c_begin + 32, false);
            } else if constexpr (!kHasResidual) {
                // Two register sets take turns (no copies).
                load_group(ra, c_begin);
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_end; c0 += 64) {
                    group(ra, rb, c0, true);
                    group(rb, ra, c0 + 32, c0 + 64 < c_end);
                }
            } else {
                // The residual flavours keep 16 prefetched residual pairs live as well; a second register set
                // would spill, so the groups run one after the other (the residual loads cover the wait).
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                    load_group(ra, c0);
                    group(ra, rb, c0, false);
                }
            }
            if (EPI == EPI_RESIDUAL_STATS) {
                double d1 = stat1, d2 = stat2;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
                    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
                }
                if (lane == 0 && row_base < p.M) {
                    const int64_t slot = (row_base >> 5) * (G_EPI_PARTS * p.tiles_n) + G_EPI_PARTS * tn + ((warp - 2) >> 2);
                    p.ln_stats[2 * slot] = d1;
                    p.ln_stats[2 * slot + 1] = d2;
                }
            }
            // 65504 is the largest finite half; anything that rounds beyond it (or an accumulator that is already
            // infinite) trips the range bit. NaNs cannot appear here without a non-finite operand, and those are
            // caught where the operands were converted.
            if (OUT != OUT_F32 && !(amax < 65520.f)) atomicOr(p.status, kStatusHalfRange);
            if (!kEarlyRelease) release_acc();
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    // Common exit: everyone arrives here, also after a wait that gave up.
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (abort_s) atomicOr(p.status, kStatusGemmTimeout);
        // This CTA takes no more tiles. The last CTA to get here leaves the counters at zero for the
        // next launch that uses the slot.
        __threadfence();
        if (atomicAdd(p.tile_counter + 1, 1) == (int)gridDim.x - 1) {
            p.tile_counter[0] = 0;
            p.tile_counter[1] = 0;
            __threadfence();
        }
    }
    if (PAIR) {
        // neither CTA frees tensor memory (or leaves) while the other may still use the pair's MMAs
        cluster_sync_all();
        if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// The driver entry point is resolved at run time so the library carries no
// link-time dependency on libcuda (it must load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

dl4s_status make_tmap_f16(CUtensorMap *map, const void *base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                          uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1)
{
    auto fn = get_encode_fn();
    if (!fn) return fail(DL4S_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    DL4S_REQUIRE(((uintptr_t)base & 15) == 0 && stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0,
                 "TMA needs a 16-byte aligned base and strides");
    const bool three = dim2 > 0;
    cuuint64_t dims[3] = {dim0, dim1, three ? dim2 : 1};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, three ? 3 : 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DL4S_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return DL4S_OK;
}

// Same choice of tile width as launch_gemm_tc_h makes.
static bool gemm_tc_wide_tiles(int64_t N) { return N % 256 == 0 || N >= 1024; }

int gemm_tc_stats_per_row_block(int64_t N) { return epi_parts(EPI_RESIDUAL_STATS, 0) * (int)ceil_div(N, gemm_tc_wide_tiles(N) ? 256 : 128); }

bool gemm_tc_supported(int64_t M, int64_t N, int64_t K)
{
    return M >= GM && N >= 64 && N % 64 == 0 && K >= GK && K % GK == 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31);
}

size_t gemm_tc_scratch_bytes(int64_t M, int64_t N, int64_t K, int split)
{
    return align_up((size_t)(M * K) * 2, 1024) + align_up((size_t)(K * N) * (split ? 4 : 2), 1024);
}

// Shortest main loop (K) that uses two-CTA tiles.
constexpr int64_t kPairMinK = 1024;

template <int BN, int EPI, int OUT, int PAIR, int TA = 0, int TB = 0>
static dl4s_status run_gemm_tc_inst2(DeviceState *st, const CUtensorMap &ta, const CUtensorMap &tb, GemmTcParams p, const char *name)
{
    constexpr int CTAS = PAIR ? 2 : 1;
    // operand ring + slack for its 1 KB alignment
    constexpr size_t smem = (size_t)gemm_stages(BN, PAIR) * (GM * GK * 2 + GK * (BN / CTAS) * 2) + 1024;
    static bool attr_set[kMaxDevices] = {false};
    if (!attr_set[st->ordinal]) {
        DL4S_CUDA_TRY(cudaFuncSetAttribute(k_gemm_tc<BN, EPI, OUT, PAIR, TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[st->ordinal] = true;
    }
    p.tiles_m = (int)ceil_div(p.M, GM * CTAS);
    p.tiles_n = (int)ceil_div(p.N, BN);
    const int workers = st->sm_count / CTAS;   // CTAs, or pairs of CTAs
    const int grid = (p.tiles_m * p.tiles_n < workers ? p.tiles_m * p.tiles_n : workers) * CTAS;
    p.tile_counter = st->tile_counters + 2 * st->tile_counter_next;
    st->tile_counter_next = (st->tile_counter_next + 1) % kTileCounterSlots;
    p.test_skip_kb = -1;
    p.wait_polls = kWaitPolls;
    // Long launches (many tiles per worker) also take the counter: handing tiles out in arrival order keeps the set
    // of tiles in flight compact while the workers drift apart (measured at M 131072, N 12288, K 4096: 39.3 ms
    // against 44.4 ms with the fixed schedule); short ones (the encoder's 2-7 tiles per worker) are better off
    // without its round trips.
    p.dynamic_tiles = st->dynamic_tiles || p.tiles_m * p.tiles_n > 16 * workers;
    if (!PAIR && !st->capturing && take_injected_failure(DL4S_INJECT_WAIT_TIMEOUT)) {
        p.test_skip_kb = p.K / GK > 1 ? 1 : 0;
        p.wait_polls = 1u << 16;
    }
    DL4S_CUDA_TRY(launch_pdl(st, k_gemm_tc<BN, EPI, OUT, PAIR, TA, TB>, dim3((unsigned)grid), dim3(gemm_threads(EPI, PAIR)), smem, CTAS, ta, tb,
                             p));
    return after_launch(st, name);
}

// Pairs of CTAs (one MMA over two SMs) for 256-column tiles with a long main loop (K >= 1024):
// measured 1480 vs 1260 TFLOP/s at 8192^3. With K = 512 a tile has only 8 k-blocks and the epilogue warps set the
// rate for either form (see the head of this file): the encoder's q/k/v projection and feed-forward 1 take
// 0.222 / 0.270 ms per step as pairs and 0.220 / 0.278 ms as single CTAs, so short products keep the single-CTA kernel.
template <int BN, int EPI, int OUT>
static dl4s_status run_gemm_tc_inst(DeviceState *st, const CUtensorMap &ta, const CUtensorMap &tb, GemmTcParams p, const char *name)
{
    if (BN == 256 && p.M >= 2 * GM && p.K >= kPairMinK)
        return run_gemm_tc_inst2<BN, EPI, OUT, (BN == 256)>(st, ta, tb, p, name);
    return run_gemm_tc_inst2<BN, EPI, OUT, 0>(st, ta, tb, p, name);
}

// The epilogue flavour is a compile-time parameter: each instance carries only its own epilogue,
// which keeps the kernel's inner loops small. The per-kernel profile tells the flavours apart by name.
template <int BN>
static dl4s_status run_gemm_tc(DeviceState *st, const CUtensorMap &ta, const CUtensorMap &tb, const GemmTcParams &p)
{
    if (p.out_mode == OUT_HEADS_F16 && p.epilogue == EPI_NONE)
        return run_gemm_tc_inst<BN, EPI_NONE, OUT_HEADS_F16>(st, ta, tb, p, "k_gemm_tc.heads_f16");
    if (p.out_mode == OUT_F16 && p.epilogue == EPI_BIAS_GELU)
        return run_gemm_tc_inst<BN, EPI_BIAS_GELU, OUT_F16>(st, ta, tb, p, "k_gemm_tc.act_f16");
    if (p.out_mode == OUT_F16 && p.epilogue == EPI_BIAS_RELU)
        return run_gemm_tc_inst<BN, EPI_BIAS_RELU, OUT_F16>(st, ta, tb, p, "k_gemm_tc.act_f16");
    if (p.out_mode == OUT_F32) {
        switch (p.epilogue) {
            case EPI_NONE: return run_gemm_tc_inst<BN, EPI_NONE, OUT_F32>(st, ta, tb, p, "k_gemm_tc");
            case EPI_BIAS: return run_gemm_tc_inst<BN, EPI_BIAS, OUT_F32>(st, ta, tb, p, "k_gemm_tc.bias_f32");
            case EPI_BIAS_GELU: return run_gemm_tc_inst<BN, EPI_BIAS_GELU, OUT_F32>(st, ta, tb, p, "k_gemm_tc.bias_f32");
            case EPI_BIAS_RELU: return run_gemm_tc_inst<BN, EPI_BIAS_RELU, OUT_F32>(st, ta, tb, p, "k_gemm_tc.bias_f32");
            case EPI_BIAS_RESIDUAL: return run_gemm_tc_inst<BN, EPI_BIAS_RESIDUAL, OUT_F32>(st, ta, tb, p, "k_gemm_tc.bias_residual_f32");
            case EPI_RESIDUAL: return run_gemm_tc_inst<BN, EPI_RESIDUAL, OUT_F32>(st, ta, tb, p, "k_gemm_tc.residual_f32");
            case EPI_RESIDUAL_STATS: return run_gemm_tc_inst<BN, EPI_RESIDUAL_STATS, OUT_F32>(st, ta, tb, p, "k_gemm_tc.residual_stats_f32");
            default: break;
        }
    }
    return fail(DL4S_ERR_UNSUPPORTED, "no tensor-core gemm instance for epilogue %d with output mode %d", p.epilogue, p.out_mode);
}

dl4s_status launch_gemm_tc_h(DeviceState *st, const void *a_half, const void *b_half, int64_t M, int64_t N, int64_t K,
                             int epilogue, const float *bias, const float *residual, const GemmTcOut &out,
                             int64_t a_groups, int64_t a_group_stride, int b_split, const DropoutSpec *drop,
                             int64_t b_split_from_col)
{
    DL4S_REQUIRE(gemm_tc_supported(M, N, K), "shape not supported by the tensor-core gemm");
    DL4S_REQUIRE(2 * K < (1ll << 31), "K too large");
    DL4S_REQUIRE(!residual || ((uintptr_t)residual & 15) == 0, "residual must be 16-byte aligned");
    DL4S_REQUIRE(a_groups >= 1 && K % a_groups == 0 && (K / a_groups) % GK == 0,
                 "A's column groups must each hold a multiple of %d columns", GK);
    const int64_t kc = K / a_groups;
    if (a_groups == 1) a_group_stride = M * K;
    DL4S_REQUIRE(a_group_stride % 8 == 0, "A's group stride must be a multiple of 8 elements");
    CUtensorMap ta, tb;
    // A as [groups][M][kc]: rows past M read as zeros, whatever lies behind them in memory.
    DL4S_TRY(make_tmap_f16(&ta, a_half, (uint64_t)kc, (uint64_t)M, (uint64_t)a_groups, (uint64_t)kc * 2,
                           (uint64_t)a_group_stride * 2, GK, GM));
    // Split B: [W_hi; W_lo] stacked along k. The main loop runs over 2K rows of B while A's k walk wraps after K,
    // so the accumulator receives A W_hi + A W_lo.
    const int64_t Kb = b_split ? 2 * K : K;
    DL4S_TRY(make_tmap_f16(&tb, b_half, (uint64_t)N, (uint64_t)Kb, 0, (uint64_t)N * 2, 0, 64, GK));
    GemmTcParams p;
    p.c = out.c; p.bias = bias; p.residual = residual;
    p.M = M; p.N = N; p.K = Kb;
    p.a_kc = (int)kc;
    p.a_groups = (int)a_groups;
    // Columns below b_split_from_col take W_hi alone; it has to fall on a tile boundary (else every column takes both).
    const int64_t bn = gemm_tc_wide_tiles(N) ? 256 : 128;
    p.kblocks_hi = (int)(K / GK);
    p.lo_from_tn = (b_split && b_split_from_col > 0 && b_split_from_col % bn == 0) ? (int)(b_split_from_col / bn) : 0;
    p.drop = drop ? *drop : DropoutSpec();
    DL4S_REQUIRE(p.drop.threshold == 0 || epi_has_residual(epilogue), "dropout is fused into the residual epilogues only");
    p.ln_stats = out.ln_stats;
    DL4S_REQUIRE(epilogue != EPI_RESIDUAL_STATS || (out.ln_stats && out.mode == OUT_F32), "the statistics epilogue needs its buffer");
    p.epilogue = epilogue;
    p.out_mode = out.mode;
    p.status = st->status_word;
    p.S = 1; p.H = 1;
    for (int i = 0; i < 3; ++i) { p.part_ptr[i] = nullptr; p.part_begin[i] = 0; p.part_d[i] = 32; }
    p.part_begin[3] = 0;
    if (out.mode == OUT_HEADS_F16) {
        DL4S_REQUIRE(out.nparts >= 1 && out.nparts <= 3 && out.S >= 1 && M % out.S == 0, "bad head-major output description");
        int begin = 0;
        for (int i = 0; i < 3; ++i) {
            p.part_begin[i] = begin;
            if (i < out.nparts) {
                DL4S_REQUIRE(out.part_d[i] % 32 == 0 && ((uintptr_t)out.part_ptr[i] & 15) == 0, "head size must be a multiple of 32");
                p.part_ptr[i] = (__half *)out.part_ptr[i];
                p.part_d[i] = out.part_d[i];
                begin += out.H * out.part_d[i];
            } else {
                p.part_begin[i] = 1 << 30;   // never selected
            }
        }
        p.part_begin[3] = begin;
        DL4S_REQUIRE(begin == N, "head-major parts cover %d columns, the product has %lld", begin, (long long)N);
        p.S = out.S; p.H = out.H;
    } else {
        DL4S_REQUIRE(out.c && ((uintptr_t)out.c & 15) == 0, "C must be 16-byte aligned");
    }
    if (gemm_tc_wide_tiles(N)) return run_gemm_tc<256>(st, ta, tb, p);
    return run_gemm_tc<128>(st, ta, tb, p);
}

dl4s_status launch_gemm_tc(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                           int epilogue, const float *bias, const float *residual, void *scratch, size_t scratch_bytes, int split,
                           const DropoutSpec *drop)
{
    DL4S_REQUIRE(gemm_tc_supported(M, N, K), "shape not supported by the tensor-core gemm");
    DL4S_REQUIRE(scratch && scratch_bytes >= gemm_tc_scratch_bytes(M, N, K, split), "scratch too small");
    __half *ah = (__half *)scratch;
    __half *bh = (__half *)((char *)scratch + align_up((size_t)(M * K) * 2, 1024));
    DL4S_TRY(launch_f32_to_f16(st, a, ah, M * K));
    // the second operand is the weight matrix in every caller: it is the one that may enter as two halves
    if (split) DL4S_TRY(launch_f32_to_f16_hilo(st, b, bh, bh + K * N, K * N));
    else DL4S_TRY(launch_f32_to_f16(st, b, bh, K * N));
    GemmTcOut out;
    out.mode = OUT_F32;
    out.c = c;
    return launch_gemm_tc_h(st, ah, bh, M, N, K, epilogue, bias, residual, out, 1, 0, split, drop);
}

// C = op(A) op(B) with at least one operand stored transposed (the shapes the backward of a product takes,
// Matrix.swift:139-173): A stored [K, M] when trans_a, B stored [N, K] when trans_b; fp32 in and out, operands rounded
// to half in their stored layout. Single-CTA tiles; needs what gemm_tc_supported asks plus M % 8 == 0 when trans_a
// (the TMA row stride of the stored matrix).
bool gemm_tc_trans_supported(int64_t M, int64_t N, int64_t K, int trans_a, int trans_b)
{
    return gemm_tc_supported(M, N, K) && (trans_a || trans_b) && (!trans_a || M % 8 == 0);
}

template <int TA, int TB>
static dl4s_status run_gemm_tc_trans(DeviceState *st, const CUtensorMap &ta, const CUtensorMap &tb, const GemmTcParams &p, bool wide)
{
    if (wide) return run_gemm_tc_inst2<256, EPI_NONE, OUT_F32, 0, TA, TB>(st, ta, tb, p, "k_gemm_tc.transposed");
    return run_gemm_tc_inst2<128, EPI_NONE, OUT_F32, 0, TA, TB>(st, ta, tb, p, "k_gemm_tc.transposed");
}

dl4s_status launch_gemm_tc_trans(DeviceState *st, const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K,
                                 int trans_a, int trans_b, void *scratch, size_t scratch_bytes)
{
    DL4S_REQUIRE(gemm_tc_trans_supported(M, N, K, trans_a, trans_b), "shape not supported by the transposed tensor-core gemm");
    DL4S_REQUIRE(scratch && scratch_bytes >= gemm_tc_scratch_bytes(M, N, K, 0), "scratch too small");
    DL4S_REQUIRE(c && ((uintptr_t)c & 15) == 0, "C must be 16-byte aligned");
    __half *ah = (__half *)scratch;
    __half *bh = (__half *)((char *)scratch + align_up((size_t)(M * K) * 2, 1024));
    DL4S_TRY(launch_f32_to_f16(st, a, ah, M * K));
    DL4S_TRY(launch_f32_to_f16(st, b, bh, K * N));
    const bool wide = gemm_tc_wide_tiles(N);
    CUtensorMap ta, tb;
    if (trans_a)   // stored [K][M]: boxes of 64 m x 64 k-rows
        DL4S_TRY(make_tmap_f16(&ta, ah, (uint64_t)M, (uint64_t)K, 0, (uint64_t)M * 2, 0, 64, GK));
    else
        DL4S_TRY(make_tmap_f16(&ta, ah, (uint64_t)K, (uint64_t)M, 1, (uint64_t)K * 2, (uint64_t)(M * K) * 2, GK, GM));
    if (trans_b)   // stored [N][K]: one box of BN rows x 64 k
        DL4S_TRY(make_tmap_f16(&tb, bh, (uint64_t)K, (uint64_t)N, 0, (uint64_t)K * 2, 0, GK, wide ? 256 : 128));
    else
        DL4S_TRY(make_tmap_f16(&tb, bh, (uint64_t)N, (uint64_t)K, 0, (uint64_t)N * 2, 0, 64, GK));
    GemmTcParams p = {};
    p.c = c;
    p.M = M; p.N = N; p.K = K;
    p.a_kc = (int)K;
    p.a_groups = 1;
    p.epilogue = EPI_NONE;
    p.out_mode = OUT_F32;
    p.status = st->status_word;
    p.S = 1; p.H = 1;
    for (int i = 0; i < 3; ++i) p.part_d[i] = 32;
    if (trans_a && trans_b) return run_gemm_tc_trans<1, 1>(st, ta, tb, p, wide);
    if (trans_a) return run_gemm_tc_trans<1, 0>(st, ta, tb, p, wide);
    return run_gemm_tc_trans<0, 1>(st, ta, tb, p, wide);
}

}  // namespace dl4s
