"""GPU tier: the benchmark configurations at their FULL sizes.

The CPU engine cannot finish these in test time, so each case is checked (a) through properties that do not depend on
the size and (b) against an exact float64 evaluation of sampled outputs (one query row of one head needs only that
head's keys and values), and the encoder against the float64 numpy formulation of the same op sequence (BLAS makes
the full configuration a matter of seconds). Tolerances are those of the tensor-core path, unscaled: max-abs 2e-3 and
relative L2 1e-3; the decode kernels are fp32 and held to 1e-5."""
import numpy as np
import pytest

from dl4s_b200 import PREC_F16, workloads
from util import F16_DEEP_MAX_ABS_DOCUMENTED, TC_MAX_ABS, TC_REL_L2, assert_tc, max_abs, rel_l2

pytestmark = pytest.mark.gpu


def exact_row(q_row, K, V, inv_t):
    """softmax(q K^T * inv_t) V in float64 for one query row against the keys it may see."""
    s = (K.astype(np.float64) @ q_row.astype(np.float64)) * inv_t
    w = np.exp(s - s.max())
    return (w / w.sum()) @ V.astype(np.float64)


def test_causal_prefill_full_size(dev):
    """Long-context causal prefill: batch 4, 16 heads, seq 8192, d 128 (tensor-core kernel)."""
    from dl4s_b200.layers import ScaledDotProductAttention
    B, H, S, d = 4, 16, 8192, 128
    q, k, v = (np.random.default_rng(s).standard_normal((B, H, S, d), dtype=np.float32) for s in (1, 2, 3))
    attn = ScaledDotProductAttention(float(np.sqrt(np.float32(d))), precision=PREC_F16)
    tq, tk, tv = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    causal = dev.StructuredMask(None, causal=True)
    out = attn(tq, tk, tv, causal).numpy()
    assert np.isfinite(out).all()
    assert max_abs(out[:, :, 0], v[:, :, 0]) < TC_MAX_ABS                       # row 0 sees key 0 only
    # sampled rows against the exact value: first / last rows of tiles, the diagonal tile, the longest rows
    rng = np.random.default_rng(5)
    rows = [1, 127, 128, 255, 256, 4095, 4096, 8190, 8191] + rng.integers(0, S, size=40).tolist()
    got, want = [], []
    for i, r in enumerate(rows):
        b, h = (i * 7) % B, (i * 5) % H
        got.append(out[b, h, r])
        want.append(exact_row(q[b, h, r], k[b, h, :r + 1], v[b, h, :r + 1], 1.0 / np.sqrt(np.float64(d))))
    assert_tc(np.array(got), np.array(want), "sampled rows of the full causal problem")
    # the causal prefix: the first 1024 rows do not depend on what follows
    half = attn(dev.tensor(q[:, :, :1024]), dev.tensor(k[:, :, :1024]), dev.tensor(v[:, :, :1024]), causal).numpy()
    assert max_abs(out[:, :, :1024], half) < TC_MAX_ABS
    # rows of the softmax sum to one: with V = 1 every output is 1
    ones = dev.tensor(np.ones((B, H, S, d), np.float32))
    assert max_abs(attn(tq, tk, ones, causal).numpy(), 1.0) < TC_MAX_ABS


def test_decode_full_size(dev):
    """Decode attention: batch 64, 32 heads, context <= 4096 with ragged lengths, d 128 (fp32 split-K kernels).
    K and V are one seeded [H, L, d] slab per tensor repeated for every batch element (8.6 GB of host random numbers
    would take minutes to draw and upload); lengths and queries differ per batch element."""
    from dl4s_b200.layers import ScaledDotProductAttention
    B, H, L, d = 64, 32, 4096, 128
    rng = np.random.default_rng(2)
    lens = np.random.default_rng(4).integers(1024, L + 1, size=B).astype(np.int32)
    q = rng.standard_normal((B, H, 1, d), dtype=np.float32)
    slab_k = rng.standard_normal((H, L, d), dtype=np.float32)
    slab_v = rng.standard_normal((H, L, d), dtype=np.float32)
    M = dev.CUDA.Memory
    k, v = M.allocateBuffer((B, H, L, d)), M.allocateBuffer((B, H, L, d))
    sk, sv = dev.tensor(slab_k), dev.tensor(slab_v)
    for b in range(B):
        M.assign(sk, M.advance(k.view(-1), b * H * L * d), H * L * d)
        M.assign(sv, M.advance(v.view(-1), b * H * L * d), H * L * d)
    out = M.allocateBuffer((B, H, 1, d))
    mask = dev.StructuredMask(lens, max_len=L)
    dev.CUDAEngine.scaledDotProductAttentionDecode(dev.tensor(q), k, v, mask.lengths, float(np.sqrt(np.float32(d))), out)
    got = out.numpy()
    assert np.isfinite(got).all()
    inv_t = 1.0 / np.sqrt(np.float64(d))
    worst = 0.0
    for b in range(B):                      # every batch element, four heads each
        for h in ((b * 3) % H, (b * 3 + 11) % H, 0, H - 1):
            n = int(lens[b])
            want = exact_row(q[b, h, 0], slab_k[h, :n], slab_v[h, :n], inv_t)
            worst = max(worst, float(np.abs(got[b, h, 0] - want).max()))
    assert worst <= 1e-5, f"decode differs from the exact value by {worst:.2e}"


@pytest.mark.parametrize("prec", ["f16", "f16_split"])
def test_encoder_full_size(dev, oracle, prec):
    """The 6-layer encoder at batch 32, seq 512 (padding mask) on the tensor-core paths against the float64 numpy
    formulation of the same op sequence (all 32 sequences) and against the C restatement of the CPU engine on two
    of them (sequences do not interact, so a sequence's output does not depend on the batch it is in)."""
    from dl4s_b200 import PREC_F16_SPLIT
    from dl4s_b200.layers import TransformerEncoder
    from oracle import oracle_np as ON
    c = workloads.encoder_config()
    p = PREC_F16 if prec == "f16" else PREC_F16_SPLIT
    enc = TransformerEncoder(6, c["heads"], c["dk"], c["dv"], 512, c["F"], layers=c["layers"], precision=p)
    got = enc(dev.tensor(c["x"]), c["lengths"]).numpy()
    assert dev.device_status() == 0
    want = ON.encoder(c["x"], c["layers"], c["heads"], c["lengths"])
    assert np.isfinite(got).all()
    ma, rl = max_abs(got, want), rel_l2(got, want)
    print(f"encoder 6 x [32,512,512] {prec}: max-abs {ma:.3e}, rel-L2 {rl:.3e} (max |want| {np.abs(want).max():.2f})")
    # the CPU engine itself (fp32, reference evaluation order) on the longest and on a padded sequence
    pick = [0, int(np.argmin(c["lengths"]))]
    want_c = oracle.encoder(c["x"][pick], c["layers"], c["heads"], c["lengths"][pick])
    ma_c, rl_c = max_abs(got[pick], want_c), rel_l2(got[pick], want_c)
    print(f"  against the C restatement on sequences {pick}: max-abs {ma_c:.3e}, rel-L2 {rl_c:.3e}")
    assert rl <= TC_REL_L2 and rl_c <= TC_REL_L2, (rl, rl_c)
    if prec == "f16_split":
        assert ma <= TC_MAX_ABS and ma_c <= TC_MAX_ABS, (ma, ma_c)
    else:
        assert ma <= F16_DEEP_MAX_ABS_DOCUMENTED and ma_c <= F16_DEEP_MAX_ABS_DOCUMENTED, (ma, ma_c)


def test_head_sharded_layer_full_width(dev):
    """The head-sharded decoder self-attention layer at its full sequence length, model width and head count (S 2048,
    D 4096, 32 heads of 128, causal), two batch elements instead of 256: batch elements are independent (the LayerNorm
    inside MultiHeadAttention is per batch element), so one of them checked against a float64 evaluation of the whole
    layer is a full-size check of everything but the batch loop. Runs through dl4s_cuda_mha_forward_sharded with a
    world of one (same kernels and chunking as the multi-GPU runs, no collective)."""
    from dl4s_b200 import sharded
    from dl4s_b200.layers import xavier_uniform
    B, S, D, H = 2, 2048, 4096, 32
    dk = D // H
    rw = np.random.default_rng(0)
    w = {n: xavier_uniform(rw, D, D) for n in ("qDense", "kDense", "vDense", "fc")}
    x = np.random.default_rng(1).standard_normal((B, S, D), dtype=np.float32)
    layer = sharded.HeadShardedMultiHeadAttention(H, D, dk, dk, w, precision=PREC_F16, chunks=2)
    got = layer(dev.tensor(x), dev.StructuredMask(None, causal=True)).numpy()
    assert got.shape == (B, S, D) and np.isfinite(got).all()
    # float64, batch element 1, head by head (the [S,S] scores of one head at a time)
    xb = x[1].astype(np.float64)
    q, k, v = (xb @ w[n].astype(np.float64) for n in ("qDense", "kDense", "vDense"))
    heads = np.empty((S, D))
    blocked = np.triu(np.ones((S, S), bool), 1)
    for h in range(H):
        sl = slice(h * dk, (h + 1) * dk)
        s = (q[:, sl] / np.sqrt(np.float64(dk))) @ k[:, sl].T
        s[blocked] -= 1e9
        e = np.exp(s - s.max(axis=1, keepdims=True))
        heads[:, sl] = (e / e.sum(axis=1, keepdims=True)) @ v[:, sl]
    z = heads @ w["fc"].astype(np.float64) + xb
    m = z.mean()
    want = (z - m) / (np.sqrt((z * z).mean() - m * m) + 1e-5)        # LayerNorm over the whole [S, D] block, scale 1, shift 0
    ma, rl = max_abs(got[1], want), rel_l2(got[1], want)
    print(f"head-sharded layer, S {S}, D {D}, {H} heads, batch element 1 of {B}: max-abs {ma:.3e}, rel-L2 {rl:.3e}")
    assert_tc(got[1], want, "head-sharded layer at full width against float64")
