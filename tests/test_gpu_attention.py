"""GPU tier: ScaledDotProductAttention through the C ABI against the CPU oracle.

fp32 mode must agree to 1e-5, tensor-core mode to max-abs 2e-3 and relative L2 1e-3."""
import numpy as np
import pytest

from dl4s_b200 import PREC_F16, PREC_FP32
from util import assert_close, assert_fp32, assert_tc, golden, max_abs

pytestmark = pytest.mark.gpu


def check(prec, got, want, what):
    (assert_fp32 if prec == PREC_FP32 else assert_tc)(got, want, what)


def run_sdpa(dev, q, k, v, mask=None, prec=PREC_FP32):
    from dl4s_b200.layers import ScaledDotProductAttention
    attn = ScaledDotProductAttention(float(np.sqrt(np.float32(q.shape[-1]))), precision=prec)
    if isinstance(mask, np.ndarray):
        mask = dev.tensor(mask)
    return attn(dev.tensor(q), dev.tensor(k), dev.tensor(v), mask).numpy()


def rand_qkv(rng, B, H, Sq, Sk, dk, dv):
    return (rng.standard_normal((B, H, Sq, dk), dtype=np.float32), rng.standard_normal((B, H, Sk, dk), dtype=np.float32),
            rng.standard_normal((B, H, Sk, dv), dtype=np.float32))


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_golden_vectors(dev, prec):
    g = golden()
    q, k, v = g["sdpa_q"], g["sdpa_k"], g["sdpa_v"]
    check(prec, run_sdpa(dev, q, k, v, None, prec), g["sdpa_nomask"], "no mask")
    check(prec, run_sdpa(dev, q, k, v, dev.makeEncoderMasks(g["sdpa_lens"]), prec), g["sdpa_padmask"], "padding")
    check(prec, run_sdpa(dev, q, k, v, dev.StructuredMask(g["sdpa_lens0"], max_len=7), prec), g["sdpa_fullmask"],
          "fully blocked sequence")
    check(prec, run_sdpa(dev, g["causal_q"], g["causal_k"], g["causal_v"], dev.makeDecoderMasks(g["causal_lens"]), prec),
          g["causal_out"], "decoder mask")


def test_dense_masks_fp32(dev, oracle):
    rng = np.random.default_rng(10)
    B, H, Sq, Sk = 2, 3, 9, 13
    q, k, v = rand_qkv(rng, B, H, Sq, Sk, 16, 8)
    for shape in ((B, 1, 1, Sk), (1, 1, Sq, Sk), (B, H, Sq, Sk), (1, H, 1, 1)):
        m = (rng.random(shape) < 0.3).astype(np.float32)
        assert_fp32(run_sdpa(dev, q, k, v, m), oracle.sdpa(q, k, v, m), f"dense mask {shape}")


SHAPES = [  # B, H, Sq, Sk, dk, dv
    (1, 1, 1, 1, 8, 8), (2, 3, 5, 7, 8, 4), (1, 2, 128, 128, 64, 64), (2, 2, 130, 257, 64, 64),
    (1, 2, 256, 256, 128, 128), (1, 1, 300, 515, 128, 128), (2, 1, 64, 1000, 32, 32), (1, 1, 513, 129, 16, 16),
]


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_shapes_no_mask(dev, oracle, prec, shape):
    rng = np.random.default_rng(11)
    q, k, v = rand_qkv(rng, *shape)
    check(prec, run_sdpa(dev, q, k, v, None, prec), oracle.sdpa(q, k, v), f"{shape}")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
@pytest.mark.parametrize("B,H,S,d", [(3, 2, 200, 64), (2, 2, 384, 128), (4, 1, 129, 64), (2, 1, 640, 128)])
def test_padding_and_causal(dev, oracle, prec, B, H, S, d):
    rng = np.random.default_rng(12)
    q, k, v = rand_qkv(rng, B, H, S, S, d, d)
    lens = rng.integers(1, S + 1, size=B).astype(np.int32)
    lens[0] = S
    check(prec, run_sdpa(dev, q, k, v, dev.makeEncoderMasks(lens), prec), oracle.sdpa(q, k, v, oracle.make_encoder_mask(lens, S)),
          "padding mask")
    check(prec, run_sdpa(dev, q, k, v, dev.makeDecoderMasks(lens), prec), oracle.sdpa(q, k, v, oracle.make_decoder_mask(lens, S)),
          "decoder mask")
    check(prec, run_sdpa(dev, q, k, v, dev.StructuredMask(None, causal=True), prec),
          oracle.sdpa(q, k, v, oracle.make_decoder_mask(np.full(B, S, np.int32), S)), "causal only")


def test_many_items_per_resident_cta(dev, oracle):
    """64-wide heads with a padding mask take the persistent kernel; 1152 (query block, batch x head) items over at most
    296 resident CTAs make every CTA walk 3-4 items with different key-tile counts (1-3), a blocked sequence and a full
    one among them: Q buffers, barrier phases and the output accumulator are reused across items."""
    rng = np.random.default_rng(21)
    B, H, S, d = 48, 8, 320, 64
    q, k, v = rand_qkv(rng, B, H, S, S, d, d)
    lens = rng.integers(1, S + 1, size=B).astype(np.int32)
    lens[0], lens[1], lens[2], lens[3] = S, 0, 128, 129
    got = run_sdpa(dev, q, k, v, dev.makeEncoderMasks(lens), PREC_F16)
    check(PREC_F16, got, oracle.sdpa(q, k, v, oracle.make_encoder_mask(lens, S)), "persistent form, ragged lengths")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_fully_blocked_sequence_is_uniform(dev, prec):
    """The reference subtracts a finite 1e9, so a sequence of length 0 averages ALL value rows."""
    rng = np.random.default_rng(13)
    q, k, v = rand_qkv(rng, 2, 2, 140, 140, 64, 64)
    out = run_sdpa(dev, q, k, v, dev.StructuredMask(np.array([0, 140], np.int32), max_len=140), prec)
    want = np.broadcast_to(v[0].mean(axis=1, keepdims=True), out[0].shape)
    assert max_abs(out[0], want) < (1e-5 if prec == PREC_FP32 else 2e-3)


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_properties_at_scale(dev, prec):
    """Size-independent checks on a long causal problem (S=2048, d=128) that the CPU oracle does not run."""
    rng = np.random.default_rng(14)
    B, H, S, d = 1, 2, 2048, 128
    q, k, v = rand_qkv(rng, B, H, S, S, d, d)
    causal = dev.StructuredMask(None, causal=True)
    tol = 1e-5 if prec == PREC_FP32 else 2e-3
    out = run_sdpa(dev, q, k, v, causal, prec)
    assert max_abs(out[:, :, 0], v[:, :, 0]) < tol                      # row 0 sees key 0 only
    half = run_sdpa(dev, q[:, :, :1024], k[:, :, :1024], v[:, :, :1024], causal, prec)
    assert max_abs(out[:, :, :1024], half) < tol                        # causal prefix property
    ones = np.ones_like(v)
    assert max_abs(run_sdpa(dev, q, k, ones, causal, prec), ones) < tol  # rows of the softmax sum to one
    out2 = run_sdpa(dev, q, k, 2 * v, causal, prec)
    assert max_abs(out2, 2 * out) < 2 * tol                             # linear in v
    zq = run_sdpa(dev, np.zeros_like(q), k, v, None, prec)              # q = 0: plain mean of the values
    assert max_abs(zq, np.broadcast_to(v.mean(axis=2, keepdims=True), zq.shape)) < tol


@pytest.mark.parametrize("B,H,L,d,min_len", [(2, 2, 300, 128, 1), (3, 4, 1000, 64, 100), (2, 2, 4096, 128, 1024),
                                              (1, 1, 256, 128, 256), (2, 3, 77, 32, 5)])
def test_decode_against_oracle(dev, oracle, B, H, L, d, min_len):
    rng = np.random.default_rng(15)
    q, k, v = rand_qkv(rng, B, H, 1, L, d, d)
    lens = rng.integers(min_len, L + 1, size=B).astype(np.int32)
    # poison rows beyond each length: they must never influence (or be read into) the result
    for b in range(B):
        k[b, :, lens[b]:] = np.nan
        v[b, :, lens[b]:] = np.nan
    from dl4s_b200.layers import ScaledDotProductAttention
    attn = ScaledDotProductAttention(float(np.sqrt(np.float32(d))))
    mask = dev.StructuredMask(lens, max_len=L)
    got = attn(dev.tensor(q), dev.tensor(k), dev.tensor(v), mask).numpy()
    kk, vv = np.nan_to_num(k), np.nan_to_num(v)
    assert_fp32(got, oracle.sdpa(q, kk, vv, oracle.make_encoder_mask(lens, L)), "decode")
    # no lengths: all rows
    k2, v2 = rng.standard_normal(k.shape, dtype=np.float32), rng.standard_normal(v.shape, dtype=np.float32)
    got = attn(dev.tensor(q), dev.tensor(k2), dev.tensor(v2), None).numpy()
    assert_fp32(got, oracle.sdpa(q, k2, v2), "decode without lengths")


def test_decode_length_beyond_the_cache_is_clamped(dev, oracle):
    """A device-side length above Lmax reads the Lmax rows that exist (the prefill and fp32 kernels clamp the same way);
    Lmax is not a multiple of the 256-key chunk, so an unclamped length would walk past the last head's rows."""
    rng = np.random.default_rng(17)
    B, H, L, d = 2, 3, 300, 128
    q, k, v = rand_qkv(rng, B, H, 1, L, d, d)
    lens = np.array([L + 5, 120], np.int32)
    from dl4s_b200.layers import ScaledDotProductAttention
    attn = ScaledDotProductAttention(float(np.sqrt(np.float32(d))))
    got = attn(dev.tensor(q), dev.tensor(k), dev.tensor(v), dev.StructuredMask(lens, max_len=L)).numpy()
    want = oracle.sdpa(q, k, v, oracle.make_encoder_mask(np.minimum(lens, L), L))
    assert_fp32(got, want, "decode with a length above Lmax")


def test_decode_length_zero_is_uniform(dev):
    rng = np.random.default_rng(16)
    q, k, v = rand_qkv(rng, 2, 2, 1, 300, 128, 128)
    from dl4s_b200.layers import ScaledDotProductAttention
    attn = ScaledDotProductAttention(float(np.sqrt(np.float32(128))))
    out = attn(dev.tensor(q), dev.tensor(k), dev.tensor(v), dev.StructuredMask(np.array([0, 300], np.int32), max_len=300)).numpy()
    assert max_abs(out[0], v[0].mean(axis=1, keepdims=True)) < 1e-5


@pytest.mark.parametrize("B,H,Sq,Sk,dk,dv,kind", [(2, 2, 9, 9, 5, 5, "causal"), (2, 3, 70, 70, 64, 64, "causal"),
                                                 (3, 2, 50, 131, 32, 48, "padding"), (1, 2, 130, 130, 128, 128, "none"),
                                                 (2, 1, 33, 33, 16, 16, "dense")])
def test_sdpa_backward_against_oracle(dev, oracle, B, H, Sq, Sk, dk, dv, kind):
    """dq, dk, dv for an upstream gradient against the CPU engine's gradients (fp32, 1e-5), with every mask kind and
    a sequence of length 0 (all keys blocked: uniform weights, gradients still defined)."""
    from dl4s_b200.layers import scaledDotProductAttentionBackward
    rng = np.random.default_rng(80 + Sq)
    q = rng.standard_normal((B, H, Sq, dk), dtype=np.float32)
    k = rng.standard_normal((B, H, Sk, dk), dtype=np.float32)
    v = rng.standard_normal((B, H, Sk, dv), dtype=np.float32)
    g = rng.standard_normal((B, H, Sq, dv), dtype=np.float32)
    lens = np.array([Sk, max(1, Sk // 3), 0][:B], np.int32)
    if kind == "causal":
        mask, want_mask = dev.makeDecoderMasks(lens), oracle.make_decoder_mask(lens, Sk)
    elif kind == "padding":
        mask, want_mask = dev.makeEncoderMasks(lens), oracle.make_encoder_mask(lens, Sk)
    elif kind == "dense":
        m = (rng.random((B, 1, Sq, Sk)) < 0.3).astype(np.float32)
        m[..., 0] = 0.0
        mask, want_mask = dev.tensor(m), m
    else:
        mask, want_mask = None, None
    dq, dkk, dvv = scaledDotProductAttentionBackward(dev.tensor(q), dev.tensor(k), dev.tensor(v), dev.tensor(g), mask)
    wq, wk, wv = oracle.sdpa_backward(q, k, v, g, want_mask)
    assert_fp32(dq.numpy(), wq, "dq")
    assert_fp32(dkk.numpy(), wk, "dk")
    assert_fp32(dvv.numpy(), wv, "dv")


@pytest.mark.parametrize("B,H,Sq,Sk,d,kind", [(2, 2, 256, 256, 64, "causal"), (3, 2, 300, 300, 128, "padding"), (2, 3, 130, 130, 64, "none"),
                                              (1, 2, 200, 330, 64, "padding"), (3, 2, 384, 384, 128, "causal"),
                                              (4, 8, 512, 512, 64, "padding"), (1, 2, 1024, 1024, 128, "causal"), (1, 1, 70, 70, 64, "causal")],
                         ids=["causal-d64", "padding-d128", "odd-rows", "cross-lengths", "causal-d128", "encoder-shape", "long-causal",
                              "one-tile"])
def test_sdpa_backward_tensor_cores(dev, oracle, B, H, Sq, Sk, d, kind):
    """The flash-style tensor-core backward (S and dP recomputed per key tile; dV, dK, dQ by tcgen05 MMAs) against the
    CPU engine's gradients: max-abs 2e-3 and relative L2 1e-3 per gradient, every structural mask kind, ragged last
    tiles, Sq != Sk, a sequence of length 0 (uniform weights, gradients still flow) and key tiles past a length
    (zero gradients)."""
    from dl4s_b200 import PREC_F16
    from dl4s_b200.layers import scaledDotProductAttentionBackward
    rng = np.random.default_rng(90 + Sq + d)
    q = rng.standard_normal((B, H, Sq, d), dtype=np.float32)
    k = rng.standard_normal((B, H, Sk, d), dtype=np.float32)
    v = rng.standard_normal((B, H, Sk, d), dtype=np.float32)
    g = rng.standard_normal((B, H, Sq, d), dtype=np.float32)
    lens = np.array([Sk, max(1, Sk // 3), 0, Sk - 5][:B], np.int32)
    if kind == "causal":
        mask, want_mask = dev.makeDecoderMasks(lens), oracle.make_decoder_mask(lens, Sk)
    elif kind == "padding":
        mask, want_mask = dev.makeEncoderMasks(lens), oracle.make_encoder_mask(lens, Sk)
    else:
        mask, want_mask = None, None
    dq, dkk, dvv = scaledDotProductAttentionBackward(dev.tensor(q), dev.tensor(k), dev.tensor(v), dev.tensor(g), mask, precision=PREC_F16)
    wq, wk, wv = oracle.sdpa_backward(q, k, v, g, want_mask)
    assert_tc(dq.numpy(), wq, "dq")
    assert_tc(dkk.numpy(), wk, "dk")
    assert_tc(dvv.numpy(), wv, "dv")
    assert dev.device_status() == 0
