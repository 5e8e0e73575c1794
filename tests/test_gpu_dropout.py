"""GPU tier: dropout as the reference applies it (NN/Layer/Dropout.swift:47-55: x * bernoulli(1 - rate), no rescaling)
with the mask computed on the device by a counter-based hash. The host regenerates every mask from (seed, counter,
element index) and the expected values are the CPU oracle's layers with that mask multiplied in at the reference's
places: MultiHeadAttention.swift:122, PointwiseFeedForward.swift:78, Transformer.swift:87."""
import ctypes

import numpy as np
import pytest

from dl4s_b200 import PREC_F16, PREC_FP32, workloads
from dl4s_b200 import layers as L
from util import assert_fp32, assert_tc, dropout_keep_mask

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def dropout_off_afterwards():
    yield
    L.setDropout(0.0)


def check(prec, got, want, what):
    (assert_fp32 if prec == PREC_FP32 else assert_tc)(got, want, what)


def oracle_mha_dropout(O, x, W, H, mask, keep):
    B, S, D = x.shape
    dk = W["qDense"].shape[1] // H
    sp = lambda t: np.ascontiguousarray(t.reshape(B, S, H, dk).transpose(0, 2, 1, 3))
    q, k, v = (sp(O.gemm(x.reshape(-1, D), W[n])) for n in ("qDense", "kDense", "vDense"))
    a = np.ascontiguousarray(O.sdpa(q, k, v, mask).transpose(0, 2, 1, 3)).reshape(B * S, H * dk)
    out = O.gemm(a, W["fc"]).reshape(B, S, D) * keep            # out_drop = dropout(out)
    return O.layernorm(out + x, np.ones(D, np.float32), np.zeros(D, np.float32))


def oracle_ffn_dropout(O, x, w, keep):
    from oracle import oracle_np as ON
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    h = ON.gelu_sigmoid((O.gemm(x2, w["W1"]) + w["b1"]).astype(np.float32), dtype=np.float32).astype(np.float32)
    o = (O.gemm(h, w["W2"]) + w["b2"]).astype(np.float32) * keep.reshape(-1, D)     # tmp4 = dropout(tmp3)
    return O.layernorm((o + x2).astype(np.float32), w["ln2_scale"], w["ln2_shift"]).reshape(x.shape)


def test_dropout_layer_mask_can_be_regenerated(dev):
    x = np.arange(1, 1 + 3 * 1000, dtype=np.float32).reshape(3, 1000)
    for rate, seed, counter in ((0.1, 7, 0), (0.5, (5 << 32) | 123, 9), (0.9, 1, 4000000000)):
        out = dev.CUDA.Memory.allocateBuffer(x.shape)
        L.call("dl4s_cuda_dropout", ctypes.c_void_p(dev.tensor(x).ptr), ctypes.c_void_p(out.ptr), x.size, ctypes.c_float(rate), seed,
               counter)
        keep = dropout_keep_mask(x.shape, rate, seed, counter)
        assert np.array_equal(out.numpy(), x * keep)
        assert abs(keep.mean() - (1 - rate)) < 0.03
    # different sites draw different masks
    assert not np.array_equal(dropout_keep_mask((1000,), 0.5, 7, 0), dropout_keep_mask((1000,), 0.5, 7, 1))
    layer = L.Dropout(0.3, seed=11)
    c0 = L.dropoutCounter()
    got = layer(dev.tensor(x)).numpy()
    assert np.array_equal(got, x * dropout_keep_mask(x.shape, 0.3, 11, c0)) and L.dropoutCounter() == c0 + 1
    layer.isActive = False
    t = dev.tensor(x)
    assert layer(t) is t


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_mha_and_ffn_with_dropout(dev, oracle, prec):
    rate, seed = 0.1, 42
    c = workloads.mha_config(B=3, S=128, D=256, H=4)
    x = c["x"]
    mha = L.MultiHeadAttention(4, 256, 64, 64, weights=c["weights"], precision=prec)
    L.setDropout(rate, seed)
    L.dropoutCounter(set_to=100)
    tx = dev.tensor(x)
    got = mha(tx, tx, tx, dev.StructuredMask(None, causal=True)).numpy()
    assert L.dropoutCounter() == 101                                 # one site
    keep = dropout_keep_mask(x.shape, rate, seed, 100)
    want = oracle_mha_dropout(oracle, x, c["weights"], 4, oracle.make_decoder_mask(np.full(3, 128, np.int32), 128), keep)
    check(prec, got, want, "MultiHeadAttention with dropout on the output projection")
    # without the mask the result is a different one
    L.setDropout(0.0)
    assert np.abs(mha(tx, tx, tx, dev.StructuredMask(None, causal=True)).numpy() - got).max() > 0.05
    # feed-forward
    rng = np.random.default_rng(70)
    w = L.encoder_layer_weights(rng, 256, 4, 64, 64, 1024)
    w["b1"] = (0.1 * rng.standard_normal(1024)).astype(np.float32)
    w["b2"] = (0.1 * rng.standard_normal(256)).astype(np.float32)
    ffn = L.PointwiseFeedForward(256, 1024, weights={"W1": w["W1"], "b1": w["b1"], "W2": w["W2"], "b2": w["b2"]}, precision=prec)
    L.setDropout(rate, seed)
    L.dropoutCounter(set_to=7)
    got = ffn(tx).numpy()
    keep = dropout_keep_mask(x.shape, rate, seed, 7)
    check(prec, got, oracle_ffn_dropout(oracle, x, w, keep), "PointwiseFeedForward with dropout after the second Dense")
    assert dev.device_status() == 0


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_encoder_and_embedding_with_dropout(dev, oracle, prec):
    """Two encoder layers: sites are taken in call order (layer 0 attention, layer 0 feed-forward, layer 1 ...)."""
    rate, seed = 0.2, 5
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=300)
    enc = L.TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=prec)
    emb = L.EmbeddingWithPositions(c["embedding"])
    L.setDropout(rate, seed)
    L.dropoutCounter(set_to=0)
    x_dev = emb(dev.tensor(c["ids"], np.int32))                       # site 0: the embedded inputs
    x = (oracle.embed(c["ids"], c["embedding"], -1) * dropout_keep_mask(c["x"].shape, rate, seed, 0)).astype(np.float32)
    assert_fp32(x_dev.numpy(), x, "embedded inputs with dropout")
    got = enc(x_dev, c["lengths"]).numpy()
    assert L.dropoutCounter() == 5
    cur = x
    mask = oracle.make_encoder_mask(c["lengths"], 128)
    for li, lw in enumerate(c["layers"]):
        W = {"qDense": lw["Wq"], "kDense": lw["Wk"], "vDense": lw["Wv"], "fc": lw["Wo"]}
        y = oracle_mha_dropout(oracle, cur, W, 8, mask, dropout_keep_mask(cur.shape, rate, seed, 1 + 2 * li))
        cur = oracle_ffn_dropout(oracle, y, lw, dropout_keep_mask(cur.shape, rate, seed, 2 + 2 * li))
    check(prec, got, cur, "encoder with dropout at both sites of both layers")
    assert dev.device_status() == 0
