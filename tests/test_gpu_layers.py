"""GPU tier: LayerNorm, MultiHeadAttention, PointwiseFeedForward, TransformerEncoder and the input preparation
through the C ABI against the CPU oracle, in both arithmetic modes."""
import numpy as np
import pytest

from dl4s_b200 import ACT_RELU, PREC_F16, PREC_F16_SPLIT, PREC_FP32
from dl4s_b200 import workloads
from util import assert_fp32, assert_fp32_rel, assert_tc, golden, max_abs, unpack_layers

pytestmark = pytest.mark.gpu


def check(prec, got, want, what):
    (assert_fp32 if prec == PREC_FP32 else assert_tc)(got, want, what)


def test_layernorm_golden_and_flavours(dev, oracle):
    from dl4s_b200.layers import LayerNorm
    g = golden()
    ln = LayerNorm([8])
    ln.scale, ln.shift = dev.tensor(g["ln_scale"]), dev.tensor(g["ln_shift"])
    assert_fp32(ln(dev.tensor(g["ln_x"])).numpy(), g["ln_out3d"], "3-D: per batch element over [rows, D]")
    assert_fp32(ln(dev.tensor(g["ln_x"].reshape(6, 8))).numpy(), g["ln_out2d"], "2-D: per row")
    rng = np.random.default_rng(20)
    for shape in ((3, 17, 64), (2, 128, 512), (100, 512), (1, 5, 16), (5, 1, 16)):
        x = (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32)
        r = rng.standard_normal(shape).astype(np.float32)
        D = shape[-1]
        sc = rng.standard_normal(D).astype(np.float32)
        sh = rng.standard_normal(D).astype(np.float32)
        ln = LayerNorm([D])
        ln.scale, ln.shift = dev.tensor(sc), dev.tensor(sh)
        assert_fp32(ln(dev.tensor(x)).numpy(), oracle.layernorm(x, sc, sh), f"{shape}")
        assert_fp32(ln(dev.tensor(x), dev.tensor(r)).numpy(), oracle.layernorm(x + r, sc, sh), f"{shape} + residual")


def test_layernorm_chunked_statistics(dev, oracle):
    """One statistic block spread over several thread blocks (the MultiHeadAttention flavour at encoder sizes)."""
    from dl4s_b200.layers import LayerNorm
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((4, 512, 512)) * 1.5 - 0.25).astype(np.float32)
    ln = LayerNorm([512])
    got = ln(dev.tensor(x)).numpy()
    assert_fp32(got, oracle.layernorm(x, np.ones(512, np.float32), np.zeros(512, np.float32)), "chunked")
    assert np.abs(got.reshape(4, -1).mean(axis=1)).max() < 1e-5


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16, PREC_F16_SPLIT], ids=["fp32", "f16", "f16_split"])
def test_mha_golden(dev, prec):
    from dl4s_b200.layers import MultiHeadAttention
    g = golden()
    mha = MultiHeadAttention(4, 16, 4, 4, weights={"qDense": g["mha_Wq"], "kDense": g["mha_Wk"], "vDense": g["mha_Wv"],
                                                   "fc": g["mha_Wo"]}, precision=prec)
    x = dev.tensor(g["mha_x"])
    check(prec, mha(x, x, x, dev.makeEncoderMasks(g["causal_lens"])).numpy(), g["mha_out"], "mha golden")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16, PREC_F16_SPLIT], ids=["fp32", "f16", "f16_split"])
def test_mha_config1_full_size(dev, oracle, prec):
    """MultiHeadAttention forward, batch 8, seq 128, d_model 512, 8 heads, no mask, compared elementwise."""
    from dl4s_b200.layers import MultiHeadAttention
    c = workloads.mha_config()
    w = c["weights"]
    mha = MultiHeadAttention(8, 512, 64, 64, weights=w, precision=prec)
    x = dev.tensor(c["x"])
    got = mha(x, x, x, None).numpy()
    one, zero = np.ones(512, np.float32), np.zeros(512, np.float32)
    want = oracle.mha(c["x"], c["x"], c["x"], w["qDense"], w["kDense"], w["vDense"], w["fc"], one, zero, 8)
    check(prec, got, want, "config 1")


def test_mha_wide_model_takes_the_paired_output_projection(dev, oracle):
    """d_model 1024 with 16 heads of 64: the output projection has K = 1024, which selects the two-CTA tiles, and its
    epilogue leaves the LayerNorm statistics (rows a multiple of 32). Compared elementwise with the oracle."""
    from dl4s_b200.layers import MultiHeadAttention
    rng = np.random.default_rng(27)
    B, S, D, H = 2, 256, 1024, 16
    x = rng.standard_normal((B, S, D), dtype=np.float32)
    mha = MultiHeadAttention(H, D, 64, 64, rng=rng, precision=PREC_F16)
    w = mha.host_weights
    sc = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    sh = (0.1 * rng.standard_normal(D)).astype(np.float32)
    mha.norm.scale, mha.norm.shift = dev.tensor(sc), dev.tensor(sh)
    lens = np.array([256, 100], np.int32)
    got = mha(dev.tensor(x), dev.tensor(x), dev.tensor(x), dev.makeDecoderMasks(lens)).numpy()
    want = oracle.mha(x, x, x, w["qDense"], w["kDense"], w["vDense"], w["fc"], sc, sh, H, oracle.make_decoder_mask(lens, S))
    assert_tc(got, want, "wide model")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_mha_cross_attention_and_masks(dev, oracle, prec):
    from dl4s_b200.layers import MultiHeadAttention
    rng = np.random.default_rng(22)
    B, Sq, Sk, D, H = 2, 70, 150, 128, 2
    xq = rng.standard_normal((B, Sq, D), dtype=np.float32)
    xk = rng.standard_normal((B, Sk, D), dtype=np.float32)
    mha = MultiHeadAttention(H, D, 64, 64, rng=rng, precision=prec)
    w = mha.host_weights
    one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
    lens = np.array([150, 31], np.int32)
    got = mha(dev.tensor(xq), dev.tensor(xk), dev.tensor(xk), dev.makeEncoderMasks(lens)).numpy()
    want = oracle.mha(xq, xk, xk, w["qDense"], w["kDense"], w["vDense"], w["fc"], one, zero, H, oracle.make_encoder_mask(lens, Sk))
    check(prec, got, want, "cross attention with padding")
    xs = rng.standard_normal((B, Sk, D), dtype=np.float32)
    got = mha(dev.tensor(xs), dev.tensor(xs), dev.tensor(xs), dev.makeDecoderMasks(lens)).numpy()
    want = oracle.mha(xs, xs, xs, w["qDense"], w["kDense"], w["vDense"], w["fc"], one, zero, H, oracle.make_decoder_mask(lens, Sk))
    check(prec, got, want, "decoder self-attention")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16, PREC_F16_SPLIT], ids=["fp32", "f16", "f16_split"])
def test_ffn(dev, oracle, prec):
    from dl4s_b200.layers import PointwiseFeedForward
    g = golden()
    w = {"W1": g["ffn_W1"], "b1": g["ffn_b1"], "W2": g["ffn_W2"], "b2": g["ffn_b2"]}
    x = dev.tensor(g["mha_x"])
    check(prec, PointwiseFeedForward(16, 32, weights=w, precision=prec)(x).numpy(), g["ffn_out"], "ffn golden (GeLU)")
    check(prec, PointwiseFeedForward(16, 32, weights=w, activation=ACT_RELU, precision=prec)(x).numpy(), g["ffn_out_relu"],
          "ffn golden (ReLU)")
    rng = np.random.default_rng(23)
    D, F, M = 256, 1024, 300
    ffn = PointwiseFeedForward(D, F, rng=rng, precision=prec)
    xb = rng.standard_normal((3, 100, D), dtype=np.float32)
    one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
    want = oracle.ffn(xb, ffn.dense1.host_weights, ffn.dense1.host_bias, ffn.dense2.host_weights, ffn.dense2.host_bias, one, zero)
    check(prec, ffn(dev.tensor(xb)).numpy(), want, "ffn 256->1024")


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16, PREC_F16_SPLIT], ids=["fp32", "f16", "f16_split"])
def test_encoder_golden_and_midsize(dev, oracle, prec):
    from dl4s_b200.layers import TransformerEncoder
    g = golden()
    layers = unpack_layers(g["enc_params"], 16, 4, 4, 4, 32, 2)
    enc = TransformerEncoder(2, 4, 4, 4, 16, 32, layers=layers, precision=prec)
    check(prec, enc(dev.tensor(g["mha_x"]), g["causal_lens"]).numpy(), g["enc_out"], "encoder golden")
    # the benchmark's architecture at a size the oracle finishes in seconds
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000)
    enc = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=prec)
    got = enc(dev.tensor(c["x"]), c["lengths"]).numpy()
    want = oracle.encoder(c["x"], c["layers"], 8, c["lengths"])
    check(prec, got, want, "encoder 2 x [2,128,512]")


@pytest.mark.parametrize("prec", [PREC_F16, PREC_F16_SPLIT], ids=["f16", "f16_split"])
def test_encoder_prepared_weights(dev, oracle, prec):
    """Weights converted once (dl4s_cuda_encoder_prepare) give the same bytes as the per-call conversion of
    dl4s_cuda_encoder_forward, follow a refresh after the parameters changed, and the split form is the more
    exact one."""
    import ctypes
    from dl4s_b200._lib import c_vp, call
    from dl4s_b200.layers import TransformerEncoder
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000)
    enc = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=prec)
    x, mask = dev.tensor(c["x"]), dev.makeEncoderMasks(c["lengths"])
    prepared = enc(x, mask).numpy()                  # the layer class prepares on first use
    assert prec in enc._prepared
    plain = dev.CUDA.Memory.allocateBuffer(c["x"].shape)
    call("dl4s_cuda_encoder_forward", c_vp(x.ptr), 2, 128, 512, 8, 64, 64, 2048, 2, c_vp(enc.params.ptr), c_vp(mask.lengths.ptr), 0,
         c_vp(plain.ptr), prec)
    assert np.array_equal(plain.numpy(), prepared)
    # new parameter values in the same block: stale copies until refreshed
    c2 = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000, seed_w=77)
    enc2 = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c2["layers"], precision=prec)
    dev.CUDA.Memory.assign(enc2.params, enc.params, enc.params.count)
    enc.weightsChanged()
    assert np.array_equal(enc(x, mask).numpy(), enc2(x, mask).numpy())
    want = oracle.encoder(c["x"], c2["layers"], 8, c["lengths"])
    check(prec, enc(x, mask).numpy(), want, "after refresh")
    enc.releasePreparedWeights()
    assert dev.device_status() == 0


def test_split_weights_are_more_exact(dev, oracle):
    from dl4s_b200.layers import TransformerEncoder
    from util import rel_l2
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000)
    want = oracle.encoder(c["x"], c["layers"], 8, c["lengths"])
    errs = {}
    for prec in (PREC_F16, PREC_F16_SPLIT):
        enc = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=prec)
        errs[prec] = rel_l2(enc(dev.tensor(c["x"]), c["lengths"]).numpy(), want)
    assert errs[PREC_F16_SPLIT] < 0.8 * errs[PREC_F16], errs


def test_operation_group_trace(dev):
    """The reference's OperationGroup names (Tensor/Graph.swift:134-163) around the launches they cover: with tracing
    on, one encoder forward enters Encoder > EncoderLayer > MultiHeadAttention > ScaledDotProductAttention /
    LayerNorm and PointwiseFeedForward > Dense / LayerNorm, once per layer, in order."""
    import ctypes
    from dl4s_b200._lib import call
    from dl4s_b200.layers import TransformerEncoder
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000)
    enc = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=PREC_F16)
    x, mask = dev.tensor(c["x"]), dev.makeEncoderMasks(c["lengths"])
    enc(x, mask)
    call("dl4s_cuda_set_trace", 1)
    try:
        enc(x, mask)
        buf = ctypes.create_string_buffer(1 << 16)
        call("dl4s_cuda_trace_read", buf, len(buf))
    finally:
        call("dl4s_cuda_set_trace", 0)
    paths = buf.value.decode().split()
    layer = ["Encoder/EncoderLayer", "Encoder/EncoderLayer/MultiHeadAttention",
             "Encoder/EncoderLayer/MultiHeadAttention/ScaledDotProductAttention",
             "Encoder/EncoderLayer/MultiHeadAttention/LayerNorm", "Encoder/EncoderLayer/PointwiseFeedForward",
             "Encoder/EncoderLayer/PointwiseFeedForward/Dense", "Encoder/EncoderLayer/PointwiseFeedForward/Dense",
             "Encoder/EncoderLayer/PointwiseFeedForward/LayerNorm"]
    assert paths == ["Encoder"] + layer * 2, paths
    call("dl4s_cuda_trace_read", buf, len(buf))
    assert buf.value == b""


def test_encoder_blocks_compose_like_the_single_call(dev):
    """TransformerEncoderBlock by TransformerEncoderBlock equals the one-call encoder (same kernels, same order)."""
    from dl4s_b200.layers import TransformerEncoder, TransformerEncoderBlock
    c = workloads.encoder_config(B=2, S=64, D=128, H=2, F=256, layers=2, vocab=100)
    enc = TransformerEncoder(2, 2, 64, 64, 128, 256, layers=c["layers"], precision=PREC_FP32)
    x = dev.tensor(c["x"])
    mask = dev.makeEncoderMasks(c["lengths"])
    whole = enc(x, mask).numpy()
    cur = x
    for lw in c["layers"]:
        cur = TransformerEncoderBlock(128, 256, 2, 64, 64, lw, precision=PREC_FP32)(cur, mask)
    assert np.array_equal(cur.numpy(), whole)


def test_embed_positional(dev, oracle):
    from dl4s_b200.layers import EmbeddingWithPositions
    rng = np.random.default_rng(24)
    E = (rng.standard_normal((1000, 64)) * 0.02).astype(np.float32)
    ids = rng.integers(0, 1000, size=(3, 50)).astype(np.int32)
    ids[1, 7] = -1
    got = EmbeddingWithPositions(E, ignoreIndex=-1)(dev.tensor(ids, np.int32)).numpy()
    assert_fp32(got, oracle.embed(ids, E, -1), "embedding * sqrt(D) + positional encoding")


@pytest.mark.parametrize("prec,half", [(PREC_FP32, 0), (PREC_F16, 0), (PREC_F16, 1)], ids=["fp32", "f16", "f16-half-gather"])
def test_mha_halves_emulate_head_sharding_on_one_gpu(dev, oracle, prec, half):
    """The two halves of MultiHeadAttention around the all-gather, with both 'ranks' run one after the other on
    this GPU: column slices of Wq/Wk/Wv per rank, rank-major gather buffer, row rebuild by strided copy, second
    half per batch slice. Must equal the unsharded layer (oracle)."""
    import ctypes
    from dl4s_b200 import sharded
    from dl4s_b200._lib import c_vp, call
    from dl4s_b200.cuda import _i64arr
    rng = np.random.default_rng(30)
    G, B, S, D, H, dk = 2, 3, 140, 128, 2, 64
    x = rng.standard_normal((B, S, D), dtype=np.float32)
    # weights Xavier-uniform and inputs N(0,1): the distributions the stated tolerances are quoted on
    from dl4s_b200.layers import xavier_uniform
    W = {n: xavier_uniform(rng, D, H * dk) for n in ("qDense", "kDense", "vDense")}
    W["fc"] = xavier_uniform(rng, H * dk, D)
    lens = np.array([140, 77, 1], np.int32)
    one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
    want = oracle.mha(x, x, x, W["qDense"], W["kDense"], W["vDense"], W["fc"], one, zero, H, oracle.make_decoder_mask(lens, S))
    tx, tl = dev.tensor(x), dev.tensor(lens, np.int32)
    Hl, C = H // G, (H // G) * dk
    if half:
        ok = ctypes.c_int32(0)
        call("dl4s_cuda_mha_heads_half_supported", B, S, D, Hl, dk, dk, H * dk, ctypes.byref(ok))
        assert ok.value == 1
        C //= 2                 # the buffers hold half elements; the copies move them as pairs in one float
    gathered = dev.CUDA.Memory.allocateBuffer((G, B, S, C))
    for g in range(G):
        wq, wk, wv = (dev.tensor(sharded.slice_head_columns(W[n], H, G, g)) for n in ("qDense", "kDense", "vDense"))
        call("dl4s_cuda_mha_heads_forward", c_vp(tx.ptr), c_vp(tx.ptr), c_vp(tx.ptr), B, S, S, D, Hl, dk, dk, c_vp(wq.ptr),
             c_vp(wk.ptr), c_vp(wv.ptr), c_vp(tl.ptr), 1, c_vp(gathered.ptr + g * B * S * C * 4), prec, half)
    host_gathered = gathered.numpy().view(np.uint32)
    fc, sc, sh = dev.tensor(W["fc"]), dev.tensor(one), dev.tensor(zero)
    for g in range(G):
        b0, b1 = sharded.batch_range(B, G, g)
        Bl = b1 - b0
        rows = dev.CUDA.Memory.allocateBuffer((Bl, S, G * C))
        call("dl4s_cuda_copy_strided_f32", c_vp(gathered.ptr), _i64arr([S * C, C, B * S * C, 1]), b0 * S * C, c_vp(rows.ptr),
             _i64arr([S * G * C, G * C, C, 1]), 0, _i64arr([Bl, S, G, C]), 4)
        assert np.array_equal(rows.numpy().view(np.uint32), sharded.rows_from_gathered(host_gathered, b0, b1))
        out = dev.CUDA.Memory.allocateBuffer((Bl, S, D))
        call("dl4s_cuda_mha_output_forward", c_vp(rows.ptr), c_vp(tx.ptr + b0 * S * D * 4), Bl, S, D, H * dk, c_vp(fc.ptr),
             c_vp(sc.ptr), c_vp(sh.ptr), c_vp(out.ptr), prec, half, 1, 0)
        check(prec, out.numpy(), want[b0:b1], f"rank {g} batch slice")
        # the same, reading the gather buffer where it lies: G column groups, B*S*C elements apart
        out2 = dev.CUDA.Memory.allocateBuffer((Bl, S, D))
        c_el, esz = Hl * dk, (2 if half else 4)
        call("dl4s_cuda_mha_output_forward", c_vp(gathered.ptr + b0 * S * c_el * esz), c_vp(tx.ptr + b0 * S * D * 4), Bl, S, D,
             H * dk, c_vp(fc.ptr), c_vp(sc.ptr), c_vp(sh.ptr), c_vp(out2.ptr), prec, half, G, B * S * c_el)
        assert np.array_equal(out2.numpy(), out.numpy()), f"rank {g}: grouped read differs from rebuilt rows"


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_head_sharded_layer_world_size_one(dev, oracle, prec):
    """dl4s_cuda_mha_forward_sharded on a device that joined no communicator is the plain layer."""
    from dl4s_b200.sharded import HeadShardedMultiHeadAttention
    c = workloads.mha_config(B=3, S=128, D=256, H=4)
    layer = HeadShardedMultiHeadAttention(4, 256, 64, 64, c["weights"], precision=prec, chunks=2)
    assert (layer.rank, layer.world) == (0, 1) and layer.owned_batches(3) == [0, 1, 2]
    got = layer(dev.tensor(c["x"]), dev.StructuredMask(None, causal=True)).numpy()
    w = c["weights"]
    one, zero = np.ones(256, np.float32), np.zeros(256, np.float32)
    want = oracle.mha(c["x"], c["x"], c["x"], w["qDense"], w["kDense"], w["vDense"], w["fc"], one, zero, 4,
                      oracle.make_decoder_mask(np.full(3, 128, np.int32), 128))
    check(prec, got, want, "world size 1")
    assert dev.device_status() == 0


def test_half_head_outputs_are_refused_off_the_tensor_core_path(dev):
    """half_output / half_input exist only where the tensor-core kernels produce and consume them."""
    import ctypes
    from dl4s_b200._lib import DL4SCudaError, c_vp, call
    B, S, D, H, dk = 1, 16, 24, 1, 8          # D and dk no tensor-core shapes
    ok = ctypes.c_int32(1)
    call("dl4s_cuda_mha_heads_half_supported", B, S, D, H, dk, dk, H * dk, ctypes.byref(ok))
    assert ok.value == 0
    x = dev.tensor(np.zeros((B, S, D), np.float32))
    w = dev.tensor(np.zeros((D, H * dk), np.float32))
    out = dev.CUDA.Memory.allocateBuffer((B, S, H * dk))
    with pytest.raises(DL4SCudaError):
        call("dl4s_cuda_mha_heads_forward", c_vp(x.ptr), c_vp(x.ptr), c_vp(x.ptr), B, S, S, D, H, dk, dk, c_vp(w.ptr),
             c_vp(w.ptr), c_vp(w.ptr), c_vp(0), 0, c_vp(out.ptr), PREC_F16, 1)


def test_graph_replay_equals_eager(dev, oracle):
    """A forward recorded into a CUDA graph replays to the same bytes as the eager calls, follows new input values
    in the same buffers, counts its kernels, and refuses what cannot be recorded."""
    from dl4s_b200 import DL4SCudaError
    from dl4s_b200.layers import TransformerEncoder
    c = workloads.encoder_config(B=2, S=128, D=512, H=8, F=2048, layers=2, vocab=1000)
    enc = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=PREC_F16)
    x, mask = dev.tensor(c["x"]), dev.makeEncoderMasks(c["lengths"])
    out = dev.CUDA.Memory.allocateBuffer(c["x"].shape)
    enc(x, mask, out=out)
    eager = out.numpy()
    with dev.Graph() as g:
        enc(x, mask, out=out)
    dev.CUDA.Memory.assign(dev.tensor(np.zeros_like(c["x"])), out, out.count)
    n0 = dev.launch_count()
    g.launch()
    per_replay = dev.launch_count() - n0
    assert per_replay > 0
    assert np.array_equal(out.numpy(), eager)
    # new values in the same input buffer
    x2 = c["x"][::-1].copy()
    dev.CUDA.Memory.assign(dev.tensor(x2), x, x.count)
    g.launch()
    enc2 = TransformerEncoder(2, 8, 64, 64, 512, 2048, layers=c["layers"], precision=PREC_F16)
    assert np.array_equal(out.numpy(), enc2(dev.tensor(x2), mask).numpy())
    g.destroy()
    # allocation inside a capture is refused, and the capture can still be closed
    with pytest.raises(DL4SCudaError):
        with dev.Graph() as g2:
            dev.CUDA.Memory.allocateBuffer((4,))
    g2.destroy()
    assert dev.device_status() == 0


def test_graph_survives_a_larger_eager_call(dev, oracle):
    """A recorded graph names the library's scratch arena by address. A later eager call with a larger shape makes
    the arena grow; the old block must stay allocated until the graph is destroyed, so the replay still computes
    the recorded forward."""
    from dl4s_b200.layers import MultiHeadAttention
    c = workloads.mha_config(B=2, S=128, D=512, H=8)
    small = MultiHeadAttention(8, 512, 64, 64, weights=c["weights"], precision=PREC_F16)
    x = dev.tensor(c["x"])
    out = dev.CUDA.Memory.allocateBuffer(c["x"].shape)
    small(x, x, x, out=out)
    eager = out.numpy()
    with dev.Graph() as g:
        small(x, x, x, out=out)
    # a much larger layer: the arena is replaced
    big_c = workloads.mha_config(B=16, S=512, D=1024, H=8, seed_x=5, seed_w=6)
    big = MultiHeadAttention(8, 1024, 128, 128, weights=big_c["weights"], precision=PREC_F16)
    xb = dev.tensor(big_c["x"])
    big(xb, xb, xb)
    dev.CUDA.Memory.assign(dev.tensor(np.zeros_like(c["x"])), out, out.count)
    g.launch()
    assert np.array_equal(out.numpy(), eager)
    big(xb, xb, xb)            # the new arena is in use between replays
    g.launch()
    assert np.array_equal(out.numpy(), eager)
    g.destroy()
    assert dev.device_status() == 0


@pytest.mark.parametrize("D,H,dk", [(128, 2, 64), (96, 3, 32), (512, 4, 128)], ids=["d64", "d32-fallback", "d128"])
def test_decode_step_with_kv_cache_equals_full_recompute(dev, oracle, D, H, dk):
    """Incremental decoding: after the prompt's keys/values are cached, each step must give the LAST row of
    MultiHeadAttention over the whole prefix with the causal mask — what DL4S recomputes per generated token."""
    from dl4s_b200.layers import MultiHeadAttention
    rng = np.random.default_rng(40 + D)
    B, S, L, steps = 3, 37, 64, 3
    lens = np.array([37, 5, 20], np.int32)
    seq = rng.standard_normal((B, L, D), dtype=np.float32)          # row t of sequence b = its t-th input
    mha = MultiHeadAttention(H, D, dk, dk, rng=rng, precision=PREC_FP32)
    w = mha.host_weights
    one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
    cache = mha.makeCache(B, L)
    prompt = seq[:, :S].copy()
    for b in range(B):
        prompt[b, lens[b]:] = 7.0                                     # padding rows: never read by later steps
    mha.prefillCache(dev.tensor(prompt), lens, cache)
    cur = lens.copy()
    for _ in range(steps):
        x_t = np.stack([seq[b, cur[b]] for b in range(B)])
        got = mha.decodeStep(dev.tensor(x_t), cache).numpy()
        # The reference's MultiHeadAttention normalises the whole [n, D] block of a prefix at once (LayerNorm over all
        # axes but the first); a step owns one token, so its LayerNorm runs over that token's [1, D] block. The
        # expected row is therefore built from the oracle's pieces: projections, causal attention over the prefix,
        # last row through Wo + residual, LayerNorm of that row.
        for b in range(B):
            n = int(cur[b]) + 1
            xs = seq[b:b + 1, :n]
            q = oracle.gemm(xs[0], w["qDense"]).reshape(1, n, H, dk).transpose(0, 2, 1, 3)
            k = oracle.gemm(xs[0], w["kDense"]).reshape(1, n, H, dk).transpose(0, 2, 1, 3)
            v = oracle.gemm(xs[0], w["vDense"]).reshape(1, n, H, dk).transpose(0, 2, 1, 3)
            a = oracle.sdpa(q, k, v, oracle.make_decoder_mask(np.array([n], np.int32), n)).transpose(0, 2, 1, 3).reshape(n, H * dk)
            pre = oracle.gemm(a[-1:], w["fc"]) + xs[0, -1:]
            want_row = oracle.layernorm(pre.reshape(1, 1, D), one, zero)[0, 0]
            assert_fp32(got[b], want_row, f"step at position {n - 1} of sequence {b}")
        cur += 1
    assert np.array_equal(cache.lengths_host, lens + steps)
    assert dev.device_status() == 0


def test_decode_step_reports_a_full_cache(dev):
    from dl4s_b200.layers import MultiHeadAttention
    rng = np.random.default_rng(44)
    mha = MultiHeadAttention(2, 128, 64, 64, rng=rng, precision=PREC_FP32)
    cache = mha.makeCache(1, 4)
    cache.setLengths(np.array([4], np.int32))
    from dl4s_b200 import DL4SCudaError
    mha.decodeStep(dev.tensor(rng.standard_normal((1, 128), dtype=np.float32)), cache)
    with pytest.raises(DL4SCudaError) as e:
        dev.device_status()
    assert e.value.status == -1 and "cache" in str(e.value)
    assert dev.device_status() == 0          # reading cleared it


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_output_head(dev, oracle, prec):
    """logSoftmax(x . E^T + bias) over the vocabulary against the CPU engine's order of operations. The embedding
    is N(0, 0.02) as in the benchmark configuration and the states are N(0,1) (what a LayerNorm leaves), so the
    log-probabilities are O(10) and the stated absolute tolerances apply; a last case with logits of O(30) is held
    to the same bounds relative to the largest |value| (half operands carry a relative error)."""
    from dl4s_b200.layers import EmbeddingWithPositions, OutputHead
    from util import FP32_TOL, TC_MAX_ABS, TC_REL_L2, assert_close
    rng = np.random.default_rng(50)
    for B, S, D, V, escale in ((2, 5, 24, 37, 0.02), (2, 100, 128, 1024, 0.02), (1, 130, 64, 2048 + 64, 0.02),
                               (2, 100, 128, 1024, 0.3)):
        E = (rng.standard_normal((V, D)) * escale).astype(np.float32)
        bias = (rng.standard_normal(V) * 0.1).astype(np.float32)
        x = rng.standard_normal((B, S, D), dtype=np.float32)
        head = OutputHead(EmbeddingWithPositions(E), bias, precision=prec)
        got = head(dev.tensor(x)).numpy()
        want = oracle.output_head(x, E, bias)
        if escale == 0.02:
            check(prec, got, want, f"output head [{B},{S},{D}] x {V}")
        else:
            big = float(np.abs(want).max())
            assert big > 10
            lim = (FP32_TOL * big, FP32_TOL) if prec == PREC_FP32 else (TC_MAX_ABS * big, TC_REL_L2)
            assert_close(got, want, lim[0], lim[1], f"output head with logits up to {big:.0f} (bound relative to that)")
        assert np.abs(np.exp(got.astype(np.float64)).sum(-1) - 1).max() < 1e-4
        # greedy decoding picks the same token
        assert np.array_equal(got.argmax(-1), want.argmax(-1)) or prec == PREC_F16


def test_log_softmax_rows_in_place_and_ragged(dev, oracle):
    from dl4s_b200._lib import c_vp, call
    rng = np.random.default_rng(51)
    for rows, n in ((3, 1), (5, 7), (4, 32000), (2, 1001)):
        x = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
        t = dev.tensor(x)
        call("dl4s_cuda_log_softmax_rows", c_vp(t.ptr), rows, n, c_vp(t.ptr))
        # values of O(20); a sum over 32000 fp32 terms carries ~1e-5 RELATIVE error in either order of summation (the
        # CPU engine adds them one after the other), so the bound is relative to the largest |value|
        assert_fp32_rel(t.numpy(), oracle.log_softmax_rows(x), f"log-softmax {rows} x {n}")


def test_layernorm_backward(dev):
    """dx, dscale, dshift of DL4S's LayerNorm against the float64 closed form (itself pinned by finite differences
    in the CPU tier), for both flavours: statistics per batch element over [rows, D] and per row."""
    from dl4s_b200._lib import c_vp, call
    from oracle import oracle_np as ON
    from util import assert_fp32_rel
    rng = np.random.default_rng(91)
    for shape in ((3, 40, 64), (5, 1, 512), (2, 128, 512)):
        outer, rows, D = shape
        x = rng.standard_normal(shape, dtype=np.float32) * 2 + 0.5
        dy = rng.standard_normal(shape, dtype=np.float32)
        g = (1 + 0.2 * rng.standard_normal(D)).astype(np.float32)
        tx, tdy, tg = dev.tensor(x), dev.tensor(dy), dev.tensor(g)
        dx, dg, db = (dev.CUDA.Memory.allocateBuffer(s) for s in (shape, (D,), (D,)))
        call("dl4s_cuda_layernorm_backward", c_vp(tx.ptr), c_vp(tdy.ptr), outer, rows, D, c_vp(tg.ptr), c_vp(dx.ptr), c_vp(dg.ptr),
             c_vp(db.ptr))
        wx, wg, wb = ON.layernorm_backward(x, dy, g)
        assert_fp32(dx.numpy(), wx, f"dx {shape}")
        assert_fp32_rel(dg.numpy(), wg, f"dscale {shape}")      # sums over up to 256 rows: relative to their size
        assert_fp32_rel(db.numpy(), wb, f"dshift {shape}")
    assert dev.device_status() == 0
