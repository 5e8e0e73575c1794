"""CPU tier: pins the oracle (oracle/dl4s_ref.c) before anything is compared with it.

1. The reference's own known-answer matmul tests (Tests/DL4STests/VecTests.swift:86-156).
2. The reference's tolerance tests on exp/log and sigmoid (VecTests.swift:158-168, 242-258) restated on the
   oracle's libm calls.
3. Analytic identities of attention, masks and DL4S's LayerNorm.
4. Agreement with an independent float64 formulation.
5. The frozen golden vectors in tests/golden/.
"""
import numpy as np
import pytest

from oracle import oracle_np as ON
from util import golden, golden_next, max_abs, rel_l2, unpack_layers


def test_gemm_known_answers_from_reference_tests(oracle):
    a = np.array([[1, 2, 3]], np.float32)
    b = np.array([[4], [5], [6]], np.float32)
    assert oracle.gemm(a, b)[0, 0] == 32                      # testMMul1x1
    c = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    assert oracle.gemm(c, a.T).ravel().tolist() == [14, 32]    # testMMul2x1
    d = np.array([[1, 2]], np.float32)
    assert oracle.gemm(d, c).ravel().tolist() == [9, 12, 15]   # testMMul1x2
    assert oracle.gemm(c, c, trans_a=True).tolist() == [[17, 22, 27], [22, 29, 36], [27, 36, 45]]  # testMMul2x2
    assert oracle.gemm(c, c, trans_b=True).tolist() == [[14, 32], [32, 77]]                        # testMMul2x2_2


def test_gemm_all_transposes_and_scaling(oracle):
    rng = np.random.default_rng(0)
    A = rng.standard_normal((5, 7), dtype=np.float32)
    B = rng.standard_normal((7, 3), dtype=np.float32)
    want = A.astype(np.float64) @ B.astype(np.float64)
    for ta in (False, True):
        for tb in (False, True):
            got = oracle.gemm(A.T.copy() if ta else A, B.T.copy() if tb else B, trans_a=ta, trans_b=tb, alpha=0.5)
            assert max_abs(got, 0.5 * want) < 1e-5


def test_exp_log_sigmoid_tolerances(oracle):
    rng = np.random.default_rng(1)
    x = rng.uniform(-5, 5, (10, 10)).astype(np.float32)
    # softmax of one row of [x, -inf...] is not available; use the identities the reference tests use
    assert max_abs(np.log(np.exp(x)), x) < 1e-4
    t = rng.standard_normal(10).astype(np.float32)
    sig = 0.5 * np.tanh(t * 0.5) + 0.5   # Unary.swift:184-186
    assert max_abs(sig, 1 / (1 + np.exp(-t))) < 1e-4


def test_softmax_rows_sum_to_one(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 129), dtype=np.float32) * 4
    p = oracle.softmax_rows(x)
    assert np.abs(p.sum(axis=1) - 1).max() < 1e-5
    assert (p >= 0).all()


def test_masks_match_definitions(oracle):
    lens = np.array([3, 5, 0], np.int32)
    m = oracle.make_encoder_mask(lens, 5)
    assert m.shape == (3, 1, 1, 5)
    assert m[0, 0, 0].tolist() == [0, 0, 0, 1, 1] and m[1].sum() == 0 and m[2].sum() == 5
    d = oracle.make_decoder_mask(np.array([4, 2], np.int32), 4)
    assert d.shape == (2, 1, 4, 4)
    want0 = (np.arange(4)[None, :] > np.arange(4)[:, None]).astype(np.float32)
    assert (d[0, 0] == want0).all()
    want1 = np.maximum(want0, (np.arange(4) >= 2).astype(np.float32)[None, :])
    assert (d[1, 0] == want1).all()


def test_attention_identities(oracle):
    rng = np.random.default_rng(3)
    B, H, Sq, Sk, d = 2, 3, 9, 11, 8
    k = rng.standard_normal((B, H, Sk, d), dtype=np.float32)
    v = rng.standard_normal((B, H, Sk, d), dtype=np.float32)
    q0 = np.zeros((B, H, Sq, d), np.float32)
    # q = 0: uniform weights -> mean of the value rows
    out = oracle.sdpa(q0, k, v)
    assert max_abs(out, np.broadcast_to(v.mean(axis=2, keepdims=True), out.shape)) < 1e-6
    # with a padding mask: mean over the unmasked rows only
    lens = np.array([4, 11], np.int32)
    out = oracle.sdpa(q0, k, v, oracle.make_encoder_mask(lens, Sk))
    assert max_abs(out[0], np.broadcast_to(v[0, :, :4].mean(axis=1, keepdims=True), out[0].shape)) < 1e-6
    # fully masked sequence: the finite -1e9 makes the weights uniform over ALL keys
    out = oracle.sdpa(rng.standard_normal((B, H, Sq, d), dtype=np.float32), k, v,
                      oracle.make_encoder_mask(np.array([0, 11], np.int32), Sk))
    assert max_abs(out[0], np.broadcast_to(v[0].mean(axis=1, keepdims=True), out[0].shape)) < 1e-6
    # causal: row 0 attends to key 0 only
    q = rng.standard_normal((B, H, Sk, d), dtype=np.float32)
    out = oracle.sdpa(q, k, v, oracle.make_decoder_mask(np.array([Sk, Sk], np.int32), Sk))
    assert max_abs(out[:, :, 0], v[:, :, 0]) < 1e-6
    # masked logits are exactly -1e9 in fp32
    assert np.float32(3.7) - np.float32(1e9) == np.float32(-1e9)


def test_layernorm_reduces_over_all_axes_but_first(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 5, 16), dtype=np.float32) * 3 + 2
    g = np.ones(16, np.float32)
    s = np.zeros(16, np.float32)
    y = oracle.layernorm(x, g, s)
    # statistics per batch element over the whole [5,16] block
    assert np.abs(y.reshape(3, -1).mean(axis=1)).max() < 1e-5
    assert np.abs(y.reshape(3, -1).std(axis=1) - 1).max() < 1e-4
    # rows are NOT individually normalised
    assert np.abs(y.mean(axis=2)).max() > 1e-2
    # 2-D input: per row
    y2 = oracle.layernorm(x.reshape(15, 16), g, s)
    assert np.abs(y2.mean(axis=1)).max() < 1e-5
    assert max_abs(y, ON.layernorm(x, g, s)) < 1e-5


def test_against_float64_formulation(oracle):
    rng = np.random.default_rng(5)
    g = golden()
    D, H, F = 16, 4, 32
    layers = unpack_layers(g["enc_params"], D, H, 4, 4, F, 2)
    x = g["mha_x"]
    lens = g["causal_lens"]
    a = oracle.encoder(x, layers, H, lens)
    b = ON.encoder(x, layers, H, lens)
    assert rel_l2(a, b) < 1e-5 and max_abs(a, b) < 1e-5
    q = rng.standard_normal((2, 2, 33, 16), dtype=np.float32)
    k = rng.standard_normal((2, 2, 47, 16), dtype=np.float32)
    v = rng.standard_normal((2, 2, 47, 8), dtype=np.float32)
    assert max_abs(oracle.sdpa(q, k, v), ON.sdpa(q, k, v)) < 1e-5
    assert max_abs(oracle.positional_encoding(64, 32), ON.positional_encoding(64, 32)) < 2e-5


def test_golden_vectors(oracle):
    g = golden()
    q, k, v = g["sdpa_q"], g["sdpa_k"], g["sdpa_v"]
    assert np.array_equal(oracle.sdpa(q, k, v), g["sdpa_nomask"])
    assert np.array_equal(oracle.sdpa(q, k, v, oracle.make_encoder_mask(g["sdpa_lens"], 7)), g["sdpa_padmask"])
    assert np.array_equal(oracle.sdpa(q, k, v, oracle.make_encoder_mask(g["sdpa_lens0"], 7)), g["sdpa_fullmask"])
    assert np.array_equal(oracle.sdpa(g["causal_q"], g["causal_k"], g["causal_v"],
                                      oracle.make_decoder_mask(g["causal_lens"], 6)), g["causal_out"])
    assert np.array_equal(oracle.layernorm(g["ln_x"], g["ln_scale"], g["ln_shift"]), g["ln_out3d"])
    assert np.array_equal(oracle.layernorm(g["ln_x"].reshape(6, 8), g["ln_scale"], g["ln_shift"]), g["ln_out2d"])
    D = 16
    one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
    assert np.array_equal(oracle.mha(g["mha_x"], g["mha_x"], g["mha_x"], g["mha_Wq"], g["mha_Wk"], g["mha_Wv"], g["mha_Wo"],
                                     one, zero, 4, oracle.make_encoder_mask(g["causal_lens"], 6)), g["mha_out"])
    assert np.array_equal(oracle.ffn(g["mha_x"], g["ffn_W1"], g["ffn_b1"], g["ffn_W2"], g["ffn_b2"], one, zero), g["ffn_out"])
    assert np.array_equal(oracle.ffn(g["mha_x"], g["ffn_W1"], g["ffn_b1"], g["ffn_W2"], g["ffn_b2"], one, zero, act=1),
                          g["ffn_out_relu"])
    layers = unpack_layers(g["enc_params"], D, 4, 4, 4, 32, 2)
    assert np.array_equal(oracle.encoder(g["mha_x"], layers, 4, g["causal_lens"]), g["enc_out"])
    assert np.array_equal(oracle.positional_encoding(10, 8), g["pe_10x8"])


def test_threads_do_not_change_values(oracle):
    rng = np.random.default_rng(6)
    q = rng.standard_normal((2, 4, 40, 16), dtype=np.float32)
    k = rng.standard_normal((2, 4, 40, 16), dtype=np.float32)
    v = rng.standard_normal((2, 4, 40, 16), dtype=np.float32)
    oracle.set_threads(1)
    a = oracle.sdpa(q, k, v)
    oracle.set_threads(4)
    b = oracle.sdpa(q, k, v)
    assert np.array_equal(a, b)


def test_embed_matches_formula(oracle):
    rng = np.random.default_rng(7)
    E = rng.standard_normal((11, 8), dtype=np.float32)
    ids = np.array([[1, 5, -1], [10, 0, 3]], np.int32)
    x = oracle.embed(ids, E, ignore_index=-1)
    pe = oracle.positional_encoding(3, 8)
    assert max_abs(x[0, 2], pe[2]) == 0
    assert max_abs(x[1, 0], E[10] * np.float32(np.sqrt(np.float32(8))) + pe[0]) < 1e-6


def test_output_head_and_log_softmax(oracle):
    """logSoftmax(x . E^T + bias): the C restatement against the float64 formulation, and the identities the
    reference's definition implies (rows exponentiate to one; adding a constant to a row changes nothing)."""
    from oracle import oracle_np as ON
    rng = np.random.default_rng(60)
    x = rng.standard_normal((3, 7, 24), dtype=np.float32)
    E = (rng.standard_normal((50, 24)) * 0.4).astype(np.float32)
    b = (rng.standard_normal(50) * 0.2).astype(np.float32)
    got = oracle.output_head(x, E, b)
    assert got.shape == (3, 7, 50)
    assert np.abs(got - ON.output_head(x, E, b)).max() < 1e-5
    assert np.abs(np.exp(got.astype(np.float64)).sum(-1) - 1).max() < 1e-5
    z = (rng.standard_normal((4, 33)) * 5).astype(np.float32)
    assert np.abs(oracle.log_softmax_rows(z + 3.0) - oracle.log_softmax_rows(z)).max() < 1e-5
    one = oracle.log_softmax_rows(np.array([[2.5]], np.float32))
    assert one.item() == 0.0


def test_sdpa_backward_matches_finite_differences_and_float64(oracle):
    """The backward restatement: against central differences of the float64 forward (pins the formulas) and
    against the float64 closed form (pins the fp32 evaluation), with padding + causal masks."""
    from oracle import oracle_np as ON
    rng = np.random.default_rng(70)
    B, H, S, d = 2, 2, 9, 5
    q, k, v, g = (rng.standard_normal((B, H, S, d)) for _ in range(4))
    lens = np.array([9, 4], np.int32)
    mask = oracle.make_decoder_mask(lens, S)
    dq, dk, dv = oracle.sdpa_backward(q, k, v, g, mask)
    rq, rk, rv = ON.sdpa_backward(q, k, v, g, mask)
    for got, want in ((dq, rq), (dk, rk), (dv, rv)):
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())

    def loss(qq, kk, vv):
        return float((ON.sdpa(qq, kk, vv, mask) * g).sum())

    eps = 1e-6
    for arr, grad in ((q, rq), (k, rk), (v, rv)):
        for idx in ((0, 0, 0, 0), (0, 1, 3, 2), (1, 0, 2, 4), (1, 1, 8, 1)):
            hi, lo = arr.copy(), arr.copy()
            hi[idx] += eps
            lo[idx] -= eps
            args_hi = [hi if a is arr else a for a in (q, k, v)]
            args_lo = [lo if a is arr else a for a in (q, k, v)]
            fd = (loss(*args_hi) - loss(*args_lo)) / (2 * eps)
            assert abs(fd - grad[idx]) <= 1e-6 * max(1.0, abs(fd)), (idx, fd, grad[idx])
    # keys a sequence cannot see get no gradient
    assert np.abs(dk[1, :, 4:]).max() == 0.0 and np.abs(dv[1, :, 4:]).max() == 0.0


def test_layernorm_backward_matches_finite_differences():
    """The closed form the device kernel implements, against central differences of the float64 forward."""
    from oracle import oracle_np as ON
    rng = np.random.default_rng(33)
    for shape in ((3, 5, 8), (4, 6)):
        x = rng.standard_normal(shape)
        dy = rng.standard_normal(shape)
        g = 1 + 0.3 * rng.standard_normal(shape[-1])
        b = 0.3 * rng.standard_normal(shape[-1])
        dx, dg, db = ON.layernorm_backward(x, dy, g)
        loss = lambda xx, gg, bb: float((ON.layernorm(xx, gg, bb) * dy).sum())
        eps = 1e-6
        for idx in [tuple(rng.integers(0, s) for s in shape) for _ in range(6)]:
            xp, xm = x.copy(), x.copy()
            xp[idx] += eps
            xm[idx] -= eps
            assert abs((loss(xp, g, b) - loss(xm, g, b)) / (2 * eps) - dx[idx]) < 1e-6
        for c in range(shape[-1]):
            gp, gm = g.copy(), g.copy()
            gp[c] += eps
            gm[c] -= eps
            assert abs((loss(x, gp, b) - loss(x, gm, b)) / (2 * eps) - dg[c]) < 1e-6
            bp, bm = b.copy(), b.copy()
            bp[c] += eps
            bm[c] -= eps
            assert abs((loss(x, g, bp) - loss(x, g, bm)) / (2 * eps) - db[c]) < 1e-6


def test_golden_vectors_of_the_next_rows(oracle):
    """The oracle reproduces the frozen backward, embedding and output-head vectors bit for bit (C restatement) and the
    float64 LayerNorm backward to rounding."""
    from oracle import oracle_np as ON
    g = golden_next()
    q, k, v, d = g["bwd_q"], g["bwd_k"], g["bwd_v"], g["bwd_dout"]
    for name, mask in (("pad", oracle.make_encoder_mask(g["bwd_lens"], 6)), ("dec", oracle.make_decoder_mask(g["bwd_lens"], 6))):
        dq, dk, dv = oracle.sdpa_backward(q, k, v, d, mask)
        assert np.array_equal(dq, g[f"bwd_{name}_dq"]) and np.array_equal(dk, g[f"bwd_{name}_dk"])
        assert np.array_equal(dv, g[f"bwd_{name}_dv"])
        # and the float64 closed form agrees with the frozen fp32 values
        wq, wk, wv = ON.sdpa_backward(q, k, v, d, mask)
        assert max_abs(dq, wq) < 1e-5 and max_abs(dk, wk) < 1e-5 and max_abs(dv, wv) < 1e-5
    x = oracle.embed(g["emb_ids"], g["emb_E"])
    assert np.array_equal(x, g["emb_out"])
    assert np.array_equal(x[0, 2], oracle.positional_encoding(5, 16)[2])          # an ignored index embeds as zeros + position
    assert np.array_equal(oracle.output_head(x, g["emb_E"], g["head_bias"]), g["head_out"])
    assert np.allclose(np.exp(g["head_out"].astype(np.float64)).sum(axis=-1), 1.0, atol=1e-5)
    dx, ds, db = ON.layernorm_backward(g["lnb_x"], g["lnb_dy"], g["lnb_scale"])
    assert max_abs(dx, g["lnb_dx"]) < 1e-12 and max_abs(ds, g["lnb_dscale"]) < 1e-12 and max_abs(db, g["lnb_dshift"]) < 1e-12
