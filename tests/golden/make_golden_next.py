"""Generates tests/golden/hotpath_next.npz: frozen CPU-oracle outputs for the rows around the attention path that
hotpath_small.npz does not cover — the attention backward (dq, dk, dv), the embedding + positional encoding, the
output head (tied-embedding logits + log-softmax) — and the float64 LayerNorm backward.

As with hotpath_small.npz, the reference (Swift) cannot run here and ships no vectors for these, so they are the
project's own: oracle outputs for fixed seeds on tiny shapes, committed so that a change in the oracle or in a
kernel shows up as a diff against frozen numbers.

Run from the repository root:  python tests/golden/make_golden_next.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from oracle import oracle_np as ON  # noqa: E402


def main():
    rng = np.random.default_rng(20251)
    out = {}
    # attention backward: padding mask, and causal + padding
    B, H, S, d = 2, 2, 6, 8
    q, k, v, g = (rng.standard_normal((B, H, S, d), dtype=np.float32) for _ in range(4))
    lens = np.array([6, 4], np.int32)
    out.update(bwd_q=q, bwd_k=k, bwd_v=v, bwd_dout=g, bwd_lens=lens)
    for name, mask in (("pad", O.make_encoder_mask(lens, S)), ("dec", O.make_decoder_mask(lens, S))):
        dq, dk, dv = O.sdpa_backward(q, k, v, g, mask)
        out.update({f"bwd_{name}_dq": dq, f"bwd_{name}_dk": dk, f"bwd_{name}_dv": dv})
    # embedding (with an ignored index) + positional encoding, and the output head over the same table
    V, D = 11, 16
    E = (rng.standard_normal((V, D)) * 0.5).astype(np.float32)
    ids = np.array([[1, 4, -1, 10, 0], [7, 7, 2, -1, -1]], np.int32)
    bias = (rng.standard_normal(V) * 0.1).astype(np.float32)
    x = O.embed(ids, E)
    out.update(emb_E=E, emb_ids=ids, emb_out=x, head_bias=bias, head_out=O.output_head(x, E, bias))
    # LayerNorm backward (float64 closed form, pinned by finite differences in tests/test_oracle.py)
    lx = rng.standard_normal((3, 5, 8)).astype(np.float32)
    ldy = rng.standard_normal((3, 5, 8)).astype(np.float32)
    lscale = (1.0 + 0.2 * rng.standard_normal(8)).astype(np.float32)
    dx, dscale, dshift = ON.layernorm_backward(lx, ldy, lscale)
    out.update(lnb_x=lx, lnb_dy=ldy, lnb_scale=lscale, lnb_dx=dx, lnb_dscale=dscale, lnb_dshift=dshift)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "hotpath_next.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
