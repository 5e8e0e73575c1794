"""GPU tier: the frozen vectors of tests/golden/hotpath_next.npz — attention backward, embedding + positional encoding,
output head, LayerNorm backward — through the C ABI. fp32 paths are held to 1e-5; the tensor-core paths do not take
shapes this small (they fall back to the fp32 kernels), which is part of what is checked."""
import numpy as np
import pytest

from dl4s_b200 import PREC_F16, PREC_FP32
from util import assert_fp32, golden_next

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("prec", [PREC_FP32, PREC_F16], ids=["fp32", "f16"])
def test_attention_backward_golden(dev, prec):
    from dl4s_b200.layers import scaledDotProductAttentionBackward
    g = golden_next()
    q, k, v, d = (dev.tensor(g[n]) for n in ("bwd_q", "bwd_k", "bwd_v", "bwd_dout"))
    for name, mask in (("pad", dev.makeEncoderMasks(g["bwd_lens"])), ("dec", dev.makeDecoderMasks(g["bwd_lens"]))):
        dq, dk, dv = scaledDotProductAttentionBackward(q, k, v, d, mask, None, prec)
        assert_fp32(dq.numpy(), g[f"bwd_{name}_dq"], f"dq ({name})")
        assert_fp32(dk.numpy(), g[f"bwd_{name}_dk"], f"dk ({name})")
        assert_fp32(dv.numpy(), g[f"bwd_{name}_dv"], f"dv ({name})")
    assert dev.device_status() == 0


def test_embedding_and_output_head_golden(dev):
    from dl4s_b200.layers import EmbeddingWithPositions, OutputHead
    g = golden_next()
    emb = EmbeddingWithPositions(g["emb_E"])
    x = emb(dev.tensor(g["emb_ids"], np.int32))
    assert_fp32(x.numpy(), g["emb_out"], "embedding + positional encoding")
    head = OutputHead(emb, g["head_bias"], precision=PREC_FP32)
    assert_fp32(head(x).numpy(), g["head_out"], "output head")
    assert dev.device_status() == 0


def test_layernorm_backward_golden(dev):
    from dl4s_b200._lib import c_vp, call
    g = golden_next()
    x, dy, sc = g["lnb_x"], g["lnb_dy"], g["lnb_scale"]
    outer, rows, D = x.shape
    tx, tdy, tg = dev.tensor(x), dev.tensor(dy), dev.tensor(sc)
    dx, dg, db = (dev.CUDA.Memory.allocateBuffer(s) for s in (x.shape, (D,), (D,)))
    call("dl4s_cuda_layernorm_backward", c_vp(tx.ptr), c_vp(tdy.ptr), outer, rows, D, c_vp(tg.ptr), c_vp(dx.ptr), c_vp(dg.ptr),
         c_vp(db.ptr))
    assert_fp32(dx.numpy(), g["lnb_dx"], "dx")
    assert_fp32(dg.numpy(), g["lnb_dscale"], "dscale")
    assert_fp32(db.numpy(), g["lnb_dshift"], "dshift")
    assert dev.device_status() == 0
