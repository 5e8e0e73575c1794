import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_small.npz")

# Tolerances of the two arithmetic modes against the DL4S CPU engine (the oracle):
# fp32 FFMA check kernels 1e-5; tensor-core path (half operands, fp32 accumulate)
# max-abs 2e-3 and relative L2 1e-3.
FP32_TOL = 1e-5
TC_MAX_ABS = 2e-3
TC_REL_L2 = 1e-3


def golden():
    return np.load(GOLDEN)


def golden_next():
    """The second fixture file: backward, embedding and output-head rows (tests/golden/make_golden_next.py)."""
    return np.load(os.path.join(os.path.dirname(GOLDEN), "hotpath_next.npz"))


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def max_abs(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max())


def assert_close(got, want, max_abs_tol, rel_l2_tol, what=""):
    """Both bounds as stated, unscaled: max |got - want| <= max_abs_tol and ||got - want|| / ||want|| <= rel_l2_tol."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    ma, rl = max_abs(got, want), rel_l2(got, want)
    assert ma <= max_abs_tol and rl <= rel_l2_tol, f"{what}: max-abs {ma:.3e} (limit {max_abs_tol:.1e}), rel-L2 {rl:.3e} (limit {rel_l2_tol:.1e})"


def assert_fp32(got, want, what=""):
    """Outputs of the attention path from the fp32 FFMA kernels: 1e-5 on both measures."""
    assert_close(got, want, FP32_TOL, FP32_TOL, what)


def assert_tc(got, want, what=""):
    """Outputs of the attention path from the tensor-core kernels: max-abs 2e-3 and relative L2 1e-3."""
    assert_close(got, want, TC_MAX_ABS, TC_REL_L2, what)


# Stacks of more than two sublayers on DL4S_PREC_F16 (weights rounded to half once): the relative L2 error stays inside
# 1e-3 but the largest single deviation grows past 2e-3 (measured 3.1e-3 on the 6-layer encoder at batch 32 x 512,
# 2.8e-3 on a 2-layer decoder = 6 sublayers). This is that measured figure with a margin, NOT a tolerance of the
# path: DL4S_PREC_F16_SPLIT is the mode that meets the stated 2e-3 at depth, and the tests hold it to that.
F16_DEEP_MAX_ABS_DOCUMENTED = 3.5e-3


def assert_tc_deep_f16(got, want, what=""):
    assert_close(got, want, F16_DEEP_MAX_ABS_DOCUMENTED, TC_REL_L2, what)


def assert_fp32_rel(got, want, what=""):
    """For EngineType primitives whose results are not O(1) (a product over K = 2048 terms, a sum over 10^5
    elements, exp of 10): fp32 cannot hold 1e-5 absolute there (one ulp of 100 is 8e-6), so the bound is relative to
    the largest expected magnitude: max |got - want| <= 1e-5 * max(1, max |want|), and relative L2 <= 1e-5."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    ma, rl = max_abs(got, want), rel_l2(got, want)
    lim = FP32_TOL * max(1.0, float(np.abs(want).max()) if want.size else 1.0)
    assert ma <= lim and rl <= FP32_TOL, f"{what}: max-abs {ma:.3e} (limit {lim:.1e}), rel-L2 {rl:.3e} (limit {FP32_TOL:.1e})"


PARAM_ORDER = ("Wq", "Wk", "Wv", "Wo", "ln1_scale", "ln1_shift", "W1", "b1", "W2", "b2", "ln2_scale", "ln2_shift")


def unpack_layers(flat, D, H, dk, dv, F, L):
    shapes = {"Wq": (D, H * dk), "Wk": (D, H * dk), "Wv": (D, H * dv), "Wo": (H * dv, D), "ln1_scale": (D,),
              "ln1_shift": (D,), "W1": (D, F), "b1": (F,), "W2": (F, D), "b2": (D,), "ln2_scale": (D,), "ln2_shift": (D,)}
    out, off = [], 0
    for _ in range(L):
        layer = {}
        for k in PARAM_ORDER:
            n = int(np.prod(shapes[k]))
            layer[k] = flat[off:off + n].reshape(shapes[k]).copy()
            off += n
        out.append(layer)
    assert off == flat.size
    return out


def dropout_keep_mask(shape, rate, seed, counter):
    """The device's dropout mask regenerated on the host: the 32-bit hash documented in include/dl4s_cuda.h over the
    row-major element index, kept where hash < floor((1 - rate) * 2^32). Returns float32 0/1 of `shape`."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.uint64)
    M = np.uint64(0xFFFFFFFF)
    lo = (i & M).astype(np.uint64)
    hi = (i >> np.uint64(32)).astype(np.uint64)
    seed = int(seed)
    h = (lo * np.uint64(0x9E3779B1) + np.uint64(seed & 0xFFFFFFFF)) & M
    h ^= h >> np.uint64(16); h = (h * np.uint64(0x85EBCA6B)) & M
    h ^= h >> np.uint64(13); h = (h * np.uint64(0xC2B2AE35)) & M
    h ^= h >> np.uint64(16)
    h = (h + ((hi ^ np.uint64(counter)) & M) * np.uint64(0x27D4EB2F) + np.uint64((seed >> 32) & 0xFFFFFFFF)) & M
    h ^= h >> np.uint64(15); h = (h * np.uint64(0x2C1B3C6D)) & M
    h ^= h >> np.uint64(12); h = (h * np.uint64(0x297A2D39)) & M
    h ^= h >> np.uint64(15)
    keep = (1.0 - float(np.float32(rate))) * 4294967296.0
    thr = 0xFFFFFFFF if keep >= 4294967295.0 else max(1, int(keep))
    return (h < np.uint64(thr)).astype(np.float32).reshape(shape)
