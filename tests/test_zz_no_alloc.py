"""GPU tier, collected last: the decode entry point that allocates nothing.

dl4s_cuda_sdpa_decode_noalloc serves hosts that cannot call cudaMalloc where decode runs (all of HBM already
handed to their own cache manager, or a step that cannot take cudaMalloc's device-wide synchronisation). Its
split-K records live in a fixed array inside the library instead of the growing scratch arena. The array is
shared by all calls and keeps the previous call's contents, so the check runs two different problems back to
back and compares each with the allocating entry point and with the CPU oracle.
"""
import ctypes

import numpy as np
import pytest

from util import FP32_TOL, assert_close

pytestmark = pytest.mark.gpu


def _decode_both(dev, q, k, v, lens):
    from dl4s_b200._lib import c_f32, c_vp, call
    B, H, _, d = q.shape
    L = k.shape[2]
    tq, tk, tv = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    tl = dev.tensor(lens, np.int32) if lens is not None else None
    lp = c_vp(tl.ptr) if tl is not None else c_vp(0)
    temperature = c_f32(float(np.sqrt(np.float32(d))))
    ref = dev.CUDA.Memory.allocateBuffer((B, H, 1, d))
    out = dev.CUDA.Memory.allocateBuffer((B, H, 1, d))
    call("dl4s_cuda_sdpa_decode", c_vp(tq.ptr), c_vp(tk.ptr), c_vp(tv.ptr), B, H, L, d, d, temperature, lp, c_vp(ref.ptr))
    call("dl4s_cuda_sdpa_decode_noalloc", c_vp(tq.ptr), c_vp(tk.ptr), c_vp(tv.ptr), B, H, L, d, temperature, lp, c_vp(out.ptr))
    return out.numpy(), ref.numpy()


def _oracle_decode(oracle, q, k, v, lens):
    L = k.shape[2]
    mask = None if lens is None else oracle.make_encoder_mask(np.clip(lens, 0, L), L)
    return oracle.sdpa(q, k, v, mask)


def test_noalloc_decode_matches_allocating_entry_point_twice_in_a_row(dev, oracle):
    rng = np.random.default_rng(99)
    # first call: long ragged contexts, many split-K records
    B, H, L, d = 3, 4, 3000, 128
    q = rng.standard_normal((B, H, 1, d), dtype=np.float32)
    k = rng.standard_normal((B, H, L, d), dtype=np.float32)
    v = rng.standard_normal((B, H, L, d), dtype=np.float32)
    lens = np.array([3000, 1, 1777], np.int32)
    got, want = _decode_both(dev, q, k, v, lens)
    assert_close(got, want, FP32_TOL, FP32_TOL, "first call")
    assert_close(got, _oracle_decode(oracle, q, k, v, lens), FP32_TOL, FP32_TOL, "first call against the CPU oracle")
    # second call right after: a different, smaller problem whose records overlay the first call's leftovers
    B, H, L, d = 2, 3, 700, 64
    q = rng.standard_normal((B, H, 1, d), dtype=np.float32)
    k = rng.standard_normal((B, H, L, d), dtype=np.float32) * 3
    v = rng.standard_normal((B, H, L, d), dtype=np.float32) + 5
    got, want = _decode_both(dev, q, k, v, None)
    assert_close(got, want, FP32_TOL, FP32_TOL, "second call")
    # values of O(5) summed over 700 keys: the CPU engine's one-after-the-other fp32 sum is itself only good to ~1e-5
    # absolute here, so against the oracle the bound is relative to the largest |value|
    want_cpu = _oracle_decode(oracle, q, k, v, None)
    assert_close(got, want_cpu, FP32_TOL * float(np.abs(want_cpu).max()), FP32_TOL, "second call against the CPU oracle")
    assert dev.device_status() == 0


def test_noalloc_decode_uses_larger_chunks_when_records_would_not_fit(dev):
    """1024 (batch, head) pairs x 4096 keys need chunks of 512 keys to fit the fixed array."""
    rng = np.random.default_rng(100)
    B, H, L, d = 16, 64, 4096, 128
    q = rng.standard_normal((B, H, 1, d), dtype=np.float32)
    slab_k = rng.standard_normal((1, H, L, d), dtype=np.float32)
    slab_v = rng.standard_normal((1, H, L, d), dtype=np.float32)
    k = np.broadcast_to(slab_k, (B, H, L, d)).copy()
    v = np.broadcast_to(slab_v, (B, H, L, d)).copy()
    lens = rng.integers(1, L + 1, size=B).astype(np.int32)
    got, want = _decode_both(dev, q, k, v, lens)
    assert_close(got, want, FP32_TOL, FP32_TOL, "chunked to fit")


def test_noalloc_decode_rejects_oversized_problems(dev):
    from dl4s_b200 import DL4SCudaError
    from dl4s_b200._lib import c_f32, c_vp, call
    buf = dev.CUDA.Memory.allocateBuffer((64,))
    # 65535 x 8 pairs x 130 floats exceed the fixed array even with one chunk per pair: nothing is launched,
    # so the tiny buffer is never touched.
    n0 = dev.launch_count()
    with pytest.raises(DL4SCudaError) as e:
        call("dl4s_cuda_sdpa_decode_noalloc", c_vp(buf.ptr), c_vp(buf.ptr), c_vp(buf.ptr), 65535, 8, 128, 128, c_f32(1.0), c_vp(0),
             c_vp(buf.ptr))
    assert "too large for the fixed scratch" in str(e.value)
    with pytest.raises(DL4SCudaError):
        call("dl4s_cuda_sdpa_decode_noalloc", c_vp(buf.ptr), c_vp(buf.ptr), c_vp(buf.ptr), 1, 1, 128, 96, c_f32(1.0), c_vp(0),
             c_vp(buf.ptr))
    assert dev.launch_count() == n0
    # an empty batch is a no-op, as for the allocating entry point
    call("dl4s_cuda_sdpa_decode_noalloc", c_vp(buf.ptr), c_vp(buf.ptr), c_vp(buf.ptr), 0, 4, 128, 128, c_f32(1.0), c_vp(0), c_vp(buf.ptr))
    assert dev.launch_count() == n0


def test_noalloc_decode_clamps_a_length_beyond_the_cache(dev, oracle):
    rng = np.random.default_rng(101)
    B, H, L, d = 2, 2, 300, 64
    q = rng.standard_normal((B, H, 1, d), dtype=np.float32)
    k = rng.standard_normal((B, H, L, d), dtype=np.float32)
    v = rng.standard_normal((B, H, L, d), dtype=np.float32)
    lens = np.array([L + 9, 17], np.int32)
    got, want = _decode_both(dev, q, k, v, lens)
    assert_close(got, want, FP32_TOL, FP32_TOL, "clamped length")
    assert_close(got, _oracle_decode(oracle, q, k, v, lens), FP32_TOL, FP32_TOL, "clamped length against the CPU oracle")
