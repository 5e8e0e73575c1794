"""GPU tier: the fp32 EngineType / MemoryOperatorsType primitives through the C ABI against numpy restatements of
the DL4S CPU engine's semantics (Engine/CPU/CPUEngine.swift)."""
import numpy as np
import pytest

from util import assert_fp32_rel, max_abs

pytestmark = pytest.mark.gpu


def up(dev, a, dtype=np.float32):
    return dev.tensor(a, dtype)


def test_memory_roundtrip_views_and_values(dev):
    M = dev.CUDA.Memory
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = up(dev, a)
    assert np.array_equal(t.numpy(), a)
    assert M.getSize(t) == 24 and M.getValue(t) == 0.0
    adv = M.advance(t, 5)
    assert M.getValue(adv) == 5.0
    M.setPointee(adv, -1.0)
    assert t.numpy().ravel()[5] == -1.0
    M.setPointee(adv, 5.0)
    view, is_copy, shape = M.get([1], t)            # leading prefix: a view
    assert not is_copy and shape == (3, 4) and np.array_equal(view.numpy(), a[1])
    sl, is_copy, shape = M.get([None, 2], t)        # not a prefix: a copy
    assert is_copy and shape == (2, 4) and np.array_equal(sl.numpy(), a[:, 2])
    M.set([None, None, 1], t, up(dev, np.full((2, 3), 7, np.float32)))
    b = a.copy(); b[:, :, 1] = 7
    assert np.array_equal(t.numpy(), b)
    c = M.allocateBuffer((2, 3, 4))
    M.assign(t, c)
    assert np.array_equal(c.numpy(), b)


def test_elementwise(dev):
    E = dev.CUDA.Engine
    rng = np.random.default_rng(0)
    for n in (1, 7, 1024, 100003):
        a = rng.standard_normal(n).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32) + 3
        ta, tb, out = up(dev, a), up(dev, b), dev.CUDA.Memory.allocateBuffer((n,))
        for fn, ref in ((E.vAdd, a + b), (E.vSub, a - b), (E.vMul, a * b), (E.vDiv, a / b)):
            fn(ta, tb, out)
            assert np.array_equal(out.numpy(), ref)
        for fn, ref in ((E.vNeg, -a), (E.relu, np.maximum(a, 0)), (E.heaviside, (a > 0).astype(np.float32))):
            fn(ta, out)
            assert np.array_equal(out.numpy(), ref)
        for fn, ref in ((E.exp, np.exp(a)), (E.tanh, np.tanh(a)), (E.sin, np.sin(a)), (E.cos, np.cos(a)),
                        (E.sqrt, np.sqrt(np.abs(a))), (E.log, np.log(np.abs(a) + 1))):
            src = ta
            if fn is E.sqrt: src = up(dev, np.abs(a))
            if fn is E.log: src = up(dev, np.abs(a) + 1)
            fn(src, out)
            assert_fp32_rel(out.numpy(), ref, fn.__name__)
        E.fill(2.5, out)
        assert (out.numpy() == 2.5).all()
    # log(exp(x)) ~ x at 1e-4, the reference's own check (VecTests.swift:158-168)
    x = rng.uniform(-5, 5, 100).astype(np.float32)
    tx, o1, o2 = up(dev, x), dev.CUDA.Memory.allocateBuffer((100,)), dev.CUDA.Memory.allocateBuffer((100,))
    E.exp(tx, o1); E.log(o1, o2)
    assert max_abs(o2.numpy(), x) < 1e-4


@pytest.mark.parametrize("ls,rs", [((4, 3, 5), (5,)), ((4, 3, 5), (4, 1, 1)), ((4, 1, 5), (1, 3, 1)), ((6,), ()),
                                   ((2, 3, 4, 5), (2, 1, 1, 5)), ((1, 5), (7, 1)), ((3, 1), (3, 1))])
def test_broadcast(dev, ls, rs):
    E = dev.CUDA.Engine
    rng = np.random.default_rng(1)
    a = rng.standard_normal(ls).astype(np.float32)
    b = (rng.standard_normal(rs).astype(np.float32) + 2.5)
    out_shape = np.broadcast_shapes(ls, rs)
    ta, tb, out = up(dev, a), up(dev, b), dev.CUDA.Memory.allocateBuffer(out_shape)
    E.broadcastAdd(ta, tb, out); assert np.array_equal(out.numpy(), a + b)
    E.broadcastSub(ta, tb, out); assert np.array_equal(out.numpy(), a - b)
    E.broadcastMul(ta, tb, out); assert np.array_equal(out.numpy(), a * b)
    E.broadcastDiv(ta, tb, out)
    # vector / broadcast scalar is a multiplication by the fp32 reciprocal (CPUEngine.swift:628-636)
    la = (1,) * (len(out_shape) - len(ls)) + tuple(ls)
    ra = (1,) * (len(out_shape) - len(rs)) + tuple(rs)
    recip = False
    for d in reversed(range(len(out_shape))):
        if la[d] > ra[d]: recip = True; break
        if ra[d] > la[d] or la[d] > 1: break
    want = a * (np.float32(1) / b) if recip else a / b
    assert np.array_equal(out.numpy(), want.astype(np.float32))


@pytest.mark.parametrize("shape,axes", [((4, 5, 6), [2]), ((4, 5, 6), [1, 2]), ((4, 5, 6), [0]), ((3, 4000), [1]),
                                        ((2, 3, 4, 5), [1, 3]), ((7,), [0])])
def test_reduce(dev, shape, axes):
    E = dev.CUDA.Engine
    rng = np.random.default_rng(2)
    a = rng.standard_normal(shape).astype(np.float32)
    ta = up(dev, a)
    rshape = tuple(s for i, s in enumerate(shape) if i not in axes)
    out = dev.CUDA.Memory.allocateBuffer(rshape or (1,))
    E.reduceSum(ta, out, axes=axes)
    assert_fp32_rel(out.numpy().reshape(rshape), a.astype(np.float64).sum(axis=tuple(axes)), "reduceSum")
    E.reduceMax(ta, out, axes=axes)
    assert np.array_equal(out.numpy().reshape(rshape), a.max(axis=tuple(axes)))
    if len(axes) == 1:
        ctx = dev.CUDA.Memory.allocateBuffer(rshape or (1,), np.int32)
        E.reduceMax(ta, out, context=ctx, axis=axes[0])
        assert np.array_equal(ctx.numpy().reshape(rshape), a.argmax(axis=axes[0]).astype(np.int32))


def test_permute_uses_the_reference_convention(dev):
    """Source axis i becomes destination axis arangement[i] (Shape.swift:127-129)."""
    E = dev.CUDA.Engine
    a = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    for arr in ([0, 2, 1, 3], [1, 2, 3, 0], [3, 0, 1, 2], [0, 1, 2, 3]):
        dst_shape = [0] * 4
        for i, d in enumerate(arr): dst_shape[d] = a.shape[i]
        out = dev.CUDA.Memory.allocateBuffer(dst_shape)
        E.permuteAxes(up(dev, a), out, arr)
        want = np.transpose(a, np.argsort(arr))   # numpy: result axis j takes source axis perm[j]
        assert np.array_equal(out.numpy(), want)


def test_stack_and_band(dev):
    E = dev.CUDA.Engine
    rng = np.random.default_rng(3)
    parts = [rng.standard_normal((2, n, 3)).astype(np.float32) for n in (1, 4, 2)]
    out = dev.CUDA.Memory.allocateBuffer((2, 7, 3))
    E.stack([up(dev, p) for p in parts], out, axis=1)
    assert np.array_equal(out.numpy(), np.concatenate(parts, axis=1))
    out0 = dev.CUDA.Memory.allocateBuffer((6, 4, 3))
    same = [rng.standard_normal((2, 4, 3)).astype(np.float32) for _ in range(3)]
    E.stack([up(dev, p) for p in same], out0, axis=0)
    assert np.array_equal(out0.numpy(), np.concatenate(same, axis=0))
    # unstack / unstackAdd are the inverse (Engine.swift:543,551)
    back = [dev.CUDA.Memory.allocateBuffer(p.shape) for p in parts]
    E.unstack(out, back, axis=1)
    for b_, p in zip(back, parts):
        assert np.array_equal(b_.numpy(), p)
    adds = [rng.standard_normal(p.shape).astype(np.float32) for p in parts]
    E.unstackAdd(out, [up(dev, a) for a in adds], back, axis=1)
    for b_, p, a in zip(back, parts, adds):
        assert np.array_equal(b_.numpy(), p + a)
    back0 = [dev.CUDA.Memory.allocateBuffer(p.shape) for p in same]
    E.unstack(out0, back0, axis=0)
    for b_, p in zip(back0, same):
        assert np.array_equal(b_.numpy(), p)
    ones = np.ones((5, 7), np.float32)
    b = dev.CUDA.Memory.allocateBuffer((5, 7))
    E.band(up(dev, ones), b, belowDiagonal=-1, aboveDiagonal=None)   # the causal mask of makeDecoderMasks
    assert np.array_equal(b.numpy(), np.triu(ones, 1))
    E.band(up(dev, ones), b, belowDiagonal=1, aboveDiagonal=0)
    assert np.array_equal(b.numpy(), np.tril(ones) - np.tril(ones, -2))


@pytest.mark.parametrize("M,N,K", [(1, 1, 3), (2, 3, 3), (33, 65, 17), (128, 128, 64), (300, 200, 100),
                                   (1, 512, 512), (7, 700, 900), (40, 1024, 2048), (64, 1536, 640)])   # few rows: split-K kernel
def test_gemm_fp32_all_transposes(dev, oracle, M, N, K):
    E = dev.CUDA.Engine
    rng = np.random.default_rng(4)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    for ta in (False, True):
        for tb in (False, True):
            a = A.T.copy() if ta else A
            b = B.T.copy() if tb else B
            out = dev.CUDA.Memory.allocateBuffer((M, N))
            E.gemm(up(dev, a), up(dev, b), out, transposeFirst=ta, transposeSecond=tb)
            assert_fp32_rel(out.numpy(), oracle.gemm(a, b, trans_a=ta, trans_b=tb), f"gemm ta={ta} tb={tb}")
    # alpha / beta
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    out = up(dev, C0)
    E.gemm(up(dev, A), up(dev, B), out, alpha=0.5, beta=2.0)
    assert_fp32_rel(out.numpy(), 0.5 * (A.astype(np.float64) @ B.astype(np.float64)) + 2.0 * C0, "alpha/beta")


def test_gemm_known_answers_from_reference_tests(dev):
    E = dev.CUDA.Engine
    c = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    out = dev.CUDA.Memory.allocateBuffer((3, 3))
    E.gemm(up(dev, c), up(dev, c), out, transposeFirst=True)
    assert out.numpy().tolist() == [[17, 22, 27], [22, 29, 36], [27, 36, 45]]
    out = dev.CUDA.Memory.allocateBuffer((2, 2))
    E.gemm(up(dev, c), up(dev, c), out, transposeSecond=True)
    assert out.numpy().tolist() == [[14, 32], [32, 77]]


def test_errors_are_reported_not_fatal(dev):
    from dl4s_b200 import DL4SCudaError
    E = dev.CUDA.Engine
    a = up(dev, np.zeros((2, 3), np.float32))
    b = up(dev, np.zeros((4, 5), np.float32))
    with pytest.raises(DL4SCudaError):
        E.broadcastAdd(a, b, dev.CUDA.Memory.allocateBuffer((4, 5)))
    assert dev.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 256, 64), (300, 256, 192), (1000, 512, 256),
                                   (4096 + 77, 1024, 512), (20000, 1536, 128), (2048, 192, 320), (260, 256, 1024),
                                   (4096 + 77, 1024, 1088), (40000, 512, 1024)])
def test_gemm_tensor_core_shapes(dev, M, N, K):
    """Tensor-core product (half operands, fp32 accumulation) against the float64 product of the half-rounded
    operands: single-CTA tiles, two-CTA tiles (256-column tiles with at least 256 rows and K >= 1024), ragged last row tile,
    more tiles than SMs (tiles handed out by the device counter), 128- and 256-column tiles."""
    from dl4s_b200 import PREC_F16
    E = dev.CUDA.Engine
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.1).astype(np.float32)
    out = dev.CUDA.Memory.allocateBuffer((M, N))
    E.gemm(up(dev, A), up(dev, B), out, precision=PREC_F16)
    got = out.numpy()
    want = A.astype(np.float16).astype(np.float64) @ B.astype(np.float16).astype(np.float64)
    err = np.abs(got - want).max()
    assert err <= 2e-5 * max(1.0, np.abs(want).max()) * np.sqrt(K), f"max error {err} vs the product of the rounded operands"
    assert dev.device_status() == 0
    # twice in a row: the work counters are left clean by the first launch
    E.gemm(up(dev, A), up(dev, B), out, precision=PREC_F16)
    assert np.array_equal(out.numpy(), got)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1000, 512, 256), (4096 + 77, 1536, 512), (300, 256, 1024), (2048, 192, 320)])
def test_gemm_split_weights(dev, M, N, K):
    """DL4S_PREC_F16_SPLIT: the second operand enters as two halves (rounded value + rounded remainder), so only the
    first operand's rounding remains. Checked against the float64 product of the half-rounded A with the exact B:
    the error must be far below what rounding B once would leave."""
    from dl4s_b200 import PREC_F16, PREC_F16_SPLIT
    E = dev.CUDA.Engine
    rng = np.random.default_rng(M * 3 + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.1).astype(np.float32)
    out = dev.CUDA.Memory.allocateBuffer((M, N))
    E.gemm(up(dev, A), up(dev, B), out, precision=PREC_F16_SPLIT)
    got = out.numpy()
    Ah = A.astype(np.float16).astype(np.float64)
    want = Ah @ B.astype(np.float64)
    single = Ah @ B.astype(np.float16).astype(np.float64)
    err, err_single = np.abs(got - want).max(), np.abs(single - want).max()
    assert err <= 2e-5 * max(1.0, np.abs(want).max()) * np.sqrt(K), f"max error {err} vs the product with the exact second operand"
    assert err < 0.1 * err_single, f"split weights leave {err}, single-rounded weights {err_single}"
    assert dev.device_status() == 0


def test_operand_outside_the_half_range_is_reported(dev):
    """A tensor-core operand at or above 65504 becomes infinite when rounded to half: the conversion sets a bit in
    the device status word, which reads back as an error and is cleared by the read."""
    from dl4s_b200 import DL4SCudaError, PREC_F16
    E = dev.CUDA.Engine
    A = np.ones((128, 64), np.float32)
    A[5, 7] = 1e5
    B = np.ones((64, 128), np.float32)
    out = dev.CUDA.Memory.allocateBuffer((128, 128))
    E.gemm(up(dev, A), up(dev, B), out, precision=PREC_F16)
    with pytest.raises(DL4SCudaError) as e:
        dev.device_status()
    assert "half range" in str(e.value) and e.value.status == -1
    assert dev.device_status() == 0
    # the same values are fine in fp32
    E.gemm(up(dev, A), up(dev, B), out)
    assert dev.device_status() == 0
    assert out.numpy()[5, 0] == np.float32(1e5 + 63)


def test_bounded_wait_runs_out_and_is_reported(dev):
    """A bounded device-side wait that runs out: the next single-CTA tensor-core product is told to leave out one
    operand load and to poll with a short limit. Its MMA thread's wait on that stage gives up, every role leaves
    through the kernel's normal exit (tensor memory freed, nothing traps or spins), the status word reads back as
    DL4S_ERR_TIMEOUT, and the device works normally afterwards."""
    from dl4s_b200 import DL4SCudaError, PREC_F16
    from dl4s_b200._lib import call
    E = dev.CUDA.Engine
    rng = np.random.default_rng(8)
    A = rng.standard_normal((128, 128)).astype(np.float32)
    B = rng.standard_normal((128, 128)).astype(np.float32)
    a, b = up(dev, A), up(dev, B)
    out = dev.CUDA.Memory.allocateBuffer((128, 128))
    assert dev.device_status() == 0
    call("dl4s_cuda_inject_failure", 4, 1)
    E.gemm(a, b, out, precision=PREC_F16)          # one tile, one CTA, two k-blocks: the second is never loaded
    with pytest.raises(DL4SCudaError) as e:
        dev.device_status()
    assert e.value.status == -5 and "wait gave up" in str(e.value)
    assert dev.device_status() == 0                # cleared by the read
    E.gemm(a, b, out, precision=PREC_F16)          # the same launch without the fault
    want = A.astype(np.float16).astype(np.float64) @ B.astype(np.float16).astype(np.float64)
    assert np.abs(out.numpy() - want).max() <= 1e-3
    assert dev.device_status() == 0


@pytest.mark.parametrize("M,N,K,ta,tb", [(256, 128, 64, True, False), (256, 128, 64, False, True), (1000, 512, 256, True, True),
                                         (1000, 512, 256, False, True), (512, 2048, 16384 // 32, True, False), (4096 + 80, 192, 320, False, True)])
def test_gemm_tensor_core_transposed(dev, M, N, K, ta, tb):
    """The products of a matmul's backward (dA = dC B^T, dB = A^T dC, Matrix.swift:139-173) on the tensor cores:
    operands stored transposed, against the float64 product of the half-rounded operands."""
    from dl4s_b200 import PREC_F16
    E = dev.CUDA.Engine
    rng = np.random.default_rng(M + 7 * N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.1).astype(np.float32)
    a = np.ascontiguousarray(A.T) if ta else A
    b = np.ascontiguousarray(B.T) if tb else B
    out = dev.CUDA.Memory.allocateBuffer((M, N))
    dev.profile_begin()
    E.gemm(up(dev, a), up(dev, b), out, transposeFirst=ta, transposeSecond=tb, precision=PREC_F16)
    prof = dev.profile_end()
    assert "k_gemm_tc.transposed" in prof, sorted(prof)
    got = out.numpy()
    want = A.astype(np.float16).astype(np.float64) @ B.astype(np.float16).astype(np.float64)
    err = np.abs(got - want).max()
    assert err <= 2e-5 * max(1.0, np.abs(want).max()) * np.sqrt(K), f"max error {err} vs the product of the rounded operands"
    assert dev.device_status() == 0
