"""Host-side mirror of the DL4S plug-in boundary for a CUDA device.

DL4S selects a back-end by type parameter: `Tensor<Float, Device>` calls the
static functions of `Device.Memory` (protocol MemoryOperatorsType,
Sources/DL4S/Engine/Engine.swift:39-139) and `Device.Engine` (protocol
EngineType, Engine.swift:143-581). This module restates that boundary in Python
on top of the C ABI (include/dl4s_cuda.h): `CUDA.Memory` and `CUDA.Engine` have
the same function names and argument meaning; `ShapedBuffer` plays the role of
DL4S's ShapedBuffer (Engine/Buffer.swift:85-107).

Nothing here computes: every method forwards to libdl4s_cuda.so and raises
DL4SCudaError when the library reports a failure (DL4S aborts the process on
the same conditions).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import c_i32, c_i64, c_f32, c_vp, call

_initialised = False


def init(devices: Optional[Sequence[int]] = None) -> None:
    """Create the device state (context, stream, scratch arena)."""
    global _initialised
    if devices is None:
        call("dl4s_cuda_init", None, 0)
    else:
        arr = (ctypes.c_int32 * len(devices))(*devices)
        call("dl4s_cuda_init", arr, len(devices))
    _initialised = True


def _ensure_init() -> None:
    if not _initialised:
        init()


def synchronize() -> None:
    call("dl4s_cuda_sync")


def device_status() -> int:
    w = ctypes.c_int32(0)
    call("dl4s_cuda_device_status", ctypes.byref(w))
    return w.value


def launch_count() -> int:
    n = ctypes.c_uint64(0)
    call("dl4s_cuda_launch_count", ctypes.byref(n))
    return n.value


def profile_begin() -> None:
    call("dl4s_cuda_profile_begin")


def profile_end() -> dict:
    """-> {kernel name: {"launches": n, "total_ms": t}} since profile_begin."""
    import json
    buf = ctypes.create_string_buffer(1 << 16)
    call("dl4s_cuda_profile_end", buf, len(buf))
    return json.loads(buf.value.decode() or "{}")


class Graph:
    """The calls made inside `with Graph() as g:` are recorded into a CUDA graph instead of run; `g.launch()`
    replays them with one launch. Buffers must exist before, and the same calls must have run once eagerly (the
    scratch arena has its size then); pointers and shapes are baked in."""

    def __init__(self):
        self._handle = c_vp(0)

    def __enter__(self):
        call("dl4s_cuda_graph_begin")
        return self

    def __exit__(self, exc_type, exc, tb):
        try:
            call("dl4s_cuda_graph_end", ctypes.byref(self._handle))
        except Exception:
            if exc_type is None:
                raise
        return False

    def launch(self) -> None:
        call("dl4s_cuda_graph_launch", self._handle)

    def destroy(self) -> None:
        if self._handle:
            call("dl4s_cuda_graph_destroy", self._handle)
            self._handle = c_vp(0)


def set_stream(cuda_stream: Optional[int]) -> None:
    call("dl4s_cuda_set_stream", c_vp(cuda_stream or 0))


def _i64arr(values):
    values = [int(v) for v in values]
    return (ctypes.c_int64 * max(1, len(values)))(*values)


def _i32arr(values):
    values = [int(v) for v in values]
    return (ctypes.c_int32 * max(1, len(values)))(*values)


class ShapedBuffer:
    """A device buffer with a shape. `parent` is set for views (advance /
    prefix slices), which share storage and are never freed on their own,
    like TensorHandle.parent in Tensor/Tensor.swift:29-43."""

    __slots__ = ("ptr", "shape", "dtype", "parent", "_owned")

    def __init__(self, ptr: int, shape, dtype=np.float32, parent=None, owned=True):
        self.ptr = int(ptr)
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.parent = parent
        self._owned = owned and parent is None

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def dim(self) -> int:
        return len(self.shape)

    @property
    def nbytes(self) -> int:
        return self.count * self.dtype.itemsize

    def view(self, *shape) -> "ShapedBuffer":
        """Tensor.view(as:) — metadata only (Tensor/Operators/Shape.swift:40-67)."""
        shape = list(shape[0]) if len(shape) == 1 and not isinstance(shape[0], int) else list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.count // max(known, 1)
        v = ShapedBuffer(self.ptr, shape, self.dtype, parent=self.parent or self)
        assert v.count == self.count, "view must keep the element count"
        return v

    def numpy(self) -> np.ndarray:
        return CUDA.Memory.assign_to_host(self)

    def free(self) -> None:
        CUDA.Memory.free(self)

    def __del__(self):
        try:
            if self._owned and self.ptr:
                _lib.load().dl4s_cuda_free(c_vp(self.ptr))
                self.ptr = 0
        except Exception:
            pass


def tensor(array, dtype=np.float32) -> ShapedBuffer:
    """Upload a host array (Tensor.init from an array + Memory.assign, Tensor.swift:116-153)."""
    a = np.ascontiguousarray(array, dtype=dtype)
    buf = CUDA.Memory.allocateBuffer(a.shape, dtype)
    CUDA.Memory.assign_from_host(a, buf)
    return buf


class CUDAMemoryOperators:
    """MemoryOperatorsType for the CUDA device (Engine.swift:39-139; the CPU
    counterpart is Engine/CPU/CPU.swift:35-231)."""

    @staticmethod
    def allocateBuffer(withShape, type=np.float32) -> ShapedBuffer:
        _ensure_init()
        shape = (withShape,) if isinstance(withShape, int) else tuple(withShape)
        n = 1
        for s in shape:
            n *= int(s)
        p = c_vp(0)
        call("dl4s_cuda_malloc", n * np.dtype(type).itemsize, ctypes.byref(p))
        return ShapedBuffer(p.value or 0, shape, type)

    @staticmethod
    def free(buffer: ShapedBuffer) -> None:
        if buffer._owned and buffer.ptr:
            call("dl4s_cuda_free", c_vp(buffer.ptr))
            buffer.ptr = 0
            buffer._owned = False

    @staticmethod
    def assign_from_host(source: np.ndarray, destination: ShapedBuffer, count: Optional[int] = None) -> None:
        src = np.ascontiguousarray(source, dtype=destination.dtype)
        n = src.size if count is None else count
        call("dl4s_cuda_memcpy_h2d", c_vp(destination.ptr), c_vp(src.ctypes.data), n * src.itemsize)

    @staticmethod
    def assign_to_host(source: ShapedBuffer, destination: Optional[np.ndarray] = None,
                       count: Optional[int] = None) -> np.ndarray:
        out = np.empty(source.shape, source.dtype) if destination is None else destination
        n = source.count if count is None else count
        call("dl4s_cuda_memcpy_d2h", c_vp(out.ctypes.data), c_vp(source.ptr), n * source.dtype.itemsize)
        return out

    @staticmethod
    def assign(source: ShapedBuffer, destination: ShapedBuffer, count: Optional[int] = None) -> None:
        n = source.count if count is None else count
        call("dl4s_cuda_memcpy_d2d", c_vp(destination.ptr), c_vp(source.ptr), n * source.dtype.itemsize)

    @staticmethod
    def getValue(source: ShapedBuffer) -> float:
        v = ctypes.c_float(0)
        call("dl4s_cuda_get_value_f32", c_vp(source.ptr), ctypes.byref(v))
        return v.value

    @staticmethod
    def getSize(buffer: ShapedBuffer) -> int:
        return buffer.count

    @staticmethod
    def setPointee(buffer: ShapedBuffer, newValue: float) -> None:
        call("dl4s_cuda_set_value_f32", c_vp(buffer.ptr), c_f32(newValue))

    @staticmethod
    def advance(buffer: ShapedBuffer, by: int) -> ShapedBuffer:
        """Same storage, start moved by `by` elements (CPU.swift:223-231)."""
        return ShapedBuffer(buffer.ptr + by * buffer.dtype.itemsize, (buffer.count - by,), buffer.dtype,
                            parent=buffer.parent or buffer)

    @staticmethod
    def get(slice, of: ShapedBuffer):
        """get(slice:of:with:) for an index list of ints / None (Engine.swift:100;
        CPU.swift:137-174): a leading-prefix index returns a view (isCopy False),
        anything else a strided copy. Returns (buffer, isCopy, shape)."""
        buf = of
        idx = list(slice) + [None] * (buf.dim - len(slice))
        strides = _strides(buf.shape)
        lead = 0
        while lead < len(idx) and idx[lead] is not None:
            lead += 1
        if all(i is None for i in idx[lead:]):
            off = sum(idx[d] * strides[d] for d in range(lead))
            shape = buf.shape[lead:]
            return ShapedBuffer(buf.ptr + off * buf.dtype.itemsize, shape, buf.dtype, parent=buf.parent or buf), False, shape
        keep = [d for d in range(buf.dim) if idx[d] is None]
        off = sum(idx[d] * strides[d] for d in range(buf.dim) if idx[d] is not None)
        shape = tuple(buf.shape[d] for d in keep)
        out = CUDAMemoryOperators.allocateBuffer(shape, buf.dtype)
        call("dl4s_cuda_copy_strided_f32", c_vp(buf.ptr), _i64arr([strides[d] for d in keep]), off, c_vp(out.ptr),
             _i64arr(_strides(shape)), 0, _i64arr(shape), len(shape))
        return out, True, shape

    @staticmethod
    def set(slice, of: ShapedBuffer, source: ShapedBuffer) -> None:
        """set(slice:of:with:from:with:) (Engine.swift:117; CPU.swift:196-213)."""
        buf = of
        idx = list(slice) + [None] * (buf.dim - len(slice))
        strides = _strides(buf.shape)
        keep = [d for d in range(buf.dim) if idx[d] is None]
        off = sum(idx[d] * strides[d] for d in range(buf.dim) if idx[d] is not None)
        shape = tuple(buf.shape[d] for d in keep)
        assert source.count == int(np.prod(shape, dtype=np.int64)), "source does not fill the slice"
        call("dl4s_cuda_copy_strided_f32", c_vp(source.ptr), _i64arr(_strides(shape)), 0, c_vp(buf.ptr),
             _i64arr([strides[d] for d in keep]), off, _i64arr(shape), len(shape))


def _strides(shape):
    """MemoryOps.strides (Memory Management/MemoryOps.swift:253-278)."""
    s, out = 1, []
    for e in reversed(shape):
        out.append(s)
        s *= int(e)
    return tuple(reversed(out))


class StructuredMask:
    """Attention mask kept in structural form: per-sequence key lengths
    (makeEncoderMasks, TransformerUtil.swift:29-36) and/or the causal band
    (makeDecoderMasks, TransformerUtil.swift:38-50). The kernels apply it in
    the tile and never materialise it."""

    def __init__(self, key_lengths=None, causal: bool = False, max_len: Optional[int] = None):
        self.host_lengths = None if key_lengths is None else np.ascontiguousarray(key_lengths, np.int32)
        self.causal = bool(causal)
        self.max_len = max_len if max_len is not None else (
            int(self.host_lengths.max()) if self.host_lengths is not None else None)
        self.lengths = None if self.host_lengths is None else tensor(self.host_lengths, np.int32)

    def dense(self, Sq: int, Sk: int) -> np.ndarray:
        """The fp32 0/1 tensor DL4S would build, [B or 1, 1, Sq or 1, Sk]."""
        B = 1 if self.host_lengths is None else len(self.host_lengths)
        m = np.zeros((B, 1, Sq if self.causal else 1, Sk), np.float32)
        if self.host_lengths is not None:
            m = np.maximum(m, (np.arange(Sk)[None, :] >= self.host_lengths[:, None]).astype(np.float32)[:, None, None, :])
        if self.causal:
            m = np.maximum(m, (np.arange(Sk)[None, :] > np.arange(Sq)[:, None]).astype(np.float32)[None, None])
        return m


def makeEncoderMasks(sequenceLengths) -> StructuredMask:
    return StructuredMask(sequenceLengths, causal=False)


def makeDecoderMasks(sequenceLengths) -> StructuredMask:
    return StructuredMask(sequenceLengths, causal=True)


def _mask_args(mask):
    """-> (lengths_ptr, causal, dense_ptr, dense_shape_array, keepalive)"""
    if mask is None:
        return c_vp(0), 0, c_vp(0), None, None
    if isinstance(mask, StructuredMask):
        lp = c_vp(mask.lengths.ptr) if mask.lengths is not None else c_vp(0)
        return lp, int(mask.causal), c_vp(0), None, mask
    assert isinstance(mask, ShapedBuffer) and mask.dim == 4, "dense masks are 4-D ShapedBuffers"
    return c_vp(0), 0, c_vp(mask.ptr), _i64arr(mask.shape), mask


class CUDAEngine:
    """EngineType for the CUDA device (Engine.swift:143-581): the fp32
    primitives an attention graph uses, plus fused hooks for the hot path."""

    precision = _lib.PREC_F16  # arithmetic of the fused hooks; PREC_FP32 selects the FFMA check kernels

    # ---- element-wise ----
    @staticmethod
    def fill(value, result: ShapedBuffer, count: Optional[int] = None):
        n = result.count if count is None else count
        if result.dtype == np.int32:
            call("dl4s_cuda_fill_i32", c_i32(int(value)), c_vp(result.ptr), n)
        else:
            call("dl4s_cuda_fill_f32", c_f32(value), c_vp(result.ptr), n)

    @staticmethod
    def _binary(name, lhs, rhs, result, count):
        n = result.count if count is None else count
        call(name, c_vp(lhs.ptr), c_vp(rhs.ptr), c_vp(result.ptr), n)

    @staticmethod
    def vAdd(lhs, rhs, result, count=None): CUDAEngine._binary("dl4s_cuda_vadd", lhs, rhs, result, count)
    @staticmethod
    def vSub(lhs, rhs, result, count=None): CUDAEngine._binary("dl4s_cuda_vsub", lhs, rhs, result, count)
    @staticmethod
    def vMul(lhs, rhs, result, count=None): CUDAEngine._binary("dl4s_cuda_vmul", lhs, rhs, result, count)
    @staticmethod
    def vDiv(lhs, rhs, result, count=None): CUDAEngine._binary("dl4s_cuda_vdiv", lhs, rhs, result, count)

    @staticmethod
    def _unary(name, values, result):
        call(name, c_vp(values.ptr), c_vp(result.ptr), result.count)

    @staticmethod
    def vNeg(val, result, count=None): CUDAEngine._unary("dl4s_cuda_vneg", val, result)
    @staticmethod
    def exp(values, result): CUDAEngine._unary("dl4s_cuda_exp", values, result)
    @staticmethod
    def log(values, result): CUDAEngine._unary("dl4s_cuda_log", values, result)
    @staticmethod
    def sqrt(values, result): CUDAEngine._unary("dl4s_cuda_sqrt", values, result)
    @staticmethod
    def relu(values, result): CUDAEngine._unary("dl4s_cuda_relu", values, result)
    @staticmethod
    def heaviside(values, result): CUDAEngine._unary("dl4s_cuda_heaviside", values, result)
    @staticmethod
    def sin(values, result): CUDAEngine._unary("dl4s_cuda_sin", values, result)
    @staticmethod
    def cos(values, result): CUDAEngine._unary("dl4s_cuda_cos", values, result)
    @staticmethod
    def tanh(values, result): CUDAEngine._unary("dl4s_cuda_tanh", values, result)

    # ---- broadcast ----
    @staticmethod
    def _broadcast(name, lhs, rhs, result):
        call(name, c_vp(lhs.ptr), _i64arr(lhs.shape), lhs.dim, c_vp(rhs.ptr), _i64arr(rhs.shape), rhs.dim,
             c_vp(result.ptr))

    @staticmethod
    def broadcastAdd(lhs, rhs, result): CUDAEngine._broadcast("dl4s_cuda_broadcast_add", lhs, rhs, result)
    @staticmethod
    def broadcastSub(lhs, rhs, result): CUDAEngine._broadcast("dl4s_cuda_broadcast_sub", lhs, rhs, result)
    @staticmethod
    def broadcastMul(lhs, rhs, result): CUDAEngine._broadcast("dl4s_cuda_broadcast_mul", lhs, rhs, result)
    @staticmethod
    def broadcastDiv(lhs, rhs, result): CUDAEngine._broadcast("dl4s_cuda_broadcast_div", lhs, rhs, result)

    # ---- reduce ----
    @staticmethod
    def reduceSum(values, result, axes=None, axis=None):
        axes = [axis] if axes is None else list(axes)
        call("dl4s_cuda_reduce_sum", c_vp(values.ptr), _i64arr(values.shape), values.dim, _i32arr(axes), len(axes),
             c_vp(result.ptr))

    @staticmethod
    def reduceMax(values, result, context=None, axes=None, axis=None):
        axes = [axis] if axes is None else list(axes)
        call("dl4s_cuda_reduce_max", c_vp(values.ptr), _i64arr(values.shape), values.dim, _i32arr(axes), len(axes),
             c_vp(result.ptr), c_vp(context.ptr if context is not None else 0))

    # ---- layout ----
    @staticmethod
    def permuteAxes(values, result, arangement):
        call("dl4s_cuda_permute_axes", c_vp(values.ptr), _i64arr(values.shape), values.dim, _i32arr(arangement),
             c_vp(result.ptr))

    @staticmethod
    def stack(buffers, result, axis):
        n, dim = len(buffers), buffers[0].dim
        ptrs = (c_vp * n)(*[b.ptr for b in buffers])
        shapes = _i64arr([s for b in buffers for s in b.shape])
        call("dl4s_cuda_stack", ptrs, shapes, n, dim, axis, c_vp(result.ptr))

    @staticmethod
    def unstack(stacked, result, axis):
        """EngineType.unstack (Engine.swift:551): `result` is the list of buffers to fill."""
        n, dim = len(result), result[0].dim
        ptrs = (c_vp * n)(*[b.ptr for b in result])
        call("dl4s_cuda_unstack", c_vp(stacked.ptr), ptrs, _i64arr([s for b in result for s in b.shape]), n, dim, axis)

    @staticmethod
    def unstackAdd(stacked, add, result, axis):
        """EngineType.unstackAdd (Engine.swift:543): result[i] = slab i of `stacked` + add[i]."""
        n, dim = len(result), result[0].dim
        ptrs = (c_vp * n)(*[b.ptr for b in result])
        adds = (c_vp * n)(*[b.ptr for b in add])
        call("dl4s_cuda_unstack_add", c_vp(stacked.ptr), adds, ptrs, _i64arr([s for b in result for s in b.shape]), n, dim, axis)

    @staticmethod
    def band(buffer, result, belowDiagonal=None, aboveDiagonal=None):
        rows, cols = buffer.shape
        call("dl4s_cuda_band", c_vp(buffer.ptr), rows, cols, belowDiagonal or 0, int(belowDiagonal is not None),
             aboveDiagonal or 0, int(aboveDiagonal is not None), c_vp(result.ptr))

    @staticmethod
    def gemm(lhs, rhs, result, alpha=1.0, beta=0.0, transposeFirst=False, transposeSecond=False, precision=None):
        M = lhs.shape[1] if transposeFirst else lhs.shape[0]
        K = lhs.shape[0] if transposeFirst else lhs.shape[1]
        N = rhs.shape[0] if transposeSecond else rhs.shape[1]
        prec = _lib.PREC_FP32 if precision is None else precision
        call("dl4s_cuda_gemm", c_vp(lhs.ptr), c_vp(rhs.ptr), c_vp(result.ptr), M, N, K, c_f32(alpha), c_f32(beta),
             int(transposeFirst), int(transposeSecond), prec)

    # ---- fused hooks (the hot path) ----
    @staticmethod
    def scaledDotProductAttention(q, k, v, mask, temperature, result, precision=None):
        B, H, Sq, dk = q.shape
        Sk, dv = v.shape[2], v.shape[3]
        lp, causal, mp, ms, _keep = _mask_args(mask)
        prec = CUDAEngine.precision if precision is None else precision
        call("dl4s_cuda_sdpa_forward", c_vp(q.ptr), c_vp(k.ptr), c_vp(v.ptr), B, H, Sq, Sk, dk, dv, c_f32(temperature),
             lp, causal, mp, ms, c_vp(result.ptr), prec)

    @staticmethod
    def scaledDotProductAttentionDecode(q, k, v, key_lengths, temperature, result):
        B, H, one, dk = q.shape
        assert one == 1
        Lmax, dv = v.shape[2], v.shape[3]
        lp = c_vp(key_lengths.ptr) if key_lengths is not None else c_vp(0)
        call("dl4s_cuda_sdpa_decode", c_vp(q.ptr), c_vp(k.ptr), c_vp(v.ptr), B, H, Lmax, dk, dv, c_f32(temperature),
             lp, c_vp(result.ptr))

    @staticmethod
    def layerNorm(x, residual, scale, shift, result):
        outer, D = x.shape[0], x.shape[-1]
        rows = x.count // max(outer * D, 1)
        call("dl4s_cuda_layernorm", c_vp(x.ptr), c_vp(residual.ptr if residual is not None else 0), outer, rows, D,
             c_vp(scale.ptr), c_vp(shift.ptr), c_vp(result.ptr))


class CUDA:
    """DeviceType (Engine.swift:30-35)."""
    Memory = CUDAMemoryOperators
    Engine = CUDAEngine
