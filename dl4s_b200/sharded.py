"""MultiHeadAttention with its heads spread over the GPUs of one node.

DL4S itself is single-device. Attention is independent per (batch, head) — the
reference literally loops over them (Tensor/Operators/Matrix.swift:106-114) — so
a layer that spans G GPUs splits like this:

  rank g  holds the columns of Wq/Wk/Wv that belong to heads [g*H/G, (g+1)*H/G)
          (column-parallel projections, no communication), runs attention on its
          heads for the whole batch -> O_g [B, S, (H/G)*dv]             (kernel side:
          dl4s_cuda_mha_heads_forward)
  all ranks  ONE collective: all-gather of O_g over NCCL / NVLink -> [G, B, S, (H/G)*dv]
  rank g  takes ITS batch slice (DL4S's LayerNorm inside MultiHeadAttention normalises
          a whole [S, D] block per batch element, so the second half is split by
          batch), applies Wo, the residual and the LayerNorm
          (dl4s_cuda_mha_output_forward, which reads the rank-major gather buffer in
          place as G column groups). The output stays sharded by batch.

With `chunks` > 1 the batch is worked through in chunks, each a complete small layer,
and the all-gather of chunk c runs on a second stream while chunk c+1 computes.

The layer, its NCCL communicator, the second stream and the gather buffers live behind
the C ABI (dl4s_cuda_comm_* and dl4s_cuda_mha_forward_sharded in include/dl4s_cuda.h);
this module binds them and needs neither torch nor any other Python package for the
collective. How the 128-byte communicator id gets from rank 0 to the other ranks is the
launcher's business (bench.py broadcasts it over its process group, the tests use a
pipe). The pure index helpers below restate the library's batch split for the CPU tests.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np


def head_range(heads: int, world: int, rank: int) -> Tuple[int, int]:
    if heads % world != 0:
        raise ValueError(f"{heads} heads do not split evenly over {world} ranks")
    per = heads // world
    return rank * per, (rank + 1) * per


def batch_range(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous batch slice of a rank; the first `batch % world` ranks take one extra element."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def slice_head_columns(w: np.ndarray, heads: int, world: int, rank: int) -> np.ndarray:
    """Columns of a projection matrix [D, heads*d] that belong to the rank's heads."""
    d = w.shape[1] // heads
    h0, h1 = head_range(heads, world, rank)
    return np.ascontiguousarray(w[:, h0 * d:h1 * d])


def rows_from_gathered(gathered: np.ndarray, b0: int, b1: int) -> np.ndarray:
    """[G, B, S, C] (rank-major all-gather result) -> [b1-b0, S, G*C]: the head-concatenated rows of a batch
    slice, heads in global order (rank g contributed heads g*H/G ...). numpy statement of the strided device copy."""
    G, B, S, C = gathered.shape
    return np.ascontiguousarray(gathered[:, b0:b1].transpose(1, 2, 0, 3).reshape(b1 - b0, S, G * C))


def rows_from_groups(flat: np.ndarray, groups: int, group_stride: int, offset: int, M: int, C: int) -> np.ndarray:
    """The addressing dl4s_cuda_mha_output_forward applies to a gathered buffer it reads in place:
    rows[m, g*C + c] = flat[offset + g*group_stride + m*C + c]."""
    g = np.arange(groups)[None, :, None]
    m = np.arange(M)[:, None, None]
    c = np.arange(C)[None, None, :]
    return np.ascontiguousarray(flat[offset + g * group_stride + m * C + c].reshape(M, groups * C))


def chunk_plan(batch: int, world: int, rank: int, chunks: int):
    """The batch is worked through in `chunks` contiguous chunks so that the all-gather of one chunk runs while the
    next chunk's projections and attention compute. Every chunk is a complete small layer: all ranks run its heads,
    gather, and each rank finishes ITS slice of the chunk. Returns one tuple per chunk:
    (c0, c1, lb0, lb1, out0) = the chunk's batch range, the rank's slice inside the chunk (relative to c0) and the
    row of the rank's output buffer where that slice goes."""
    chunks = max(1, min(chunks, batch))
    plan, out0 = [], 0
    for c in range(chunks):
        c0, c1 = batch_range(batch, chunks, c)
        lb0, lb1 = batch_range(c1 - c0, world, rank)
        plan.append((c0, c1, lb0, lb1, out0))
        out0 += lb1 - lb0
    return plan


def owned_batches(batch: int, world: int, rank: int, chunks: int):
    """Global batch indices of the rows of a rank's output, in output order."""
    idx = []
    for c0, _c1, lb0, lb1, _o in chunk_plan(batch, world, rank, chunks):
        idx.extend(range(c0 + lb0, c0 + lb1))
    return idx


def comm_unique_id() -> bytes:
    """Rank 0: the 128-byte id every rank passes to comm_init."""
    import ctypes
    from ._lib import call
    buf = (ctypes.c_uint8 * 128)()
    call("dl4s_cuda_comm_unique_id", buf)
    return bytes(buf)


def comm_init(rank: int, world: int, unique_id: Optional[bytes] = None) -> None:
    """The current device joins the communicator (collective: every rank calls it)."""
    import ctypes
    from ._lib import call
    if world > 1:
        assert unique_id is not None and len(unique_id) == 128
        buf = (ctypes.c_uint8 * 128).from_buffer_copy(unique_id)
        call("dl4s_cuda_comm_init", rank, world, buf)
    else:
        call("dl4s_cuda_comm_init", rank, world, None)


def comm_destroy() -> None:
    from ._lib import call
    call("dl4s_cuda_comm_destroy")


def comm_info() -> Tuple[int, int, int]:
    """(rank, world, NCCL version in use or 0)."""
    import ctypes
    from ._lib import call
    r, w, v = ctypes.c_int32(0), ctypes.c_int32(1), ctypes.c_int32(0)
    call("dl4s_cuda_comm_info", ctypes.byref(r), ctypes.byref(w), ctypes.byref(v))
    return r.value, w.value, v.value


def comm_timing() -> Tuple[float, float]:
    """(gather ms, exposed ms) of the last sharded forward on this device; waits for it."""
    import ctypes
    from ._lib import call
    g, e = ctypes.c_float(0), ctypes.c_float(0)
    call("dl4s_cuda_comm_timing", ctypes.byref(g), ctypes.byref(e))
    return g.value, e.value


class HeadShardedMultiHeadAttention:
    """The layer above on the CUDA device. Call comm_init on every rank first (a device that never joined runs as a
    world of one). Construct on every rank with the FULL host weights; each rank uploads only its column slices.
    `__call__(x, mask)` takes the full input [B, S, D] (replicated on every rank) and returns this rank's part of the
    output [len(owned_batches), S, D] as a ShapedBuffer. With chunks > 1 (and more than one rank) the gather of
    chunk c runs on a second stream under the compute of chunk c+1. Every rank must make the same calls in the same
    order: each call contains collectives."""

    def __init__(self, heads: int, hiddenDim: int, keyDim: int, valueDim: int, weights: dict,
                 precision: Optional[int] = None, chunks: int = 1):
        from . import cuda
        self.cuda = cuda
        self.rank, self.world, _ = comm_info()
        self.heads, self.keyDim, self.valueDim, self.hiddenDim = heads, keyDim, valueDim, hiddenDim
        h0, h1 = head_range(heads, self.world, self.rank)
        self.local_heads = h1 - h0
        self.precision = precision
        self.chunks = chunks if self.world > 1 else 1
        self.qDense = cuda.tensor(slice_head_columns(weights["qDense"], heads, self.world, self.rank))
        self.kDense = cuda.tensor(slice_head_columns(weights["kDense"], heads, self.world, self.rank))
        self.vDense = cuda.tensor(slice_head_columns(weights["vDense"], heads, self.world, self.rank))
        self.fc = cuda.tensor(weights["fc"])
        self.norm_scale = cuda.tensor(weights.get("norm_scale", np.ones(hiddenDim, np.float32)))
        self.norm_shift = cuda.tensor(weights.get("norm_shift", np.zeros(hiddenDim, np.float32)))

    def owned_batches(self, batch: int):
        """Global batch indices of the rows of this rank's output, in output order (asked of the library)."""
        import ctypes
        from ._lib import call
        rows = ctypes.c_int64(0)
        idx = (ctypes.c_int64 * max(batch, 1))()
        call("dl4s_cuda_mha_sharded_plan", batch, self.world, self.rank, self.chunks, ctypes.byref(rows), idx)
        return [int(idx[i]) for i in range(rows.value)]

    def __call__(self, x, mask=None, out=None):
        from ._lib import c_vp, call
        from .cuda import CUDAEngine, StructuredMask
        cuda = self.cuda
        B, S, D = x.shape
        lens_ptr, causal = 0, 0
        if mask is not None:
            assert isinstance(mask, StructuredMask), "the sharded layer takes structural masks"
            lens_ptr = mask.lengths.ptr if mask.lengths is not None else 0
            causal = int(mask.causal)
        prec = CUDAEngine.precision if self.precision is None else self.precision
        rows_out = len(self.owned_batches(B))
        out = out or cuda.CUDA.Memory.allocateBuffer((rows_out, S, D))
        call("dl4s_cuda_mha_forward_sharded", c_vp(x.ptr), B, S, D, self.heads, self.keyDim, self.valueDim,
             c_vp(self.qDense.ptr), c_vp(self.kDense.ptr), c_vp(self.vDense.ptr), c_vp(self.fc.ptr),
             c_vp(self.norm_scale.ptr), c_vp(self.norm_shift.ptr), c_vp(lens_ptr), causal, c_vp(out.ptr), prec, self.chunks)
        return out
