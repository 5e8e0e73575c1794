"""GPU tier, two GPUs: dl4s_cuda_mha_forward_sharded with its NCCL all-gather, through the C ABI by ctypes, one
process per GPU (spawned here; the communicator id travels through a pipe). Each rank checks the batch rows it owns
against the CPU oracle's unsharded layer. Skipped on a box with one GPU; the single-GPU tests emulate the two
halves of the layer on one device and the CPU tier checks the index arithmetic among gloo ranks."""
import multiprocessing as mp
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, conn, prec_name, chunks, result):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from dl4s_b200 import PREC_F16, PREC_FP32, cuda, sharded, workloads
        from oracle import oracle as O
        from util import FP32_TOL, TC_MAX_ABS, TC_REL_L2, max_abs, rel_l2
        cuda.init([rank])
        if rank == 0:
            ident = sharded.comm_unique_id()
            for c in conn:
                c.send(ident)
        else:
            ident = conn.recv()
        sharded.comm_init(rank, world, ident)
        assert sharded.comm_info()[:2] == (rank, world) and sharded.comm_info()[2] > 0
        prec = PREC_FP32 if prec_name == "fp32" else PREC_F16
        B, S, D, H = 5, 256, 512, 8                     # B not divisible by the world size on purpose
        c = workloads.mha_config(B=B, S=S, D=D, H=H)
        lens = np.array([256, 100, 1, 256, 177], np.int32)
        layer = sharded.HeadShardedMultiHeadAttention(H, D, D // H, D // H, c["weights"], precision=prec, chunks=chunks)
        x = cuda.tensor(c["x"])
        mask = cuda.StructuredMask(lens, causal=True)
        got1 = layer(x, mask).numpy()
        got = layer(x, mask).numpy()                      # a second call reuses the gather buffers and events
        assert np.array_equal(got, got1)
        w = c["weights"]
        one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
        O.set_threads(4)
        want = O.mha(c["x"], c["x"], c["x"], w["qDense"], w["kDense"], w["vDense"], w["fc"], one, zero, H,
                     O.make_decoder_mask(lens, S))
        mine = layer.owned_batches(B)
        assert got.shape == (len(mine), S, D)
        if mine:
            ma, rl = max_abs(got, want[mine]), rel_l2(got, want[mine])
            lim = (FP32_TOL, FP32_TOL) if prec == PREC_FP32 else (TC_MAX_ABS, TC_REL_L2)
            assert ma <= lim[0] and rl <= lim[1], (rank, ma, rl)
        assert cuda.device_status() == 0
        sharded.comm_destroy()
        result.put((rank, mine, None))
    except Exception as e:      # report instead of hanging the other rank's collective check
        import traceback
        result.put((rank, None, traceback.format_exc()))
        raise


@pytest.mark.parametrize("prec,chunks", [("fp32", 1), ("f16", 1), ("f16", 2)])
def test_two_ranks_equal_the_unsharded_layer(dev, prec, chunks):
    import ctypes
    from dl4s_b200._lib import load
    n = ctypes.c_int32(0)
    load().dl4s_cuda_device_count(ctypes.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    pipes = [ctx.Pipe() for _ in range(world - 1)]
    result = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(0, world, [p[0] for p in pipes], prec, chunks, result))]
    procs += [ctx.Process(target=_rank, args=(r, world, pipes[r - 1][1], prec, chunks, result)) for r in range(1, world)]
    for p in procs:
        p.start()
    owned, errors = [], []
    for _ in procs:
        rank, mine, err = result.get(timeout=300)
        if err:
            errors.append(f"rank {rank}:\n{err}")
        else:
            owned += mine
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert not errors, "\n".join(errors)
    assert sorted(owned) == list(range(5))
