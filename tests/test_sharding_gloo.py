"""CPU tier: the multi-GPU layout of MultiHeadAttention (heads over ranks, one all-gather, second half by batch
slice) checked among world_size-2 and -4 gloo ranks, with the CPU oracle standing in for the device kernels.
What is under test is the host logic of dl4s_b200/sharded.py: the column slices, the rank-major gather layout,
the row rebuild and the batch split; and bench.py's max-over-ranks reduction."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, causal):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    from dl4s_b200 import sharded
    from oracle import oracle as O
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)                       # same seed on every rank: replicated input and weights
        B, S, D, H, dk = 5, 12, 32, 4, 8                      # B not divisible by the world size on purpose
        x = rng.standard_normal((B, S, D), dtype=np.float32)
        W = {n: (rng.standard_normal((D, H * dk)) * 0.2).astype(np.float32) for n in ("qDense", "kDense", "vDense")}
        W["fc"] = (rng.standard_normal((H * dk, D)) * 0.2).astype(np.float32)
        lens = np.array([12, 7, 1, 12, 9], np.int32)
        mask = O.make_decoder_mask(lens, S) if causal else O.make_encoder_mask(lens, S)
        one, zero = np.ones(D, np.float32), np.zeros(D, np.float32)
        want = O.mha(x, x, x, W["qDense"], W["kDense"], W["vDense"], W["fc"], one, zero, H, mask)

        # first half on the rank's heads (oracle: projections with the column slices, attention per head)
        h0, h1 = sharded.head_range(H, world, rank)
        Hl = h1 - h0
        wq, wk, wv = (sharded.slice_head_columns(W[n], H, world, rank) for n in ("qDense", "kDense", "vDense"))
        split = lambda t: t.reshape(B, S, Hl, dk).transpose(0, 2, 1, 3)
        q, k, v = split(O.gemm(x.reshape(-1, D), wq)), split(O.gemm(x.reshape(-1, D), wk)), split(O.gemm(x.reshape(-1, D), wv))
        heads_local = np.ascontiguousarray(O.sdpa(q, k, v, mask).transpose(0, 2, 1, 3).reshape(B, S, Hl * dk))
        # the one collective
        gathered = torch.empty((world,) + heads_local.shape, dtype=torch.float32)
        dist.all_gather_into_tensor(gathered.view(-1), torch.from_numpy(heads_local).reshape(-1))
        b0, b1 = sharded.batch_range(B, world, rank)
        rows = sharded.rows_from_gathered(gathered.numpy(), b0, b1)
        # second half on the rank's batch slice
        pr = O.gemm(rows.reshape(-1, H * dk), W["fc"]).reshape(b1 - b0, S, D) + x[b0:b1]
        got = O.layernorm(pr, one, zero) if b1 > b0 else pr
        assert got.shape == want[b0:b1].shape
        if b1 > b0:
            err = float(np.abs(got - want[b0:b1]).max())
            assert err <= 1e-5, f"rank {rank}: sharded result differs from the unsharded layer by {err}"
        # every batch element is owned exactly once
        owned = torch.zeros(B)
        owned[b0:b1] = 1
        dist.all_reduce(owned)
        assert bool((owned == 1).all())
        # the chunked schedule (the gather of one chunk overlaps the next chunk's compute on the device): every chunk
        # is a complete small layer; the second half reads the gathered buffer in place as column groups
        chunks = 2
        outs = []
        for c0, c1, lb0, lb1, out0 in sharded.chunk_plan(B, world, rank, chunks):
            Bc = c1 - c0
            g_c = torch.empty((world, Bc, S, Hl * dk), dtype=torch.float32)
            dist.all_gather_into_tensor(g_c.view(-1), torch.from_numpy(np.ascontiguousarray(heads_local[c0:c1])).reshape(-1))
            assert out0 == len(outs)
            if lb1 == lb0:
                continue
            rows_c = sharded.rows_from_groups(g_c.numpy().reshape(-1), world, Bc * S * Hl * dk, lb0 * S * Hl * dk,
                                              (lb1 - lb0) * S, Hl * dk)
            pr_c = O.gemm(rows_c, W["fc"]).reshape(lb1 - lb0, S, D) + x[c0 + lb0:c0 + lb1]
            outs.extend(O.layernorm(pr_c, one, zero))
        mine = sharded.owned_batches(B, world, rank, chunks)
        assert len(mine) == len(outs)
        for b, o in zip(mine, outs):
            assert float(np.abs(o - want[b]).max()) <= 1e-5
        owned = torch.zeros(B)
        owned[mine] = 1
        dist.all_reduce(owned)
        assert bool((owned == 1).all())
        # bench.py's timing reduction: max over ranks
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,causal", [(2, False), (2, True), (4, True)])
def test_head_sharded_mha_equals_unsharded(world, causal):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), causal), nprocs=world, join=True)


def test_ranges_cover_everything():
    sys.path.insert(0, ROOT)
    from dl4s_b200 import sharded
    for world in (1, 2, 4, 8):
        heads = [sharded.head_range(32, world, r) for r in range(world)]
        assert heads[0][0] == 0 and heads[-1][1] == 32 and all(a[1] == b[0] for a, b in zip(heads, heads[1:]))
        for B in (1, 7, 8, 256):
            bs = [sharded.batch_range(B, world, r) for r in range(world)]
            assert bs[0][0] == 0 and bs[-1][1] == B and all(a[1] == b[0] for a, b in zip(bs, bs[1:]))
            for chunks in (1, 3, 4, 300):
                owned = [b for r in range(world) for b in sharded.owned_batches(B, world, r, chunks)]
                assert sorted(owned) == list(range(B)), "every batch element is finished by exactly one rank"
                for r in range(world):
                    plan = sharded.chunk_plan(B, world, r, chunks)
                    assert plan[0][0] == 0 and plan[-1][1] == B and all(a[1] == b[0] for a, b in zip(plan, plan[1:]))
                    assert [p[4] for p in plan] == list(np.cumsum([0] + [p[3] - p[2] for p in plan[:-1]]))
    with pytest.raises(ValueError):
        sharded.head_range(6, 4, 0)


def test_library_plan_equals_the_python_statement():
    """dl4s_cuda_mha_sharded_plan (host arithmetic inside the library, the split dl4s_cuda_mha_forward_sharded uses)
    against the index helpers the gloo ranks above are checked with."""
    import ctypes
    sys.path.insert(0, ROOT)
    from dl4s_b200 import sharded
    from dl4s_b200._lib import call
    for world in (1, 2, 4, 8):
        for B in (1, 5, 8, 256):
            for chunks in (1, 3, 4, 64, 300):
                seen = []
                for r in range(world):
                    rows = ctypes.c_int64(-1)
                    idx = (ctypes.c_int64 * B)()
                    call("dl4s_cuda_mha_sharded_plan", B, world, r, chunks, ctypes.byref(rows), idx)
                    got = [int(idx[i]) for i in range(rows.value)]
                    want = sharded.owned_batches(B, world, r, min(chunks, 64) if world > 1 else 1)
                    assert got == want, (world, B, chunks, r)
                    seen += got
                assert sorted(seen) == list(range(B))


def test_rows_from_groups_is_the_rank_major_gather_read_in_place():
    sys.path.insert(0, ROOT)
    from dl4s_b200 import sharded
    G, B, S, C = 3, 4, 5, 2
    gathered = np.arange(G * B * S * C, dtype=np.float32).reshape(G, B, S, C)
    for b0, b1 in ((0, 4), (1, 3), (3, 4)):
        want = sharded.rows_from_gathered(gathered, b0, b1).reshape(-1, G * C)
        got = sharded.rows_from_groups(gathered.reshape(-1), G, B * S * C, b0 * S * C, (b1 - b0) * S, C)
        assert np.array_equal(got, want)
