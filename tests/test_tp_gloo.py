"""Partitioning logic of the multi-GPU configs on CPU ranks (gloo, world size 2): sharded
MLP == unsharded oracle, column-sharded GEMM == oracle.  The compute stand-in is the
oracle (test infrastructure); the product kernels are exercised by the gpu tests."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_problem():
    rng = np.random.Generator(np.random.Philox(3))
    t, d, f = 48, 64, 176
    x = rng.normal(0, 1, (t, d)).astype(np.float16)
    gain = rng.uniform(0.5, 1.5, d).astype(np.float16)
    wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
    return x, gain, wg, wu, wd


def worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from hexagon_mlir_b200 import tp
    x, gain, wg, wu, wd = make_problem()

    def compute(xc, g, a, b, c, out, eps, add_residual):
        xn = xc.numpy()
        h = oracle.rmsnorm(xn, g.numpy(), eps, threads=1)
        act = oracle.swiglu(oracle.gemm_f16(h, a.numpy(), threads=1), oracle.gemm_f16(h, b.numpy(), threads=1), threads=1)
        y = oracle.gemm_f16(act, c.numpy(), threads=1)
        if add_residual:
            y = oracle.add_f16(y, xn, threads=1)
        out.copy_(torch.from_numpy(y))

    T = torch.from_numpy
    block = tp.TensorParallelMLP(T(gain), tp.shard_columns(T(wg), rank, world), tp.shard_columns(T(wu), rank, world),
                                 tp.shard_rows(T(wd), rank, world), eps=1e-6, group=dist.group.WORLD, chunks=3,
                                 compute=compute)
    out = torch.zeros_like(T(x))
    block(T(x), out)
    # column-sharded GEMM: every rank owns a column block, results are disjoint
    lo, hi = tp.shard_bounds(wg.shape[1], rank, world)
    cblock = oracle.gemm_f16(x, np.ascontiguousarray(wg[:, lo:hi]), threads=1)
    q.put((rank, out.numpy(), lo, hi, cblock))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds_cover_and_align():
    from hexagon_mlir_b200 import tp
    for extent in (11008, 16384, 176, 40, 8, 7):
        for world in (1, 2, 4, 8):
            cuts = [tp.shard_bounds(extent, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == extent
            for (l0, h0), (l1, h1) in zip(cuts, cuts[1:]):
                assert h0 == l1
            assert all(lo % 8 == 0 for lo, _ in cuts)
    assert tp.shard_bounds(11008, 3, 8) == (4128, 5504)
    with pytest.raises(ValueError):
        tp.shard_bounds(64, 2, 2)


def test_tensor_parallel_mlp_and_sharded_gemm_world2():
    import oracle
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x, gain, wg, wu, wd = make_problem()
    want = oracle.mlp(x, gain, wg, wu, wd, 1e-6).astype(np.float32)
    full = np.zeros((x.shape[0], wg.shape[1]), np.float16)
    for rank, out, lo, hi, cblock in results:
        err = np.abs(out.astype(np.float32) - want).max() / np.abs(want).max()
        assert err <= 1e-2, (rank, err)  # partial sums are rounded to fp16 before the reduce
        full[:, lo:hi] = cblock
    assert np.array_equal(results[0][1], results[1][1])  # every rank holds the same block output
    assert np.array_equal(full, oracle.gemm_f16(x, wg))
