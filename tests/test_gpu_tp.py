"""Tensor-parallel MLP block and column-sharded GEMM on real GPUs (NCCL, one process per
GPU).  Skipped when fewer than two devices are visible."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    rng = np.random.Generator(np.random.Philox(3))
    t, d, f = 512, 1024, 2752
    x = rng.normal(0, 1, (t, d)).astype(np.float16)
    gain = np.ones(d, np.float16)
    wg = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wu = rng.normal(0, 0.02, (d, f)).astype(np.float16)
    wd = rng.normal(0, 0.02, (f, d)).astype(np.float16)
    return x, gain, wg, wu, wd


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    import hexagon_mlir_b200 as hm
    from hexagon_mlir_b200 import tp
    hm.init(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    x, gain, wg, wu, wd = _problem()
    T = lambda a: torch.from_numpy(a).cuda()
    block = tp.TensorParallelMLP(T(gain), tp.shard_columns(T(wg), rank, world), tp.shard_columns(T(wu), rank, world),
                                 tp.shard_rows(T(wd), rank, world), eps=1e-6, group=dist.group.WORLD, chunks=2)
    xt = T(x)
    out = torch.zeros_like(xt)
    for _ in range(2):
        block(xt, out)
    torch.cuda.synchronize()
    status = hm.device_status()
    lo, hi = tp.shard_bounds(wg.shape[1], rank, world)
    cshard = torch.zeros((x.shape[0], hi - lo), dtype=torch.float16, device="cuda")
    tp.ColumnShardedGemm(rank, world)(xt, tp.shard_columns(T(wg), rank, world), cshard)
    torch.cuda.synchronize()
    # the same block with the reduction fused into the kernels (peer stores over NVLink)
    fused = tp.FusedTensorParallelMLP(T(gain), tp.shard_columns(T(wg), rank, world), tp.shard_columns(T(wu), rank, world),
                                      tp.shard_rows(T(wd), rank, world), tokens=x.shape[0], eps=1e-6,
                                      group=dist.group.WORLD, timeout_ms=20000)
    runs = [fused(xt).clone() for _ in range(3)]
    torch.cuda.synchronize()
    status = status or hm.device_status()
    fused_same = all(torch.equal(r, runs[0]) for r in runs)
    # the all-reduce by the library's own kernel over the switch's multicast addresses, where the
    # machine maps them (bit-identical on every rank and run to run, or skipped)
    mc_out = None
    # barrier kernels around the launch / both rendezvous inside it / the fused call with two token
    # chunks, each chunk's all-reduce beside the next chunk's GEMM
    for rdv, ch in (("barriers", 1), ("own_barriers", 1), ("kernel", 1), ("entry", 1), ("kernel", 2)):
        mc = tp.MulticastTensorParallelMLP(T(gain), tp.shard_columns(T(wg), rank, world), tp.shard_columns(T(wu), rank, world),
                                           tp.shard_rows(T(wd), rank, world), tokens=x.shape[0], eps=1e-6,
                                           group=dist.group.WORLD, timeout_ms=20000, rendezvous=rdv, chunks=ch)
        if not mc.available():
            break
        mruns = [mc(xt).clone() for _ in range(3)]
        mruns.append(mc.captured(xt).clone())     # and replayed from a captured graph (the flag epoch lives on the device)
        mruns.append(mc.captured(xt).clone())
        torch.cuda.synchronize()
        mc.release()
        status = status or hm.device_status()
        same = all(torch.equal(r, mruns[0]) for r in mruns)
        if mc_out is not None:
            got = mruns[0].cpu().numpy()
            if ch == 1:
                same = same and bool(np.array_equal(mc_out[0], got))  # both rendezvous forms: the same bytes
            else:  # chunked down GEMMs may take another variant (fp32 sums associated differently)
                same = same and bool(np.abs(got.astype(np.float32) - mc_out[0].astype(np.float32)).max()
                                     <= 2.0 ** -8 * np.abs(mc_out[0].astype(np.float32)).max())
            got = None
        mc_out = (mruns[0].cpu().numpy() if mc_out is None else mc_out[0], same and (mc_out is None or mc_out[1]))
    # the library's own communicator exists (the block created it): a host-buffer GEMM whose A every
    # rank holds — each rank uploads its row slab of every panel, the slabs are all-gathered on the GPUs
    on, lib_rank, lib_world = hm.tp_info()
    rng = np.random.Generator(np.random.Philox(11))
    m, k, n_loc = 4096, 4096, 4224
    ha = rng.uniform(-1, 1, (m, k)).astype(np.float16)                      # the same on every rank
    hb = np.random.Generator(np.random.Philox(12 + rank)).uniform(-1, 1, (k, n_loc)).astype(np.float16)
    hc = np.zeros((m, n_loc), np.float16)
    hm.set_option("replicatedOperandA", 1)
    hm.matmul[(1,)](ha, hb, hc)
    hm.set_option("replicatedOperandA", 0)
    status = status or hm.device_status()
    rows = np.arange(0, m, 97)
    import oracle
    want = oracle.gemm_f16(np.ascontiguousarray(ha[rows]), hb).astype(np.float32)
    host_err = float(np.abs(hc[rows].astype(np.float32) - want).max() / np.abs(want).max())
    # a narrow column block under a tall A: more row panels than column panels, the slab exchanges
    # on their own stream beside the uploads
    m2, n2 = 12288, 1280
    ha2 = rng.uniform(-1, 1, (m2, k)).astype(np.float16)
    hb2 = np.ascontiguousarray(hb[:, :n2])
    hc2 = np.zeros((m2, n2), np.float16)
    hm.set_option("replicatedOperandA", 1)
    hm.matmul[(1,)](ha2, hb2, hc2)
    hm.set_option("replicatedOperandA", 0)
    status = status or hm.device_status()
    rows2 = np.arange(0, m2, 251)
    want2 = oracle.gemm_f16(np.ascontiguousarray(ha2[rows2]), hb2).astype(np.float32)
    host_err = max(host_err, float(np.abs(hc2[rows2].astype(np.float32) - want2).max() / np.abs(want2).max()))
    # the same call with the slabs forced through ncclAllGather is not run here: the mode is fixed
    # per process; which one ran is reported
    slab_mode = hm.tp_slab_exchange_mode()
    q.put((rank, status, out.cpu().numpy(), lo, hi, cshard.cpu().numpy(), runs[0].cpu().numpy(), fused_same,
           (on, lib_rank, lib_world), host_err, mc_out, slab_mode))
    dist.barrier()
    hm.tp_shutdown()
    q.close()
    q.join_thread()  # results flushed to the parent
    os._exit(0)      # (tearing the group down under live symmetric-memory mappings can block)


@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_mlp_on_gpus(oracle, cuda, world):
    if cuda.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    x, gain, wg, wu, wd = _problem()
    want = oracle.mlp(x, gain, wg, wu, wd, 1e-6).astype(np.float32)
    full = np.zeros((x.shape[0], wg.shape[1]), np.float16)
    for rank, status, out, lo, hi, cshard, fused_out, fused_same, lib_group, host_err, mc_out, slab_mode in results:
        assert status == 0
        assert slab_mode in ("copy engines", "ncclAllGather") and slab_mode == results[0][11]  # every rank took the same form
        assert lib_group == (True, rank, world)       # ncclAllReduce ran inside the library, on its own communicator
        assert host_err <= 1e-2, (rank, host_err)      # sharded upload + all-gather of A
        if mc_out is not None:
            merr = np.abs(mc_out[0].astype(np.float32) - want).max() / np.abs(want).max()
            assert merr <= 1e-2 and mc_out[1], (rank, merr)
            assert np.array_equal(mc_out[0], results[0][10][0])
        err = np.abs(out.astype(np.float32) - want).max() / np.abs(want).max()
        assert err <= 1e-2, (rank, err)
        full[:, lo:hi] = cshard
        # fused form: fp16 partials summed in fp32 by the row owner; every rank ends with the same bytes
        ferr = np.abs(fused_out.astype(np.float32) - want).max() / np.abs(want).max()
        assert ferr <= 1e-2, (rank, ferr)
        assert fused_same
    assert np.array_equal(results[0][6], results[1][6])
    assert np.array_equal(results[0][2], results[1][2])
    ref = oracle.gemm_f16(x, wg).astype(np.float32)
    assert np.abs(full.astype(np.float32) - ref).max() / np.abs(ref).max() <= 1e-2
