"""Multi-GPU partitioning of the two configs that shard: the large GEMM (column blocks of
B and C per rank, no collective) and the Llama-style MLP block (column-split gate/up,
row-split down, one all-reduce of the block output).

The reference partitions a decode GEMM the same way inside one device: every program
takes one [K, BN] column block of a single resident weight
(qcom_hexagon_backend/test/Dialect/Hmx/Transforms/weight-resident-nsplit.mlir:9-27);
across GPUs the cut is the same, one process per GPU, torch.distributed for the plumbing.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import launcher as _l


def shard_bounds(extent: int, rank: int, world: int, granule: int = 8):
    """[lo, hi) of this rank's block of `extent`, cut on multiples of `granule` (the
    16-byte alignment the tensor-core path needs for fp16 row strides)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    units = -(-extent // granule)
    lo = min(extent, (rank * units // world) * granule)
    hi = min(extent, ((rank + 1) * units // world) * granule)
    return lo, hi


def shard_columns(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[1], rank, world)
    return t[:, lo:hi].contiguous()


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi].contiguous()


def _device_mlp(x, gain, wg, wu, wd, out, eps, add_residual):
    _l.mlp_block[(1,)](x, gain, wg, wu, wd, out, eps=eps, add_residual=add_residual)


def init_group(group=None) -> None:
    """Create the library's own NCCL communicator over the ranks of `group` (default: the world):
    rank 0 draws the 128-byte id in C++, torch.distributed only carries it to the other ranks."""
    on, _, world = _l.tp_info()
    want = dist.get_world_size(group)
    if on:
        if world != want:
            raise RuntimeError(f"the library's group has {world} ranks, the process group {want}")
        return
    rank = dist.get_rank(group)
    box = [_l.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    _l.tp_init(box[0], rank, want)


class TensorParallelMLP:
    """out = x + down(swiglu(gate(h), up(h))), h = rmsnorm(x)·gain, hidden dimension sharded.

    Each rank holds Wg[:, lo:hi], Wu[:, lo:hi], Wd[lo:hi, :] and computes a partial
    [T, D] output (rank 0's includes the residual); the partials are summed with one
    all-reduce per chunk.  The token dimension can be cut into `chunks` pieces so that the
    all-reduce of piece i runs while piece i+1 is computed.  The whole step — kernels and
    ncclAllReduce — is ONE call into the library (`mlp_block_tp_float16`, C++); this class only
    creates the library's communicator from the process group.  With `compute` given (the CPU tests
    of the partitioning logic inject a stand-in) the same schedule runs in Python over
    torch.distributed instead.
    """

    def __init__(self, gain, wg, wu, wd, eps=1e-6, group=None, chunks=1, compute=None):
        self.gain, self.wg, self.wu, self.wd = gain, wg, wu, wd
        self.eps = float(eps)
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.chunks = max(1, int(chunks))
        self.native = compute is None
        self.compute = compute or _device_mlp
        self._graph = None
        self._graph_key = None
        if self.native and self.world > 1:
            init_group(group)

    def captured(self, x, out):
        """Run the block through a CUDA graph captured on first use for this (x, out) pair.

        The tensor-parallel step is a dozen short launches plus one NCCL call per chunk; issued
        from Python it is bound by the host.  Capturing the whole step (kernels and all-reduces)
        and replaying it removes that cost.  The graph reads and writes the very tensors given
        here: refill `x` in place between replays."""
        key = (x.data_ptr(), out.data_ptr(), tuple(x.shape))
        if self._graph is None or self._graph_key != key:
            self(x, out)  # warm-up outside capture: workspaces, NCCL channels, kernel attributes
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                self(x, out)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    self(x, out)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self._graph, self._graph_key = graph, key
        self._graph.replay()
        return out

    def release(self):
        """Drop the captured graph (it holds the collective's work objects).  Call this before
        the process group is destroyed: tearing the group down under a live graph can block."""
        if self._graph is not None:
            torch.cuda.synchronize()
            self._graph = None
            self._graph_key = None

    def __call__(self, x, out):
        if self.world == 1:
            self.compute(x, self.gain, self.wg, self.wu, self.wd, out, self.eps, True)
            return out
        if self.native:
            _l.mlp_block_tp[(1,)](x, self.gain, self.wg, self.wu, self.wd, out, eps=self.eps, chunks=self.chunks)
            return out
        # rank 0's partial carries the residual (added in its down-projection's epilogue), so the
        # all-reduce delivers the finished block: no partial buffer, no separate add pass
        fold = self.rank == 0
        t = x.shape[0]
        step = -(-t // self.chunks)
        works = []
        for r0 in range(0, t, step):
            r1 = min(t, r0 + step)
            part = out[r0:r1]
            self.compute(x[r0:r1], self.gain, self.wg, self.wu, self.wd, part, self.eps, fold)
            works.append(dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for w in works:
            w.wait()
        return out


class FusedTensorParallelMLP:
    """The same block with the reduction fused into the kernels instead of an all-reduce.

    The ranks' buffers are mapped into each other's address space (torch symmetric memory over
    NVLink).  The down projection's read-out stores each fp16 partial row straight into the
    receive slot of the rank that owns the row (rows are dealt out in `world` contiguous
    blocks), so the reduce-scatter half of the exchange runs under the GEMM; after a barrier a
    small kernel sums each owner's `world` slots in fp32, adds the residual rows and stores the
    finished rows into every rank's output; a second barrier and every rank holds the block
    output.  Partials are rounded to fp16 once and summed in fp32, so the result is at least
    as close to the single-GPU block as the all-reduce form.  Needs tokens divisible by the
    world size and a world of at most 8.
    """

    def __init__(self, gain, wg, wu, wd, tokens, eps=1e-6, group=None, timeout_ms=10000):
        import torch.distributed._symmetric_memory as symm
        if group is None:
            group = dist.group.WORLD
        self.gain, self.wg, self.wu, self.wd = gain, wg, wu, wd
        self.eps = float(eps)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.tokens, self.width = int(tokens), int(wd.shape[1])
        if self.tokens % self.world or self.world > 8:
            raise ValueError("tokens must be divisible by the world size (<= 8)")
        self.rows = self.tokens // self.world
        self.timeout_ms = int(timeout_ms)
        dev = wd.device
        self.recv = symm.empty((self.world, self.rows, self.width), dtype=torch.float16, device=dev)
        self.out = symm.empty((self.tokens, self.width), dtype=torch.float16, device=dev)
        self._h_recv = symm.rendezvous(self.recv, group)
        self._h_out = symm.rendezvous(self.out, group)
        self._recv_ptrs = [int(p) for p in self._h_recv.buffer_ptrs]
        self._out_ptrs = [int(p) for p in self._h_out.buffer_ptrs]

    def captured(self, x):
        """The same step replayed from a CUDA graph captured on first use for this `x` (kernels and
        both barriers); refill `x` in place between replays."""
        key = (x.data_ptr(), tuple(x.shape))
        if getattr(self, "_graph", None) is None or self._graph_key != key:
            self(x)
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                self(x)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    self(x)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self._graph, self._graph_key = graph, key
        self._graph.replay()
        return self.out

    def release(self):
        """Drop the captured graph before the process group or the symmetric buffers go."""
        if getattr(self, "_graph", None) is not None:
            torch.cuda.synchronize()
            self._graph = None

    def __call__(self, x):
        """Returns the block output (a buffer this object owns; valid until the next call)."""
        if tuple(x.shape) != (self.tokens, self.width):
            raise ValueError(f"expected x of shape {(self.tokens, self.width)}")
        _l.mlp_block_push(x, self.gain, self.wg, self.wu, self.wd, self._recv_ptrs, self.world, self.rank, self.eps)
        self._h_recv.barrier(channel=0, timeout_ms=self.timeout_ms)  # every rank's partial rows have landed
        lo = self.rank * self.rows
        _l.tp_reduce_rows(self.recv, x[lo:lo + self.rows], self._out_ptrs, self.world, self.rank)
        self._h_out.barrier(channel=1, timeout_ms=self.timeout_ms)   # every rank's finished rows have landed
        return self.out


class MulticastTensorParallelMLP:
    """The block with its all-reduce done by this library's own kernel over NVSwitch multicast.

    Every rank writes its fp16 partial [T, D] (with the residual in its share of the 256-row blocks:
    options mlpResidualMod / mlpResidualRem) into a symmetric buffer;
    after a barrier each rank sums ITS rows over all ranks' copies with `multimem.ld_reduce` (the
    switch adds in fp32 and rounds once) and writes the sums into every copy with `multimem.st`;
    after a second barrier every rank holds the block output.  Per GPU 1/world of the buffer
    crosses NVLink in each direction.  Needs a multicast mapping (NVSwitch; `available()` tells),
    tokens divisible by the world size.

    rendezvous="kernel" (default): both barriers are inside the all-reduce launch (flag words in
    the symmetric buffer, stored through the multicast address, polled locally, every wait
    bounded); "barriers": the symmetric-memory handle's barrier kernels around the launch; "entry":
    the wait for the other ranks' partials inside the launch, a barrier kernel after it;
    "own_barriers": the whole block as ONE call into the library (`mlp_block_tp_multicast_float16`),
    which puts its own one-warp barrier launches (`b200mlir_tp_barrier`) around the all-reduce.

    chunks > 1 (rendezvous="kernel" only): the whole block is ONE call into the library
    (`mlp_block_tp_multicast_float16`); the down projection is cut into token chunks and each
    chunk's all-reduce runs on a second stream beside the next chunk's GEMM."""

    def __init__(self, gain, wg, wu, wd, tokens, eps=1e-6, group=None, timeout_ms=10000, rendezvous="kernel",
                 chunks=1):
        import torch.distributed._symmetric_memory as symm
        if group is None:
            group = dist.group.WORLD
        self.gain, self.wg, self.wu, self.wd = gain, wg, wu, wd
        self.eps = float(eps)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.tokens, self.width = int(tokens), int(wd.shape[1])
        if self.tokens % self.world:
            raise ValueError("tokens must be divisible by the world size")
        self.rows = self.tokens // self.world
        self.timeout_ms = int(timeout_ms)
        if rendezvous not in ("kernel", "barriers", "entry", "own_barriers"):
            raise ValueError("rendezvous is 'kernel', 'entry', 'barriers' or 'own_barriers'")
        self.rendezvous = rendezvous
        self.chunks = int(chunks)
        if self.chunks > 1 and rendezvous != "kernel":
            raise ValueError("token chunks need rendezvous='kernel'")
        n = self.tokens * self.width
        self._buf = symm.empty((n + 64,), dtype=torch.float16, device=wd.device)  # the output, then 16 flag words
        self._h = symm.rendezvous(self._buf, group)
        off = int(getattr(self._h, "offset", 0) or 0)          # of this tensor inside the rendezvoused allocation
        self._mc = int(getattr(self._h, "multicast_ptr", 0) or 0)
        if self._mc:
            self._mc += off
        self._peers = [int(p) + off for p in self._h.buffer_ptrs]   # every rank's copy, as this process maps it
        self.out = self._buf[:n].view(self.tokens, self.width)
        self._buf[n:].zero_()
        self._state = torch.zeros(4, dtype=torch.int32, device=wd.device)
        torch.cuda.synchronize(wd.device)
        self._h.barrier(channel=0, timeout_ms=self.timeout_ms)  # every rank's flags read zero before the first launch
        torch.cuda.synchronize(wd.device)
        self._graph = None

    def available(self) -> bool:
        return self._mc != 0

    def __call__(self, x):
        """Returns the block output (a buffer this object owns; valid until the next call)."""
        if not self._mc:
            raise RuntimeError("no multicast mapping on this machine")
        if self.chunks > 1 or self.rendezvous == "own_barriers":   # ONE call into the library
            _l.mlp_block_tp_multicast[(1,)](x, self.gain, self.wg, self.wu, self.wd, self.out, mc_buf=self._mc,
                                            peer_bufs=self._peers, flags_elem_offset=self.tokens * self.width, state=self._state,
                                            rank=self.rank, world=self.world, eps=self.eps, chunks=self.chunks)
            return self.out
        _l.set_option("mlpResidualMod", self.world)   # the ranks take turns, by 256-row block, in adding x
        _l.set_option("mlpResidualRem", self.rank)
        try:
            _l.mlp_block[(1,)](x, self.gain, self.wg, self.wu, self.wd, self.out, eps=self.eps, add_residual=True)
        finally:
            _l.set_option("mlpResidualMod", 1)
        n = self.rows * self.width
        if self.rendezvous == "kernel":
            _l.tp_allreduce_multimem_sync(self._mc, self._peers, self.rank * n, n, self.tokens * self.width, self.rank,
                                          self.world, self._state)
            return self.out
        if self.rendezvous == "entry":   # the wait for the partials inside the launch, a barrier kernel after it
            _l.tp_allreduce_multimem_sync(self._mc, self._peers, self.rank * n, n, self.tokens * self.width, self.rank,
                                          self.world, self._state, exit_rendezvous=False)
            self._h.barrier(channel=1, timeout_ms=self.timeout_ms)
            return self.out
        self._h.barrier(channel=0, timeout_ms=self.timeout_ms)   # every rank's partial is written
        _l.tp_allreduce_multimem(self._mc, self._mc, self.rank * n, n, like=self.out)
        self._h.barrier(channel=1, timeout_ms=self.timeout_ms)   # every rank's rows have been written everywhere
        return self.out

    def captured(self, x):
        key = (x.data_ptr(), tuple(x.shape))
        if self._graph is None or self._graph_key != key:
            self(x)
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                self(x)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    self(x)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self._graph, self._graph_key = graph, key
        self._graph.replay()
        return self.out

    def release(self):
        if self._graph is not None:
            torch.cuda.synchronize()
            self._graph = None


class ColumnShardedGemm:
    """C[:, lo:hi] = A · B[:, lo:hi] on each rank; A replicated; no collective."""

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world

    def bounds(self, n: int):
        return shard_bounds(n, self.rank, self.world)

    def __call__(self, a, b_shard, c_shard):
        _l.matmul[(1,)](a, b_shard, c_shard)
        return c_shard
