"""The read-out executor of seam 2 on the host, the way the reference locks its ring and executor
protocol without a device (bin/runtime/test/test_hmx_spsc_ring_contract.py:36-60): return codes of
configure, publish-before-configure refused, the descriptor surviving publish -> read-out bit for
bit, one read-out call per group in publish order, the full ring answered with a short count and
never with a block, drain as a real barrier, shutdown and rebind."""
import ctypes
import threading
import time

import pytest

from hexagon_mlir_b200._capi import HmxReadoutBatch, HmxReadoutFn


@pytest.fixture()
def ex(hm):
    lib = hm._capi.lib()
    lib.hexagon_runtime_hmx_exec_shutdown()
    yield lib
    lib.hexagon_runtime_hmx_exec_shutdown()


def batch(i, g=4):
    return HmxReadoutBatch(rowStart=4 * i, rowCount=g, validRows=32 - (i % 3), nCroutons=7 + i,
                           ar=0x1000_0000_0000 + 2048 * i, dst=0x2000_0000_0000 + 64 * i)


def fields(b):
    return (b.rowStart, b.rowCount, b.validRows, b.nCroutons, b.ar, b.dst)


def test_configure_return_codes_and_publish_before_configure(ex):
    one = (HmxReadoutBatch * 1)(batch(0))
    assert ex.hexagon_runtime_hmx_exec_publish(one, 1) == 0          # before configure: dropped, not queued
    assert ex.hexagon_runtime_hmx_exec_configure(HmxReadoutFn(), 1) == -1   # null function
    seen = []
    fn = HmxReadoutFn(lambda b, n: seen.append((n, fields(b[0]))))
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 1) == 0
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 0) == 0          # below one thread is clamped to one
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 4) == -2         # one vector thread, whatever was asked for
    assert ex.hexagon_runtime_hmx_exec_publish(one, 1) == 1           # ... and the executor still works
    assert ex.hexagon_runtime_hmx_exec_publish(None, 3) == 0
    assert ex.hexagon_runtime_hmx_exec_publish(one, 0) == 0
    ex.hexagon_runtime_hmx_exec_drain()
    assert seen == [(1, fields(batch(0)))]


def test_descriptors_survive_in_order_one_call_per_group(ex):
    seen = []
    fn = HmxReadoutFn(lambda b, n: seen.append((n, fields(b[0]))))
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 1) == 0
    before = ex.b200mlir_hmx_exec_batches_run()
    sent = []
    for start in range(0, 60, 5):   # more than three turns of the 16-slot ring
        group = [batch(i, g=1 + i % 8) for i in range(start, start + 5)]
        arr = (HmxReadoutBatch * 5)(*group)
        done = 0
        while done < 5:             # a short count is the caller's to handle: offer the tail again
            sub = (HmxReadoutBatch * (5 - done))(*group[done:])
            done += ex.hexagon_runtime_hmx_exec_publish(sub, 5 - done)
        sent += [fields(b) for b in group]
        del arr
    ex.hexagon_runtime_hmx_exec_drain()
    assert [f for _, f in seen] == sent
    assert all(n == 1 for n, _ in seen)
    assert ex.b200mlir_hmx_exec_batches_run() - before == 60


def test_full_ring_returns_short_and_never_blocks(ex):
    gate, entered = threading.Event(), threading.Event()
    seen = []

    def readout(b, n):
        entered.set()
        gate.wait(10)
        seen.append(b[0].rowStart)
    fn = HmxReadoutFn(readout)
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 1) == 0
    first = (HmxReadoutBatch * 1)(batch(0))
    assert ex.hexagon_runtime_hmx_exec_publish(first, 1) == 1
    assert entered.wait(5)          # the read-out thread is inside batch 0 and holds its slot
    many = (HmxReadoutBatch * 40)(*[batch(i) for i in range(1, 41)])
    t0 = time.perf_counter()
    accepted = ex.hexagon_runtime_hmx_exec_publish(many, 40)
    assert time.perf_counter() - t0 < 1.0      # returned while the consumer was stuck: no blocking
    assert accepted == 14                      # 15 usable slots, one still held by batch 0
    assert ex.hexagon_runtime_hmx_exec_publish(many, 40) == 0   # full ring: nothing accepted
    gate.set()
    ex.hexagon_runtime_hmx_exec_drain()
    assert seen == [4 * i for i in range(0, 15)]                # the tail was the caller's to read out


def test_drain_is_a_barrier_and_shutdown_then_rebind(ex):
    marks = []

    def slow(b, n):
        time.sleep(0.02)
        marks.append(b[0].rowStart)
    fn = HmxReadoutFn(slow)
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 1) == 0
    arr = (HmxReadoutBatch * 8)(*[batch(i) for i in range(8)])
    assert ex.hexagon_runtime_hmx_exec_publish(arr, 8) == 8
    ex.hexagon_runtime_hmx_exec_drain()
    assert marks == [4 * i for i in range(8)]   # every effect visible once drain has returned
    ex.hexagon_runtime_hmx_exec_drain()         # nothing outstanding: returns at once
    ex.hexagon_runtime_hmx_exec_shutdown()
    assert ex.hexagon_runtime_hmx_exec_publish(arr, 8) == 0     # after shutdown: refused
    other = []
    fn2 = HmxReadoutFn(lambda b, n: other.append(b[0].nCroutons))
    assert ex.hexagon_runtime_hmx_exec_configure(fn2, 1) == 0   # a new resident thread
    assert ex.hexagon_runtime_hmx_exec_publish(arr, 3) == 3
    ex.hexagon_runtime_hmx_exec_drain()
    assert other == [7, 8, 9] and len(marks) == 8
    # replacing the function waits for the read-out in flight, then the new one takes the next batch
    assert ex.hexagon_runtime_hmx_exec_configure(fn, 1) == 0
    assert ex.hexagon_runtime_hmx_exec_publish(arr, 1) == 1
    ex.hexagon_runtime_hmx_exec_drain()
    assert len(marks) == 9 and ctypes.sizeof(HmxReadoutBatch) == 32
