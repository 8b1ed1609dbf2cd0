"""Seam-2 behaviours on the device that hosts compiled against the reference rely on: the
indirect-tensor allocation returning a table of block pointers, 2 KiB alignment from the plain
allocator, a copy ring that reclaims finished descriptors and never refuses a start, one device
per process, a stream per host thread, and the L2 persistence window of a resident weight."""
import ctypes
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_alloc_2d_returns_a_table_of_block_pointers(hm, cuda):
    """bin/runtime/src/HexagonCAPI.cpp:89-94, src/HexagonBuffer.cpp:89-113: one allocation, blocks at
    a stride of the block size rounded up to the alignment, and the return value is the TABLE."""
    lib = hm._capi.lib()
    hm.init(0)
    n, blk, align = 5, 3000, 2048
    tab = lib.hexagon_runtime_alloc_2d(n, blk, align, True)
    assert tab
    ptrs = (ctypes.c_void_p * n).from_address(tab)          # host code indexes the table directly
    addrs = [int(p) for p in ptrs]
    stride = (blk + align - 1) // align * align
    assert all(a % align == 0 for a in addrs)
    assert [a - addrs[0] for a in addrs] == [i * stride for i in range(n)]
    # the blocks are device memory: fill each through the runtime's copy and read back
    for i, a in enumerate(addrs):
        src = np.full(blk, i + 1, np.uint8)
        lib.hexagon_runtime_copy(a, src.ctypes.data, blk, True, False)
    for i, a in enumerate(addrs):
        back = np.zeros(blk, np.uint8)
        lib.hexagon_runtime_copy(back.ctypes.data, a, blk, False, True)
        assert (back == i + 1).all()
    # a kernel reads the same table (pinned host memory mapped into the device's address space)
    t = cuda.zeros(n, dtype=cuda.int64, device="cuda")
    lib.hexagon_runtime_copy(t.data_ptr(), tab, 8 * n, True, False)
    assert t.cpu().tolist() == addrs
    lib.hexagon_runtime_free_2d(tab)
    assert hm._capi.last_error()[0] == 0
    lib.hexagon_runtime_free_2d(tab)                          # not a live table any more: refused, no crash
    assert hm._capi.last_error()[0] == 2
    assert lib.hexagon_runtime_alloc_2d(0, 64, 128, False) is None
    assert lib.hexagon_runtime_alloc_2d(4, 64, 4096, False) is None


def test_alloc_1d_serves_tile_alignment(hm):
    """The lowering keeps the requested alignment on every on-chip allocation and tile buffers ask
    for 2048 (HexagonMemToLLVMPass.cpp:538-542)."""
    lib = hm._capi.lib()
    hm.init(0)
    held = []
    for align in (128, 256, 512, 1024, 2048):
        for _ in range(3):
            p = lib.hexagon_runtime_alloc_1d(2048 * 3 + 17, align, True)
            assert p and p % align == 0
            held.append(p)
    src = np.arange(2048, dtype=np.uint8)
    back = np.zeros_like(src)
    lib.hexagon_runtime_copy(held[-1], src.ctypes.data, 2048, True, False)
    lib.hexagon_runtime_copy(back.ctypes.data, held[-1], 2048, False, True)
    assert np.array_equal(src, back)
    for p in held:
        lib.hexagon_runtime_free_1d(p)
        assert hm._capi.last_error()[0] == 0
    assert lib.hexagon_runtime_alloc_1d(64, 4096, True) is None and hm._capi.last_error()[0] == 2
    assert lib.hexagon_runtime_alloc_1d(64, 96, True) is None


def test_copy_ring_reclaims_finished_descriptors(hm):
    """300 starts, a wait on the last token only: legal in the reference, whose ring reclaims every
    descriptor no longer in flight and blocks when full (bin/runtime/UserDMA/RingBuffer.h:103-116);
    no start may be refused."""
    lib = hm._capi.lib()
    hm.init(0)
    src = np.arange(300 * 64, dtype=np.uint8).reshape(300, 64)
    dst = np.zeros_like(src)
    st = ctypes.c_int(9)
    tok = 0
    for i in range(300):
        tok = lib.hexagon_runtime_dma_start(src[i].ctypes.data, 0, dst[i].ctypes.data, 0, 64, False, False,
                                            ctypes.byref(st))
        assert tok != 0xFFFFFFFF and st.value == 0, i
    lib.hexagon_runtime_dma_wait(tok)
    assert np.array_equal(src, dst)
    lib.hexagon_runtime_dma_wait(tok)        # retired tokens: nothing to wait for
    lib.hexagon_runtime_dma_wait(3)


def test_one_device_per_process(hm):
    hm.init(0)
    hm.init(0)                                # the same device again is fine
    with pytest.raises(hm.B200Error) as e:
        hm.init(1)                            # refused even when a second GPU exists
    assert e.value.code == 2 and "one device per process" in e.value.message


def test_each_host_thread_has_its_own_stream(hm, oracle, cuda):
    """Two host threads launch on their own streams at once; neither sees the other's stream, and
    both results are right."""
    rng = np.random.Generator(np.random.Philox(8))
    a = [cuda.from_numpy(rng.uniform(-1, 1, (512, 768)).astype(np.float16)).cuda() for _ in range(2)]
    b = [cuda.from_numpy(rng.uniform(-1, 1, (768, 640)).astype(np.float16)).cuda() for _ in range(2)]
    c = [cuda.zeros((512, 640), dtype=cuda.float16, device="cuda") for _ in range(2)]
    streams = [cuda.cuda.Stream() for _ in range(2)]
    cuda.cuda.synchronize()
    errors = []

    def work(i):
        try:
            with cuda.cuda.stream(streams[i]):
                for _ in range(20):
                    hm.matmul[(1,)](a[i], b[i], c[i])   # binds this thread's stream, then launches on it
                streams[i].synchronize()
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)
    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    cuda.cuda.synchronize()
    for i in range(2):
        want = oracle.gemm_f16(a[i].cpu().numpy(), b[i].cpu().numpy()).astype(np.float32)
        assert np.abs(c[i].cpu().numpy().astype(np.float32) - want).max() / np.abs(want).max() <= 1e-2
    assert hm.device_status() == 0


def test_l2_persistence_window_for_a_resident_weight(hm, oracle, cuda):
    """A weight registered with l2_persist=1 (the decode case of weight residency,
    backend/hexagon_options.py:94-101): results unchanged, the window follows a change of stream,
    and unregistering the weight takes it away."""
    rng = np.random.Generator(np.random.Philox(2))
    k, n = 4096, 2048
    wq = cuda.from_numpy(rng.integers(-127, 128, (k, n), dtype=np.int8)).cuda()
    s = cuda.from_numpy(rng.uniform(0.001, 0.02, n).astype(np.float16)).cuda()
    a = cuda.from_numpy(rng.normal(0, 1, (16, k)).astype(np.float16)).cuda()
    want = oracle.w8a16(a.cpu().numpy(), wq.cpu().numpy(), s.cpu().numpy()).astype(np.float32)
    hm.register_w8a16_weight(wq, s, l2_persist=True)
    try:
        outs = []
        for stream in (cuda.cuda.current_stream(), cuda.cuda.Stream(), cuda.cuda.Stream()):
            with cuda.cuda.stream(stream):
                c = cuda.zeros((16, n), dtype=cuda.float16, device="cuda")
                for _ in range(3):
                    hm.w8a16_matmul[(1,)](a, wq, s, c)
                stream.synchronize()
                outs.append(c)
        for c in outs:
            got = c.cpu().numpy().astype(np.float32)
            assert np.abs(got - want).max() / np.abs(want).max() <= 1e-2
            assert cuda.equal(c, outs[0])
    finally:
        hm.unregister_w8a16_weight(wq)
    assert hm.device_status() == 0
