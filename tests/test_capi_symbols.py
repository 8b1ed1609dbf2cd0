"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200mlir_capi.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"B200_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_reference_entry_points():
    names = declared_symbols()
    for must in ["matmul", "klooped_matmul", "softmax_kernel_float16", "softmax_kernel_float32",
                 "rms_norm_fwd_kernel_float16", "rms_norm_fwd_kernel_float32",
                 "silu_kernel_float16", "silu_kernel_float32",
                 "hexagon_runtime_alloc_1d", "hexagon_runtime_free_1d", "hexagon_runtime_copy",
                 "hexagon_runtime_resident_scope_enter_v2", "hexagon_runtime_workspace_resident_v2",
                 "hexagon_runtime_weight_resident_v2", "hexagon_runtime_weight_resident_ddr_v2",
                 "hexagon_runtime_resident_free_v2", "hexagon_runtime_hmx_ensure",
                 "hexagon_runtime_hmx_unlock", "hexagon_runtime_dma_start",
                 "hexagon_runtime_dma2d_start", "hexagon_runtime_dma_wait"]:
        assert must in names, must
    assert len(names) >= 50


def test_library_exports_every_declared_symbol(hm):
    handle = ctypes.CDLL(hm.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(handle, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol(hm):
    from hexagon_mlir_b200 import _capi
    assert sorted(_capi._SIGNATURES) == declared_symbols()


def test_no_torch_types_in_the_abi():
    text = open(os.path.join(ROOT, "include", "b200mlir_capi.h")).read()
    assert "torch" not in text.lower() and "at::" not in text


def test_library_does_not_link_the_oracle(hm):
    import subprocess
    out = subprocess.run(["ldd", hm.LIB_PATH], capture_output=True, text=True).stdout
    assert "oracle" not in out


def test_options_roundtrip_and_unknown_option(hm):
    hm.set_option("rmsNormEpsilon", 1e-6)
    assert hm.get_option("rmsNormEpsilon") == pytest.approx(1e-6)
    hm.set_option("rmsNormEpsilon", 1e-5)
    with pytest.raises(hm.B200Error) as e:
        hm.set_option("noSuchOption", 1)
    assert e.value.code == 2


def test_descriptor_layout_matches_mlir_memref():
    from hexagon_mlir_b200._capi import MemRef1D, MemRef2D
    assert ctypes.sizeof(MemRef1D) == 8 * 5 and ctypes.sizeof(MemRef2D) == 8 * 7
    assert MemRef2D.sizes.offset == 24 and MemRef2D.strides.offset == 40


def test_compute_fails_loudly_without_a_device(hm):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = np.zeros((32, 32), np.float16)
    with pytest.raises(hm.B200Error) as e:
        hm.matmul[(1,)](a, a, a)
    assert e.value.code == 1  # B200MLIR_ERR_NO_DEVICE: no CPU fallback exists


def test_descriptor_contract_errors_before_any_device_work(hm):
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs the no-device path to observe ordering")
    a = np.zeros((32, 32), np.float16)
    with pytest.raises(ValueError):
        hm.matmul[(1,)](a, a, np.zeros(32, np.float16))  # wrong rank
    with pytest.raises(TypeError):
        hm.matmul[(1,)](a, a, a, noSuchOption=1)
    # reference options and constexpr-style extras are accepted
    with pytest.raises(hm.B200Error):
        hm.matmul[(1,)](a, a, a, enableMultiThreading=True, enableVTCMTiling=True, N_ROWS=32)


def test_resident_scope_rules_without_device(hm):
    lib = hm._capi.lib()
    # one immutable scope per process (HexagonCAPI.cpp:132-150 of the reference)
    assert lib.hexagon_runtime_resident_scope_enter_v2(0x1234, 0x5678) == 0
    assert lib.hexagon_runtime_resident_scope_enter_v2(0x1234, 0x5678) == 0
    assert lib.hexagon_runtime_resident_scope_enter_v2(1, 2) == -1
    assert hm._capi.last_error()[0] == 4
    lib.hexagon_runtime_hmx_ensure()
    lib.hexagon_runtime_hmx_unlock()
    # a refused copy start reports through status and the sentinel token
    st = ctypes.c_int(7)
    tok = lib.hexagon_runtime_dma_start(None, 0, None, 0, 16, False, False, ctypes.byref(st))
    assert tok == 0xFFFFFFFF and st.value == -1
    lib.hexagon_runtime_dma_wait(tok)  # returns at once


def test_tensor_parallel_group_state_without_a_group(hm):
    """No group initialised: rank 0 of 1; the collective entries refuse instead of touching NCCL."""
    assert hm.tp_info() == (False, 0, 1)
    hm.tp_shutdown()                     # nothing to shut down: not an error
    with pytest.raises(ValueError):
        hm.tp_init(b"short", 0, 2)       # the id is 128 bytes


def test_block_table_and_leaf_argument_checks_without_a_device(hm):
    import torch
    if torch.cuda.is_available():
        pytest.skip("needs the no-device path")
    lib = hm._capi.lib()
    lib.hexagon_runtime_free_2d(12345)   # not a table returned by alloc_2d: refused, nothing freed
    assert hm._capi.last_error()[0] == 2
    assert lib.hexagon_runtime_alloc_2d(4, 64, 128, False) is None and hm._capi.last_error()[0] == 1   # no device
    lib.hmx_acc_clear_f16()              # a leaf without a device: the library's error, no crash
    assert hm._capi.last_error()[0] == 1


def test_host_gemm_panel_plan(hm):
    """Which host-buffer GEMMs are pipelined, and how they are cut: panel edges on multiples of
    256, at most 16 panels each way, the panels cover the problem, row and column panels counted
    separately (the per-rank column blocks of the headline GEMM at 1, 2, 4 and 8 ranks)."""
    assert hm.host_gemm_plan(1024, 1024, 1024) is None           # small: staged whole
    assert hm.host_gemm_plan(16384, 512, 8192) is None           # a block narrower than a panel
    assert hm.host_gemm_plan(4096, 4100, 4096) is None           # N not a multiple of 8
    for world in (1, 2, 4, 8):
        plan = hm.host_gemm_plan(16384, 16384 // world, 8192)
        assert plan["row_panels"] == 16 and plan["panel_rows"] == 1024
        assert plan["col_panels"] == min(16, 16 // world) and plan["panel_cols"] == 1024
    for m, n, k in ((4360, 4104, 4096), (12288, 1280, 4096), (1280, 9000, 4096), (9000, 2048, 4096), (100000, 1024, 512)):
        plan = hm.host_gemm_plan(m, n, k)
        assert plan["panel_rows"] % 256 == 0 and plan["panel_cols"] % 256 == 0
        assert 1 <= plan["row_panels"] <= 16 and 1 <= plan["col_panels"] <= 16
        assert (plan["row_panels"] - 1) * plan["panel_rows"] < m <= plan["row_panels"] * plan["panel_rows"]
        assert (plan["col_panels"] - 1) * plan["panel_cols"] < n <= plan["col_panels"] * plan["panel_cols"]
