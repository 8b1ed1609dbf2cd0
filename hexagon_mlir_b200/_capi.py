"""ctypes binding of libb200mlir.so (the C ABI declared in include/b200mlir_capi.h).

The library is the product; this module only loads it and builds memref
descriptors.  There is no fallback: if the shared library is missing, loading
raises, and on a machine without a usable sm_100 device every compute call
fails with the library's own error.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200MLIR_LIB names another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("B200MLIR_LIB") or os.path.join(_HERE, "libb200mlir.so")

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_void_p = ctypes.c_void_p


class MemRef1D(ctypes.Structure):
    """MemRefDescriptor<T,1> (test/utils/dsp/include/common.h:15-27 of the reference)."""
    _fields_ = [("allocated", c_void_p), ("aligned", c_void_p), ("offset", c_i64),
                ("sizes", c_i64 * 1), ("strides", c_i64 * 1)]


class MemRef2D(ctypes.Structure):
    _fields_ = [("allocated", c_void_p), ("aligned", c_void_p), ("offset", c_i64),
                ("sizes", c_i64 * 2), ("strides", c_i64 * 2)]


class MemRef4D(ctypes.Structure):
    _fields_ = [("allocated", c_void_p), ("aligned", c_void_p), ("offset", c_i64),
                ("sizes", c_i64 * 4), ("strides", c_i64 * 4)]


class HmxReadoutBatch(ctypes.Structure):
    """HmxReadoutBatch (bin/runtime/include/HmxVectorExecutor.h:103-110 of the reference), 64-bit pointers."""
    _fields_ = [("rowStart", ctypes.c_uint32), ("rowCount", ctypes.c_uint32), ("validRows", ctypes.c_uint32),
                ("nCroutons", ctypes.c_uint32), ("ar", c_void_p), ("dst", c_void_p)]


HmxReadoutFn = ctypes.CFUNCTYPE(None, ctypes.POINTER(HmxReadoutBatch), ctypes.c_uint32)


class B200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200mlir error {code}: {message}")
        self.code = code
        self.message = message


_lib = None

_GRID = [c_int] * 6
_M2 = ctypes.POINTER(MemRef2D)
_M1 = ctypes.POINTER(MemRef1D)
_M4 = ctypes.POINTER(MemRef4D)

_SIGNATURES = {
    "b200mlir_init": (c_int, [c_int]),
    "b200mlir_set_stream": (c_int, [c_void_p]),
    "b200mlir_synchronize": (c_int, []),
    "b200mlir_last_error": (c_int, [ctypes.c_char_p, c_int]),
    "b200mlir_version": (ctypes.c_char_p, []),
    "b200mlir_launch_count": (c_i64, []),
    "b200mlir_reset_launch_count": (None, []),
    "b200mlir_device_status": (c_int, []),
    "b200mlir_set_option": (c_int, [ctypes.c_char_p, ctypes.c_double]),
    "b200mlir_get_option": (c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_double)]),
    "matmul": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M2] + _GRID),
    "klooped_matmul": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M2] + _GRID),
    "multispan_matmul": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M2] + _GRID),
    "matmul_f32out": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M2, c_i64, _M2] + _GRID),
    "matmul_i8": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M2] + _GRID),
    "attention_fwd_kernel_float16": (None, [c_i64, _M4] * 4 + [ctypes.c_float] + _GRID),
    "attention_fwd_kernel_float32": (None, [c_i64, _M4] * 4 + [ctypes.c_float] + _GRID),
    "online_softmax": (None, [c_i64, _M2, c_i64, _M2] + _GRID),
    "softmax_kernel_float16": (None, [c_i64, _M2, c_i64, _M2] + _GRID),
    "softmax_kernel_float32": (None, [c_i64, _M2, c_i64, _M2] + _GRID),
    "rms_norm_fwd_kernel_float16": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M1] + _GRID),
    "rms_norm_fwd_kernel_float32": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M1] + _GRID),
    "silu_kernel_float16": (None, [c_i64, _M1, c_i64, _M1] + _GRID),
    "silu_kernel_float32": (None, [c_i64, _M1, c_i64, _M1] + _GRID),
    "add_kernel_float16": (None, [c_i64, _M1, c_i64, _M1, c_i64, _M1] + _GRID),
    "swiglu_kernel_float16": (None, [c_i64, _M1, c_i64, _M1, c_i64, _M1] + _GRID),
    "w8a16_matmul": (None, [c_i64, _M2, c_i64, _M2, c_i64, _M1, c_i64, _M2] + _GRID),
    "mlp_block_float16": (None, [c_i64, _M2, c_i64, _M1, c_i64, _M2, c_i64, _M2, c_i64, _M2,
                                 c_i64, _M2, ctypes.c_float, c_int] + _GRID),
    "mlp_block_push_float16": (None, [c_i64, _M2, c_i64, _M1, c_i64, _M2, c_i64, _M2, c_i64, _M2,
                                      ctypes.POINTER(c_void_p), c_int, c_int, ctypes.c_float] + _GRID),
    "b200mlir_tp_unique_id": (c_int, [c_void_p]),
    "b200mlir_tp_init": (c_int, [c_void_p, c_int, c_int]),
    "b200mlir_tp_info": (c_int, [ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "b200mlir_tp_slab_exchange_mode": (c_int, []),
    "b200mlir_host_gemm_plan": (c_int, [c_i64, c_i64, c_i64, ctypes.POINTER(c_i64)]),
    "b200mlir_tp_shutdown": (c_int, []),
    "b200mlir_tp_all_reduce_float16": (c_int, [c_void_p, c_i64]),
    "mlp_block_tp_float16": (None, [c_i64, _M2, c_i64, _M1, c_i64, _M2, c_i64, _M2, c_i64, _M2,
                                    c_i64, _M2, ctypes.c_float, c_int] + _GRID),
    "mlp_block_tp_multicast_float16": (None, [c_i64, _M2, c_i64, _M1, c_i64, _M2, c_i64, _M2, c_i64, _M2,
                                              c_i64, _M2, c_void_p, ctypes.POINTER(c_void_p), c_i64, c_void_p, c_int,
                                              c_int, ctypes.c_float, c_int] + _GRID),
    "b200mlir_tp_allreduce_multimem_float16": (c_int, [c_void_p, c_void_p, c_i64, c_i64]),
    "b200mlir_tp_barrier": (c_int, [ctypes.POINTER(c_void_p), c_i64, c_int, c_int, c_int, c_void_p]),
    "b200mlir_tp_allreduce_multimem_sync_float16": (c_int, [c_void_p, ctypes.POINTER(c_void_p), c_i64, c_i64, c_i64,
                                                            c_int, c_int, c_void_p, c_int]),
    "b200mlir_mlp_phase_times": (c_int, [ctypes.POINTER(ctypes.c_double), c_int]),
    "b200mlir_tp_reduce_rows_float16": (c_int, [c_void_p, c_void_p, c_i64, ctypes.POINTER(c_void_p), c_int, c_int,
                                                c_i64, c_i64]),
    "hexagon_runtime_alloc_1d": (c_void_p, [ctypes.c_size_t, ctypes.c_uint64, ctypes.c_bool]),
    "hexagon_runtime_free_1d": (None, [c_void_p]),
    "hexagon_runtime_alloc_2d": (c_void_p, [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_uint64,
                                            ctypes.c_bool]),
    "hexagon_runtime_free_2d": (None, [c_void_p]),
    "hexagon_runtime_copy": (None, [c_void_p, c_void_p, ctypes.c_size_t, ctypes.c_bool,
                                    ctypes.c_bool]),
    "hexagon_runtime_build_crouton": (c_void_p, [c_void_p, ctypes.c_size_t]),
    "hexagon_runtime_get_contiguous_memref": (c_void_p, [c_void_p]),
    "hexagon_runtime_resident_scope_enter_v2": (ctypes.c_int32, [ctypes.c_uint64, ctypes.c_uint64]),
    "hexagon_runtime_workspace_resident_v2": (c_void_p, [ctypes.c_uint64, ctypes.c_uint32,
                                                         ctypes.c_uint32, ctypes.c_uint32]),
    "hexagon_runtime_weight_resident_v2": (c_void_p, [ctypes.c_uint64, ctypes.c_uint32,
                                                      ctypes.c_uint32]),
    "hexagon_runtime_weight_resident_ddr_v2": (c_void_p, [ctypes.c_uint64, ctypes.c_uint32,
                                                          ctypes.c_uint32]),
    "hexagon_runtime_resident_free_v2": (ctypes.c_int32, [c_void_p, ctypes.c_uint32]),
    "hexagon_runtime_hmx_ensure": (None, []),
    "hexagon_runtime_hmx_unlock": (None, []),
    "hmx_bias_init_unit_f16": (None, [c_void_p]),
    "hmx_bias_load_f16": (None, [c_void_p, ctypes.c_uint]),
    "hmx_acc_clear_f16": (None, []),
    "hmx_acc_store_f16": (None, [c_void_p, ctypes.c_uint]),
    "hmx_mma_f16": (None, [c_void_p, c_void_p, ctypes.c_uint]),
    "hmx_pack_act_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_act_f16_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f16_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_act_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_act_f32_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f32_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f16_T": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f16_T_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f32_T": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_f32_T_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_act_tail_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_tail_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_act_tail_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_tail_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_tail_f16_T": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_pack_weight_tail_f32_T": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_f16_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_f32_bulk": (None, [c_void_p, c_void_p, ctypes.c_uint, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_tail_f16": (None, [c_void_p, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hmx_unpack_acc_tail_f32": (None, [c_void_p, c_void_p, ctypes.c_uint, c_void_p, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "hexagon_runtime_hmx_exec_configure": (ctypes.c_int32, [HmxReadoutFn, ctypes.c_int32]),
    "hexagon_runtime_hmx_exec_publish": (ctypes.c_uint32, [ctypes.POINTER(HmxReadoutBatch), ctypes.c_uint32]),
    "hexagon_runtime_hmx_exec_drain": (None, []),
    "hexagon_runtime_hmx_exec_shutdown": (None, []),
    "b200mlir_hmx_exec_batches_run": (ctypes.c_uint64, []),
    "hexagon_runtime_dma_start": (ctypes.c_uint32, [c_void_p, c_int, c_void_p, c_int,
                                                    ctypes.c_uint32, ctypes.c_bool, ctypes.c_bool,
                                                    ctypes.POINTER(c_int)]),
    "hexagon_runtime_dma2d_start": (ctypes.c_uint32, [c_void_p, c_int, c_void_p, c_int,
                                                      ctypes.c_uint32, ctypes.c_uint32,
                                                      ctypes.c_uint32, ctypes.c_uint32,
                                                      ctypes.c_bool, ctypes.c_bool, ctypes.c_bool,
                                                      ctypes.c_uint32, ctypes.POINTER(c_int)]),
    "hexagon_runtime_dma_wait": (None, [ctypes.c_uint32]),
    "b200mlir_w8a16_register_weight": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_int]),
    "b200mlir_w8a16_unregister_weight": (c_int, [c_void_p]),
    "b200mlir_w8a16_matmul_static_scratch": (c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_void_p, c_i64,
                                                     c_i64, c_i64, c_i64, c_void_p]),
    "b200mlir_pack_weight_f16": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64]),
    "b200mlir_pack_act_f16": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64]),
    "b200mlir_unpack_acc_f16": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64]),
    "b200mlir_gemm_variant_count": (c_int, []),
    "b200mlir_gemm_variant_info": (c_int, [c_int, ctypes.c_char_p, c_int]),
    "b200mlir_gemm_variant_verdict": (c_int, [c_int, c_i64, c_i64, c_i64, ctypes.c_char_p, c_int]),
    "b200mlir_gemm_explain": (c_int, [c_i64, c_i64, c_i64, ctypes.c_char_p, c_int]),
    "b200mlir_gemm_autotune": (c_int, [c_i64, c_i64, c_i64, ctypes.c_char_p, c_int]),
    "b200mlir_gemm_search_scripted": (c_int, [c_i64, c_i64, c_i64,
                                              ctypes.POINTER(ctypes.c_double), c_int, c_int,
                                              ctypes.POINTER(ctypes.c_double), ctypes.c_double,
                                              ctypes.c_char_p, c_int]),
    "b200mlir_autotune_cache_load": (c_int, [ctypes.c_char_p]),
    "b200mlir_autotune_cache_save": (c_int, [ctypes.c_char_p]),
    "b200mlir_autotune_cache_clear": (None, []),
    "b200mlir_benchmark": (c_int, [ctypes.CFUNCTYPE(None, c_void_p), c_void_p, c_int,
                                   ctypes.POINTER(ctypes.c_double)]),
    "b200mlir_benchmark_report": (c_int, [ctypes.CFUNCTYPE(None, c_void_p), c_void_p, c_int, ctypes.c_char_p,
                                          ctypes.c_char_p, ctypes.POINTER(ctypes.c_double),
                                          ctypes.POINTER(ctypes.c_longlong)]),
    "b200mlir_perf_report_save": (c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_double, ctypes.c_char_p,
                                          c_int, ctypes.c_longlong]),
    "b200mlir_fill_random": (c_int, [c_void_p, ctypes.c_int32, c_i64, ctypes.c_uint64, c_int, ctypes.c_double,
                                     ctypes.c_double]),
    "b200mlir_selftest_bounded_wait": (c_int, [c_int]),
    "b200mlir_dtype_size": (c_int, [ctypes.c_int32]),
    "b200mlir_tensor_dump": (c_int, [ctypes.c_char_p, ctypes.c_int32, c_i64, ctypes.POINTER(c_i64), c_void_p]),
    "b200mlir_tensor_file_info": (c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(c_i64),
                                          ctypes.POINTER(c_i64), ctypes.POINTER(c_i64)]),
    "b200mlir_tensor_load": (c_int, [ctypes.c_char_p, c_int, c_void_p, c_i64]),
    "b200mlir_manifest_json": (c_int, [ctypes.c_char_p, c_int]),
    "b200mlir_manifest_reset": (None, []),
}


def lib() -> ctypes.CDLL:
    """Load libb200mlir.so; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m hexagon_mlir_b200.build` "
                "(there is no CPU or PyTorch fallback for this library)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error():
    buf = ctypes.create_string_buffer(1024)
    code = lib().b200mlir_last_error(buf, 1024)
    return code, buf.value.decode(errors="replace")


def check() -> None:
    """Raise B200Error if the most recent call on this thread failed."""
    code, msg = last_error()
    if code != 0:
        raise B200Error(code, msg)
