"""ctypes binding of libmcop_b200.so: the C ABI of include/mcop_b200.h, usable without torch.

`load()` returns the library with argument and result types set for every exported entry point.
Pointers are plain integers (e.g. `tensor.data_ptr()`); the stream is a `cudaStream_t` value (0 = default).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libmcop_b200.so")

P, I64, I32, F32, SZ = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes): mirrors include/mcop_b200.h declaration by declaration
SIGNATURES = {
    "mcop_version": (I32, []),
    "mcop_last_error": (C.c_char_p, []),
    "mcop_device_error": (I32, []),
    "mcop_fused_add_rmsnorm": (I32, [P, I64, P, P, I64, I64, F32, I32, P]),
    "mcop_add_rmsnorm_quant_i8": (I32, [P, P, P, I64, P, P, P, I64, I64, F32, I32, P]),
    "mcop_rmsnorm_smooth_quant_i8": (I32, [P, P, P, P, P, P, P, P, I64, I64, F32, I32, I32, P]),
    "mcop_rmsnorm": (I32, [P, P, P, P, P, I64, I64, F32, I32, I32, I32, P]),
    "mcop_head_rmsnorm": (I32, [P, P, P, I64, I64, I64, F32, I32, I32, I32, I32, P]),
    "mcop_scale_dynamic_quant_i8": (I32, [P, P, P, P, I64, I64, I32, P]),
    "mcop_dynamic_scaled_int8_quant": (I32, [P, P, P, I64, I64, I32, P]),
    "mcop_selftest_wait_timeout": (I32, [I32, P]),
    "mcop_rope_inplace": (I32, [P, P, P, P, I32, I64, I64, I32, I32, I32, I32, I64, I64, I64, I32, I32, P]),
    "mcop_rope_kv_copy": (I32, [P, P, P, P, P, I64, P, P, P, I64, I64, I64, I32, I32, I32, I64, I64, I64, I32, P]),
    "mcop_rope_packed": (I32, [P, P, P, P, I64, P, P, I32, I64, I32, I32, I32, I32, P]),
    "mcop_fused_rope_fwd": (I32, [P, P, P, I64, P, I64, I32, I32, I32, I32, I32, P]),
    "mcop_fused_rope_bwd": (I32, [P, P, P, I64, P, I64, I32, I32, I32, I32, I32, P]),
    "mcop_kv_store_i8": (I32, [P, I64, I64, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, I64, P, P, I32, I64, I32, I32, I32, I32, P]),
    "mcop_reshape_and_cache_flash": (I32, [P, P, I64, I64, P, P, I64, I64, I64, P, I64, I32, I32, I32, I64, I32, P]),
    "mcop_reshape_and_cache": (I32, [P, P, I64, I64, P, P, P, I64, I32, I32, I32, I32, I64, I32, P]),
    "mcop_rope_kv_store_i8_paged": (I32, [P, P, P, P, P, I32, I64, P, P, P, P, P, I64, I32, I32, I32, I32, I64, I64, I64, I32, I64, I32, I32, P]),
    "mcop_moe_softmax_topk": (I32, [P, P, P, I64, I32, I32, P]),
    "mcop_grouped_topk": (I32, [P, P, P, P, I64, I32, I32, I32, I32, I32, C.c_double, I32, I32, I32, P]),
    "mcop_topk_softmax": (I32, [P, P, P, P, I64, I32, I32, I32, I32, P]),
    "mcop_moe_gate_grouped_sigmoid": (I32, [P, P, P, P, P, I64, I32, I32, I32, I32, I32, F32, I32, I32, I32, I32, P]),
    "mcop_moe_gate_grouped_sigmoid_shared": (I32, [P, P, P, P, I64, I32, I32, I32, I32, I32, I32, C.c_double, I32, P]),
    "mcop_moe_scatter_workspace_bytes": (SZ, [I64, I32, I32]),
    "mcop_moe_scatter_quant_i8": (I32, [P, P, P, P, P, P, P, P, P, P, I64, I64, I32, I32, P, SZ, P]),
    "mcop_moe_gather_workspace_bytes": (SZ, [I64, I64]),
    "mcop_moe_sum": (I32, [P, P, I64, I32, I64, I32, P]),
    "mcop_moe_sum_reduce": (I32, [P, P, I64, I32, I64, C.c_double, I32, P]),
    "mcop_moe_align_block_size_workspace_bytes": (SZ, [I64, I32]),
    "mcop_moe_align_block_size": (I32, [P, I64, I32, I32, P, I64, P, I64, P, P, P, SZ, P]),
    "mcop_moe_gather": (I32, [P, P, P, P, I32, I64, I64, I64, P, SZ, P]),
    "mcop_moe_gather_weighted": (I32, [P, P, P, P, P, P, P, I32, I64, I64, I64, I32, I32, P, SZ, P]),
    "mcop_moe_swiglu_quant_i8": (I32, [P, P, P, P, P, P, I64, I64, I32, P]),
    "mcop_add_rmsnorm_quant_i8_norm_out": (I32, [P, P, P, P, I64, P, P, P, I64, I64, F32, I32, P]),
    "mcop_add_rmsnorm_quant_i8_padded": (I32, [P, P, P, P, P, P, P, I64, I64, I64, F32, I32, I32, P]),
    "mcop_silu_mul_quant_i8": (I32, [P, I32, P, I32, I64, I64, P, P, I64, I64, P]),
    "mcop_silu_mul_quant_i8_masked_pack": (I32, [P, I32, P, I32, P, I64, I64, I64, I64, P]),
    "mcop_moe_gather_noalloc": (I32, [P, P, P, I64, I64, I64, P]),
}

GATHER_NOALLOC_SCRATCH_BYTES = 4 << 20

F32_CODE, BF16_CODE, F16_CODE = 0, 1, 2
# codes of mcop_device_error()
DEVERR_POSITION, DEVERR_SLOT, DEVERR_KV_INDEX, DEVERR_SELFTEST = 16, 17, 18, 99

_lib = None


def load(path: str | None = None):
    """Load libmcop_b200.so (raises OSError if it has not been built; there is no fallback)."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    lib = C.CDLL(path or LIBRARY_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


def last_error(lib=None) -> str:
    return (lib or load()).mcop_last_error().decode()


def check(rc: int, lib=None):
    if rc != 0:
        raise RuntimeError(f"mcop_b200 error {rc}: {last_error(lib)}")
