"""ctypes binding of libawq_b200.so (the C ABI declared in include/awq_b200.h).

There is no fallback: if the shared library is missing the import fails with the
build command, and every wrapper raises AwqBackendError on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# AWQ_B200_LIB selects another build of the library (for comparing two builds in one process tree)
LIB_PATH = os.environ.get("AWQ_B200_LIB") or os.path.join(_HERE, "lib", "libawq_b200.so")

AWQ_OK = 0
AWQ_ERR_INVALID_ARGUMENT = -1
AWQ_ERR_WORKSPACE = -2
AWQ_ERR_CUDA = -3
AWQ_ERR_DEVICE_TIMEOUT = -4
AWQ_ERR_UNSUPPORTED = -5


class AwqBackendError(Exception):
    """Raised for any non-zero status of the C ABI (the counterpart of the reference's
    AirBackendError, python/air/backend/abc.py:52-61)."""

    def __init__(self, message, status=None):
        super().__init__(message)
        self.status = status


# name -> (restype, argtypes); mirrors include/awq_b200.h one to one
_P = c_void_p
SIGNATURES = {
    "awq_b200_version": (c_int, []),
    "awq_b200_last_error": (c_char_p, []),
    "awq_b200_set_decode_kernel": (c_int, [c_int]),
    "awq_b200_set_gemm_kernel": (c_int, [c_int]),
    "awq_b200_set_deterministic": (c_int, [c_int]),
    "awq_b200_set_wait_limit": (c_int, [ctypes.c_longlong]),
    "awq_b200_static_check": (c_int, [_P]),
    "awq_b200_dequant_bf16": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "awq_b200_dequant_1d_bf16": (c_int, [_P, _P, _P, _P, c_int, c_int, _P]),
    "awq_b200_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "awq_b200_workspace_init": (c_int, [_P, c_size_t, _P]),
    "awq_b200_workspace_check": (c_int, [_P, _P]),
    "awq_b200_gemv_bf16": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemv_act": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gateup_swiglu_act": (c_int, [_P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_rmsnorm_act": (c_int, [_P, _P, c_float, _P, c_int, c_int, c_int, _P]),
    "awq_b200_add_rmsnorm_act": (c_int, [_P, _P, _P, c_float, _P, _P, c_int, c_int, c_int, _P]),
    "awq_b200_gemv_bf16_static": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "awq_b200_gemv_f32": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_rmsnorm_bf16": (c_int, [_P, _P, c_float, _P, c_int, c_int, _P]),
    "awq_b200_add_rmsnorm_bf16": (c_int, [_P, _P, _P, c_float, _P, _P, c_int, c_int, _P]),
    "awq_b200_gateup_swiglu_bf16": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_interleave_gate_up": (c_int, [_P] * 9 + [c_int, c_int, c_int, _P]),
    "awq_b200_ffn_decode_bf16": (c_int, [_P, _P, c_float] + [_P] * 10 + [c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemv_f32_push": (c_int, [_P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_tp_reduce_add_rmsnorm_act": (c_int, [_P, _P, _P, c_int, _P, c_float, _P, _P, c_int, c_int, c_int, _P, _P]),
    "awq_b200_set_ffn_stack_tuning": (c_int, [c_int, c_int]),
    "awq_b200_ffn_stack_plan_bytes": (c_size_t, [c_int]),
    "awq_b200_ffn_stack_workspace_bytes": (c_size_t, [c_int]),
    "awq_b200_ffn_stack_tp_slot_bytes": (c_size_t, [c_int, c_int]),
    "awq_b200_ffn_stack_plan": (c_int, [_P, c_size_t, c_int] + [_P] * 7 + [c_int, c_int, c_int]),
    "awq_b200_ffn_stack_decode_bf16": (c_int, [_P, c_int, _P, _P, _P, c_float, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_ffn_stack_decode_tp_bf16": (c_int, [_P, c_int, _P, _P, _P, c_float, c_int, c_int, c_int, c_int, _P, c_size_t,
                                                  c_size_t, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemm_bf16": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "awq_b200_rope_halfsplit_bf16": (c_int, [_P, c_size_t, _P, _P, c_size_t, c_int, c_int, c_int, _P]),
    "awq_b200_linear_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "awq_b200_silu_mul_bf16": (c_int, [_P, _P, _P, c_size_t, _P]),
    "awq_b200_gemm_fused_bf16": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "awq_b200_gemm_check": (c_int, [_P]),
    "awq_b200_gemm_decode_workspace_bytes": (c_size_t, [c_int, c_int]),
    "awq_b200_gemm_decode_f32": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemm_decode_act": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemm_decode_f8_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "awq_b200_gemm_decode_f8": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_gemm_decode_bf16": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "awq_b200_repack_B_to_A": (c_int, [_P] * 6 + [c_int, c_int, c_int, _P]),
    "awq_b200_repack_A_to_B": (c_int, [_P] * 6 + [c_int, c_int, c_int, _P]),
    "awq_b200_repack_C_to_B": (c_int, [_P] * 4 + [c_int, c_int, c_int, c_int, c_int, _P]),
}

_lib = None


def load():
    """Load the shared library once and set the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AwqBackendError(
            f"{LIB_PATH} is missing: build it with `python -m mlir_air_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        if os.environ.get("AWQ_B200_LIB") and not hasattr(lib, name):
            continue  # an older build selected for comparison may lack the newest entry points
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().awq_b200_last_error().decode("utf-8", "replace")


def check(status: int, what: str = ""):
    if status != AWQ_OK:
        raise AwqBackendError(f"{what or 'awq_b200'} failed ({status}): {last_error()}", status)


def call(name: str, *args):
    """Call `name` and raise AwqBackendError unless it returns AWQ_OK."""
    check(getattr(load(), name)(*args), name)
