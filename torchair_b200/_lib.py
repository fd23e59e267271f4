"""ctypes binding of libtorchair_b200.so (the C ABI declared in include/tab_api.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.  ctypes drops
the GIL around every call, as the reference does around its native run
(torchair/core/torchair.cpp:253).
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER

_P = c_void_p
_I = c_int
_L = c_int64

# name -> argument types (return type is int unless listed in _RESTYPE)
SIGNATURES = {
    "tab_version": [],
    "tab_last_error": [],
    "tab_launch_count": [],
    "tab_dynamic_quant": [_P, _I, _P, _L, _L, _P, _P, _P],
    "tab_swiglu": [_P, _I, _L, _L, _P, _P],
    "tab_dequant_swiglu_quant": [_P, _P, _L, _P, _P, _L, _I, _L, _L, _P, _P, _P],
    "tab_moe_init_routing_workspace_bytes": [_L, _L, _L, POINTER(c_size_t)],
    "tab_moe_init_routing": [_P, _I, _P, _P, _L, _L, _L, _L, _L, _P, _P, _P, _P, c_size_t, _P],
    "tab_moe_init_routing_static": [_P, _I, _P, _P, _L, _L, _L, _L, _L, _P, _P, _P, _P],
    "tab_moe_dispatch_pack_workspace_bytes": [_L, _L, _L, POINTER(c_size_t)],
    "tab_moe_dispatch_pack": [_P, _I, _P, _L, _L, _L, _L, _I, _P, _P, _P, _P, _P, _I, _P, c_size_t, _P],
    "tab_moe_exchange_plan": [_P, _L, _L, _L, _I, _P, _P, _P, _P],
    "tab_moe_exchange_rows": [_P, _P, _P, _L, _L, _L, _I, _L, _L, _I, _P, _P, _P],
    "tab_moe_compute_expert_tokens": [_P, _L, _L, _P, _P],
    "tab_moe_gating_top_k_softmax": [_P, _I, _P, _L, _L, _L, _P, _P, _P, _P],
    "tab_moe_gating_top_k": [_P, _P, _P, _I, _L, _L, _L, _L, _L, _I, _I, c_float, c_float, _P, _P, _P, _P],
    "tab_moe_finalize_routing": [_P, _I, _P, _P, _P, _P, _P, _P, _L, _L, _L, _P, _P],
    "tab_moe_init_routing_v2": [_P, _I, _P, _L, _L, _L, _L, _L, _I, _I, _I, _L, _P, _L, _P, _P, _P, _P, _P, c_size_t, _P],
    "tab_moe_dispatch_pack_ex": [_P, _I, _P, _L, _L, _L, _L, _L, _I, _P, _P, _L, _P, _L, _I, _P, _P, _P, _P, _P, _I, _P, c_size_t, _P],
    "tab_ep_signal": [_P, _P, _L, _P],
    "tab_ep_wait": [_P, _P, _L, _I, _P, _I, _P],
    "tab_ep_send_rows": [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _I, _P, _P, _I, _P],
    "tab_ep_signal_wait": [_P, _P, _P, _P, _L, _P, _I, _P, _P],
    "tab_ep_unpack_rows_fused": [_P, _P, _L, _L, _L, _L, _L, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "tab_ep_return_plan_fused": [_P, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P, _I, _P],
    "tab_ep_unpack_rows": [_P, _P, _L, _L, _L, _L, _I, _P, _P, _P],
    "tab_ep_return_rows": [_P, _P, _L, _L, _L, _L, _L, _L, _P, _P],
    "tab_ep_return_plan": [_P, _L, _L, _L, _L, _L, _L, _P, _P, _P],
    "tab_moe_combine": [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P],
    "tab_moe_combine_ex": [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P, _P, _L, _L, _L, _L, _P, _P, _P, _P, _P],
    "tab_moe_combine_ack": [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P, _P, _L, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _L, _P],
    "tab_prepack_weight_i8": [_P, _L, _L, _L, _P, _P],
    "tab_grouped_matmul_w8a8": [_P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _I, _P, _L, _P],
    "tab_grouped_matmul_w8a8_scatter": [_P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _I, _P, _L, _P],
    "tab_grouped_matmul_swiglu_quant_workspace_bytes": [_L, _L, POINTER(c_size_t)],
    "tab_grouped_matmul_swiglu_quant": [_P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _I, _P, _P, _P, c_size_t, _L, _P],
    "tab_grouped_matmul_finalize_routing_workspace_bytes": [_L, _L, POINTER(c_size_t)],
    "tab_grouped_matmul_finalize_routing": [_P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _L, _P, _L, c_float, _L, _P, _P, _I, _L, _P, _P,
                                            c_size_t, _L, _P],
    "tab_gmm_status": [POINTER(c_int), _P],
    "tab_gmm_status_reset": [_P],
    "tab_routing_status": [POINTER(c_int), _P],
    "tab_quant_status": [POINTER(c_int), _P],
    "tab_selftest_reciprocal": [_I, _P, _P],
}
_RESTYPE = {"tab_last_error": c_char_p, "tab_launch_count": ctypes.c_longlong}

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libtorchair_b200.so")
_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once and types every exported entry point."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m torchair_b200._build` "
                    "(needs nvcc); torchair_b200 has no fallback implementation")
            lib = ctypes.CDLL(LIB_PATH)
            for name, argtypes in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = _RESTYPE.get(name, c_int)
            _lib = lib
    return _lib


def last_error() -> str:
    msg = load().tab_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def call(name: str, *args) -> None:
    """Calls an int-returning entry point; raises RuntimeError with the library's message on failure."""
    rc = getattr(load(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {last_error()}")


def launch_count() -> int:
    """Kernels enqueued by the library so far in this process (launches recorded during a CUDA-graph capture count once)."""
    return int(load().tab_launch_count())


def workspace_bytes(name: str, *dims: int) -> int:
    out = c_size_t(0)
    call(name, *dims, ctypes.byref(out))
    return int(out.value)
