"""ctypes binding of libprichs_moe.so: one Python function per symbol of include/prichs_moe.h.

The library is built in-tree by `python -m prichs_b200.build`; loading fails loudly when it is missing --
there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# PRICHS_B200_LIB selects another build of the same library for a whole process (the tests run the ragged cases
# against the index-checking build, libprichs_moe_check.so, this way). Read here, on the Python side; the C library
# itself reads no environment variable.
LIB_PATH = os.environ.get("PRICHS_B200_LIB") or os.path.join(_PKG, "libprichs_moe.so")

OK, ERR_BAD_SHAPE, ERR_CAPACITY, ERR_CUDA, ERR_COMM, ERR_TIMEOUT, ERR_BAD_ARG, ERR_BOUNDS = 0, -1, -2, -3, -4, -5, -6, -7
DTYPE_F32, DTYPE_BF16 = 0, 1
MODE_BF16, MODE_F32 = 0, 1


class Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden_dim", "intermediate_dim", "num_experts", "top_k", "max_tokens",
                                       "mode", "device", "ep_world", "ep_rank", "ep_max_recv_rows", "ep_waves",
                                       # tuning (0 = default): see prichs_moe_config_t
                                       "route_kernel", "scan_placement", "separate_prenorm", "gemm_kernel", "pdl",
                                       "host_chunk_tokens", "router_ctas_per_sm", "ep_reserve_sms", "ep_shared_copy_sms",
                                       "ep_combine_mode", "ep_dispatch_kernel", "ep_timeout_ms", "ep_nccl_barriers")]

TUNING_FIELDS = ("route_kernel", "scan_placement", "separate_prenorm", "gemm_kernel", "pdl", "host_chunk_tokens",
                 "router_ctas_per_sm", "ep_reserve_sms", "ep_shared_copy_sms", "ep_combine_mode", "ep_dispatch_kernel", "ep_timeout_ms", "ep_nccl_barriers")


# name -> (restype, argtypes); the full export list of include/prichs_moe.h
_fp = C.POINTER(C.c_float)
SYMBOLS = {
    "prichs_moe_create": (C.c_int, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "prichs_moe_destroy": (C.c_int, [C.c_void_p]),
    "prichs_moe_upload_weights": (C.c_int, [C.c_void_p, C.POINTER(_fp), C.c_int]),
    "prichs_moe_set_bias": (C.c_int, [C.c_void_p, _fp, C.c_int]),
    "prichs_moe_get_bias": (C.c_int, [C.c_void_p, _fp, C.c_int]),
    "prichs_moe_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, _fp, C.c_int, C.c_void_p, C.c_int,
                                     C.c_int, C.c_void_p]),
    "prichs_moe_block_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_float, _fp, C.c_int, C.c_void_p,
                                           C.c_int, C.c_int, C.c_void_p]),
    "prichs_moe_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_void_p),
                                      C.c_int, C.c_void_p]),
    "prichs_moe_block_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_void_p,
                                            C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p]),
    "prichs_moe_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _fp, C.c_int, C.c_void_p, C.c_int]),
    "prichs_moe_sync_status": (C.c_int, [C.c_void_p]),
    "prichs_moe_get_counts": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int]),
    "prichs_moe_get_routing": (C.c_int, [C.c_void_p, _fp, C.POINTER(C.c_int32), _fp, C.c_int]),
    "prichs_moe_update_aux_free_bias": (C.c_int, [C.c_void_p, C.POINTER(C.c_size_t), C.c_int, C.c_size_t, C.c_float]),
    "prichs_moe_update_bias_from_last": (C.c_int, [C.c_void_p, C.c_float, C.c_size_t, C.c_void_p]),
    "prichs_moe_ep_unique_id": (C.c_int, [C.c_void_p]),
    "prichs_moe_ep_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "prichs_moe_ep_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "prichs_ep_wait_or_abort": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "prichs_moe_ep_recv_rows": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
    "prichs_last_error": (C.c_char_p, []),
    "prichs_bounds_checking": (C.c_int, []),
    "prichs_kernel_launches": (C.c_int64, []),
    "prichs_moe_enable_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "prichs_moe_get_stage_ms": (C.c_int, [C.c_void_p, _fp]),
    "prichs_moe_get_ep_timeline": (C.c_int, [C.c_void_p, _fp, C.c_int]),
    "prichs_moe_debug_copy": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_size_t]),
    "prichs_moe_forward_train": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, _fp, C.c_int, C.c_void_p, C.c_int,
                                           C.c_int, C.c_void_p]),
    "prichs_moe_get_stash": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t]),
    "prichs_moe_get_expert_assignments": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t,
                                                    C.POINTER(C.c_size_t)]),
    "prichs_engine_moe_forward_shared": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p,
                                                   C.c_void_p, C.c_void_p]),
    "prichs_engine_moe_routing": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "prichs_engine_moe_forward_expert": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t),
                                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "prichs_engine_moe_finalize_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "prichs_moe_debug_set": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong]),
    "prichs_moe_route_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "launch_moe_gather": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "launch_moe_scatter_add": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                      C.c_void_p]),
    "launch_swiglu_forward": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library with argument types set. Raises if the shared object was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m prichs_b200.build` "
                               "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().prichs_last_error().decode("utf-8", "replace")
