"""ctypes binding of the C ABI declared in ``include/rmn_b200.h``.

Thin by design: argument marshalling and status -> exception translation
only. There is no CPU fallback; if the shared library has not been built the
import of :func:`lib` fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

from . import _build

OK, ERR_BAD_ARG, ERR_ALLOC, ERR_PROBE_LIMIT, ERR_TIMEOUT, ERR_CUDA, ERR_RANGE, ERR_UNSUPPORTED, ERR_TOO_LARGE = range(9)
F32, BF16 = 0, 1
HYPER_CUBE, HYPER_CROSS, CUSTOM = 0, 1, 2
MAX_W = 8

# name -> (restype, argtypes); mirrors include/rmn_b200.h one to one
SIGNATURES = {
    "rmn_version": (c_int, []),
    "rmn_status_string": (c_char_p, [c_int]),
    "rmn_launch_count": (ctypes.c_ulonglong, []),
    "rmn_tensor_core_launch_count": (ctypes.c_ulonglong, []),
    "rmn_device_status": (c_int, [c_void_p]),
    "rmn_table_bytes": (c_size_t, [c_uint32]),
    "rmn_table_build_workspace_bytes": (c_size_t, [c_uint32]),
    "rmn_table_build": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_size_t, c_void_p]),
    "rmn_table_build_begin": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "rmn_table_build_finish": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "rmn_table_build_static_max_rows": (c_uint32, []),
    "rmn_table_build_static": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "rmn_table_info": (c_int, [c_void_p, c_void_p, c_void_p]),
    "rmn_readback_small": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "rmn_table_find": (c_int, [c_void_p, c_void_p, c_uint32, c_int, c_void_p, c_void_p]),
    "rmn_coords_stride": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p]),
    "rmn_region_volume": (c_int, [c_int, c_int, c_void_p, c_int]),
    "rmn_region_offsets": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "rmn_kmap_workspace_bytes": (c_size_t, [c_uint32, c_int]),
    "rmn_kmap_build": (c_int, [c_void_p, c_void_p, c_uint32, c_int, c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_size_t, c_void_p]),
    "rmn_kmap_build_self": (c_int, [c_void_p, c_void_p, c_uint32, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_size_t, c_void_p]),
    "rmn_kmap_pairs": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64,
                               c_void_p]),
    "rmn_kmap_pairs_background": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64,
                                          c_void_p]),
    "rmn_kmap_pairs_status": (c_int, [c_void_p, c_uint32, c_int, c_void_p]),
    "rmn_kmap_transpose": (c_int, [c_void_p, c_uint32, c_int, c_uint32, c_void_p, c_void_p]),
    "rmn_conv_forward": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p, c_uint32,
                                 c_void_p, c_int, c_void_p]),
    "rmn_conv_forward_fused": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p, c_uint32,
                                       c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "rmn_conv_backward_input": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p, c_uint32,
                                        c_void_p, c_int, c_void_p]),
    "rmn_conv_backward_weight_workspace_bytes": (c_size_t, [c_uint32, c_int, c_int, c_int, c_int]),
    "rmn_conv_backward_weight": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_uint32, c_int, c_void_p, c_int,
                                         c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "rmn_conv_plan_bytes": (c_size_t, [c_uint32, c_int]),
    "rmn_conv_plan_workspace_bytes": (c_size_t, [c_uint32, c_int]),
    "rmn_conv_plan_build": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_void_p, c_size_t, c_void_p,
                                    c_size_t, c_void_p]),
    "rmn_conv_forward_planned": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                         c_uint32, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "rmn_conv_backward_input_planned": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p,
                                                c_void_p, c_uint32, c_void_p, c_int, c_void_p]),
    "rmn_conv_forward_stats_planned": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p,
                                               c_void_p, c_uint32, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                               c_void_p, c_void_p, c_size_t, c_void_p]),
    "rmn_channel_dot_stats_workspace_bytes": (c_size_t, [c_int]),
    "rmn_channel_dot_stats": (c_int, [c_void_p, c_void_p, c_uint32, c_int, c_int, c_void_p, c_void_p, c_size_t,
                                      c_void_p]),
    "rmn_bn_forward_coeffs": (c_int, [c_void_p, ctypes.c_double, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      ctypes.c_float, ctypes.c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p]),
    "rmn_bn_backward_coeffs": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, ctypes.c_double, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "rmn_affine2": (c_int, [c_void_p, c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p]),
    "rmn_comm_unique_id": (c_int, [c_void_p]),
    "rmn_comm_init": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "rmn_comm_destroy": (c_int, [c_void_p]),
    "rmn_allreduce_grads_workspace_bytes": (c_size_t, [c_void_p, c_int]),
    "rmn_allreduce_grads": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_int, c_int,
                                    c_void_p]),
    "rmn_coords_expand": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "rmn_field_quantize": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_void_p]),
    "rmn_coords_discretize": (c_int, [c_void_p, c_int, c_uint64, ctypes.c_double, c_void_p, c_void_p]),
    "rmn_field_splat": (c_int, [c_void_p, c_void_p, c_int, c_uint32, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "rmn_channel_stats_workspace_bytes": (c_size_t, [c_int]),
    "rmn_channel_stats": (c_int, [c_void_p, c_uint32, c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "rmn_conv_forward_stats": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_int, c_void_p, c_uint32,
                                       c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t,
                                       c_void_p]),
    "rmn_affine_act": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "rmn_pool_forward": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_uint32, c_int, c_void_p, c_void_p,
                                 c_int, c_void_p]),
    "rmn_pool_backward": (c_int, [c_void_p, c_uint32, c_int, c_void_p, c_int, c_uint32, c_int, c_void_p, c_void_p,
                                  c_int, c_void_p]),
}

_lib = None


class RmnError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().rmn_status_string(status).decode()
        super().__init__(f"{where}: {text} (status {status})")


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m riemannengine_b200._build` "
                "(there is no CPU fallback)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        raise RmnError(status, where)
