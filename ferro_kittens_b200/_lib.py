"""Loads the C-ABI shared library and declares its entry points for ctypes.

There is no fallback: if the CUDA library is missing or fails to load, every
operation of this package raises. The bindings below are the Python spelling of
``include/ferro_kittens.h``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_uint16, c_uint32, c_uint64, c_void_p

from .build import LIBRARY, build_library

FK_OK = 0
FK_ERR_INVALID = -1
FK_ERR_SHAPE = -2
FK_ERR_ALIGNMENT = -3
FK_ERR_TOO_LARGE = -4
FK_ERR_DRIVER = -5
FK_ERR_TIMEOUT = -6
FK_ERR_DEVICE_STALL = -7

FK_BF16, FK_F16, FK_F32 = 0, 1, 2
FK_SWIZZLE_NONE, FK_SWIZZLE_128B = 0, 3


class FerroKittensError(RuntimeError):
    """A C-ABI call returned an error; ``code`` is the FK_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class Layout(ctypes.Structure):
    """``fk_layout_t``."""

    _fields_ = [
        ("base", c_uint64),
        ("rank", c_uint32),
        ("element", c_uint32),
        ("extents", c_uint64 * 5),
        ("strides_bytes", c_uint64 * 5),
    ]


class Plan(ctypes.Structure):
    """``fk_plan_t``."""

    _fields_ = [("bytes", c_uint64)]


# name -> (restype, argtypes); also the list the symbol test walks.
SIGNATURES = {
    "fk_last_error": (c_char_p, []),
    "fk_layout_packed": (c_int, [POINTER(Layout), c_uint64, c_uint32, c_uint32, POINTER(c_uint64)]),
    "fk_layout_strided": (c_int, [POINTER(Layout), c_uint64, c_uint32, c_uint32, POINTER(c_uint64),
                                  POINTER(c_uint64)]),
    "fk_layout_descriptor_shape": (c_int, [POINTER(Layout), c_uint32, c_uint32, POINTER(c_uint64),
                                           POINTER(c_uint32)]),
    "fk_layout_check": (c_int, [POINTER(Layout), POINTER(c_uint64), POINTER(c_uint32)]),
    "fk_tensor_map": (c_int, [c_void_p, POINTER(Layout), c_uint32, c_uint32, c_uint32]),
    "fk_encode_bf16_panels": (c_int, [c_void_p, c_uint64, c_uint32, c_uint32, c_uint64, c_uint64]),
    "fk_plan_sizing": (None, [POINTER(Plan)]),
    "fk_plan_reserve": (c_uint64, [POINTER(Plan), c_uint64, c_uint64]),
    "fk_plan_tile": (c_uint64, [POINTER(Plan), c_uint32, c_uint64, c_uint64]),
    "fk_plan_tile_ring": (c_uint64, [POINTER(Plan), c_uint32, c_uint64, c_uint64, c_uint64]),
    "fk_plan_semaphores": (c_uint64, [POINTER(Plan), c_uint64]),
    "fk_plan_tmem_slot": (c_uint64, [POINTER(Plan)]),
    "fk_gemm_shared_bytes": (c_uint32, []),
    "fk_gemm_threads": (c_uint32, []),
    "fk_flash_shared_bytes": (c_uint32, []),
    "fk_flash_threads": (c_uint32, []),
    "fk_gemm_grid": (c_uint32, [c_uint32, c_uint32, c_uint32]),
    "fk_gemm_group": (c_uint32, [c_uint32, c_uint32, c_uint32]),
    "fk_gemm_item_columns": (c_uint32, [c_uint32, c_uint32, c_uint32, c_uint32, c_uint32]),
    "fk_gemm_launch_tiled": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p, c_uint32, c_uint32,
                                     c_uint32, c_uint32, c_uint32, c_void_p, c_void_p]),
    "fk_admit_shared_plan": (c_int, [c_void_p, c_uint32, POINTER(c_uint32)]),
    "fk_grouped": (None, [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]),
    "fk_swizzled_chunk_offset": (c_uint32, [c_uint32, c_uint32, c_uint32]),
    "fk_operand_descriptor": (c_uint64, [c_uint64, c_uint32]),
    "fk_instruction_descriptor": (c_uint32, [c_uint32, c_uint32, c_int, c_int]),
    "fk_tmem_address": (c_uint32, [c_uint32, c_uint32, c_uint32]),
    "fk_gemm_bf16_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32,
                                    c_uint32, c_void_p, c_void_p]),
    "fk_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32,
                             c_uint32, c_void_p, c_void_p]),
    "fk_gemm_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32,
                               c_uint32, c_void_p, c_void_p]),
    "fk_gemm_launch_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32,
                                     c_uint32, c_uint32, c_void_p, c_void_p]),
    "fk_gemm_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32,
                              c_uint32, c_uint32, c_void_p, c_void_p]),
    "fk_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32, c_uint32,
                        c_uint32, c_void_p, c_void_p]),
    "fk_gemm_workspace_bytes": (c_uint64, [c_uint32, c_uint32, c_uint32, c_uint32]),
    "fk_gemm_fused_workspace": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32,
                                        c_uint32, c_uint32, c_void_p, c_uint64, c_void_p, c_void_p]),
    "fk_gemm_bf16_host": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32]),
    "fk_gemm_bf16_host_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_uint32]),
    "fk_flash_fwd_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_uint32, c_uint32, c_float, c_int, c_void_p, c_void_p]),
    "fk_flash_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32,
                             c_uint32, c_float, c_int, c_void_p, c_void_p]),
    "fk_flash_fwd_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32,
                                  c_uint32, c_float, c_int]),
    "fk_flash_bwd_shared_bytes": (c_uint32, []),
    "fk_flash_bwd_threads": (c_uint32, []),
    "fk_flash_bwd_workspace_bytes": (c_uint64, [c_uint32, c_uint32]),
    "fk_flash_bwd": (c_int, [c_void_p] * 10 + [c_uint32, c_uint32, c_float, c_int, c_void_p, c_void_p]),
    "fk_rows_shared_bytes": (c_uint32, []),
    "fk_rows_threads": (c_uint32, []),
    "fk_softmax_rows": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p]),
    "fk_layernorm_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_float, c_void_p, c_void_p]),
    "fk_groupnorm_tile": (c_int, [c_void_p, c_void_p, c_uint32, c_float, c_void_p, c_void_p]),
    "fk_wait_stream": (c_int, [c_void_p, c_uint32]),
    "fk_wait_event": (c_int, [c_void_p, c_uint32]),
    "fk_launch_budget_ms": (c_uint32, []),
    "fk_selftest_deadline": (c_int, [c_uint32, c_uint32]),
    "fk_selftest_call_guard": (c_int, [c_int, c_uint32, POINTER(c_uint64), POINTER(c_uint64)]),
    "fk_status_check": (c_int, [c_void_p, c_void_p]),
    "fk_selftest_stall": (c_int, [c_void_p, c_void_p, c_uint32]),
    "fk_selftest_exp2": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p]),
}

_library = None


def library() -> ctypes.CDLL:
    """The loaded library; raises if it cannot be built or loaded."""
    global _library
    if _library is None:
        build_library()  # returns at once when the library is newer than every source
        handle = ctypes.CDLL(str(LIBRARY))
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(handle, name)  # AttributeError if the symbol is missing
            function.restype = restype
            function.argtypes = argtypes
        _library = handle
    return _library


def last_error() -> str:
    return library().fk_last_error().decode()


def check(code: int) -> None:
    """Raise ``FerroKittensError`` for a non-zero return code."""
    if code != FK_OK:
        raise FerroKittensError(code, last_error())
