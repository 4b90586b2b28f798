"""CPU oracle for the two hot paths -- TEST INFRASTRUCTURE, NOT PRODUCT.

ctypes bindings over ``fk_oracle.c``, the plain-C restatement of the CPU
references in ferro-kittens' ``examples/src/gemm.rs`` and
``examples/src/flash_forward.rs``. Only the tests, the smoke run and the
benchmark's CPU-baseline leg import this package; the library never does.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_float, c_int, c_size_t, c_uint16

import numpy as np

from .build import build_oracle

_lib = ctypes.CDLL(str(build_oracle()))

_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")

_lib.fko_threads.restype = c_int
_lib.fko_set_threads.argtypes = [c_int]
_lib.fko_set_threads.restype = None
_lib.fko_to_bf16.argtypes = [c_float]
_lib.fko_to_bf16.restype = c_uint16
_lib.fko_from_bf16.argtypes = [c_uint16]
_lib.fko_from_bf16.restype = c_float
_lib.fko_gemm_a_value.argtypes = [c_size_t, c_size_t]
_lib.fko_gemm_a_value.restype = c_float
_lib.fko_gemm_b_value.argtypes = [c_size_t, c_size_t]
_lib.fko_gemm_b_value.restype = c_float
_lib.fko_gemm_stage.argtypes = [c_int, c_size_t, c_size_t, _u16p]
_lib.fko_gemm_stage.restype = None
_lib.fko_to_f16.argtypes = [c_float]
_lib.fko_to_f16.restype = c_uint16
_lib.fko_exp2_approx.argtypes = [c_float]
_lib.fko_exp2_approx.restype = c_float
_lib.fko_bf16_add.argtypes = [c_uint16, c_uint16]
_lib.fko_bf16_add.restype = c_uint16
_lib.fko_gemm_stage_f16.argtypes = [c_int, c_size_t, c_size_t, _u16p]
_lib.fko_gemm_stage_f16.restype = None
_lib.fko_gemm_check_c.argtypes = [_u16p, c_size_t, c_size_t, c_size_t, POINTER(c_double), POINTER(c_size_t)]
_lib.fko_gemm_check_c.restype = c_size_t
_lib.fko_gemm_expected.argtypes = [c_size_t, c_size_t, c_size_t]
_lib.fko_gemm_expected.restype = c_uint16
_lib.fko_gemm_exact.argtypes = [c_size_t, c_size_t, c_size_t]
_lib.fko_gemm_exact.restype = c_float
_lib.fko_gemm_rows.argtypes = [_u16p, _u16p, c_size_t, c_size_t, c_size_t, c_size_t, ctypes.c_void_p, ctypes.c_void_p]
_lib.fko_gemm_rows.restype = None
_lib.fko_flash_permutation.argtypes = [c_size_t] * 4
_lib.fko_flash_permutation.restype = c_size_t
for _name in ("fko_flash_q_value", "fko_flash_k_value", "fko_flash_v_value"):
    getattr(_lib, _name).argtypes = [c_size_t] * 3
    getattr(_lib, _name).restype = c_float
_lib.fko_flash_stage.argtypes = [c_int, c_size_t, c_size_t, _u16p]
_lib.fko_flash_stage.restype = None
_lib.fko_flash_rows.argtypes = [_u16p, _u16p, _u16p, c_size_t, c_size_t, c_size_t, c_double, c_int, _f64p, ctypes.c_void_p]
_lib.fko_flash_rows.restype = None
_lib.fko_softmax_input.argtypes = [c_size_t] * 3
_lib.fko_softmax_input.restype = c_float
_lib.fko_softmax_expected.argtypes = [c_size_t] * 3
_lib.fko_softmax_expected.restype = c_double
_lib.fko_softmax_stage.argtypes = [c_size_t, c_size_t, _u16p]
_lib.fko_softmax_stage.restype = None
_lib.fko_softmax_rows.argtypes = [_u16p, c_size_t, _f64p]
_lib.fko_softmax_rows.restype = None
_lib.fko_layernorm_value.argtypes = [c_size_t, c_size_t]
_lib.fko_layernorm_value.restype = c_float
_lib.fko_layernorm_input.argtypes = [c_size_t, c_size_t]
_lib.fko_layernorm_input.restype = c_float
_lib.fko_layernorm_gamma.argtypes = [c_size_t]
_lib.fko_layernorm_gamma.restype = c_float
_lib.fko_layernorm_beta.argtypes = [c_size_t]
_lib.fko_layernorm_beta.restype = c_float
_lib.fko_layernorm_stage.argtypes = [c_size_t, _u16p, _u16p, _u16p]
_lib.fko_layernorm_stage.restype = None
_lib.fko_layernorm_rows.argtypes = [_u16p, _u16p, _u16p, c_size_t, c_double, _f64p]
_lib.fko_layernorm_rows.restype = None
_lib.fko_groupnorm_tiles.argtypes = [_u16p, c_size_t, c_double, _f64p]
_lib.fko_groupnorm_tiles.restype = None
_lib.fko_flash_backward.argtypes = [_u16p, _u16p, _u16p, _u16p, c_size_t, c_double, c_int, _f64p, _f64p, _f64p]
_lib.fko_flash_backward.restype = None


def threads() -> int:
    """Host threads the OpenMP loops use."""
    return _lib.fko_threads()


def use_all_cores() -> int:
    """Let the OpenMP loops use every core this process may run on (a launcher may have set
    OMP_NUM_THREADS=1); returns the count."""
    import os

    count = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    _lib.fko_set_threads(count)
    return threads()


def to_bf16(value: float) -> int:
    return _lib.fko_to_bf16(value)


def from_bf16(bits: int) -> float:
    return _lib.fko_from_bf16(bits)


def bf16_to_f32(words: np.ndarray) -> np.ndarray:
    """Widen an array of bf16 words to fp32 (exact)."""
    return (words.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 words with the reference's rule (gemm.rs:444-447), vectorised."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + (np.uint32(0x7FFF) + ((bits >> 16) & 1))) >> 16).astype(np.uint16)


def gemm_a_value(row: int, depth: int) -> float:
    return _lib.fko_gemm_a_value(row, depth)


def gemm_b_value(column: int, depth: int) -> float:
    return _lib.fko_gemm_b_value(column, depth)


def gemm_stage(which: str, rows: int, k: int) -> np.ndarray:
    """The reference's integer operand ``a`` or ``b`` as [rows, k] bf16 words."""
    out = np.empty((rows, k), dtype=np.uint16)
    _lib.fko_gemm_stage(0 if which == "a" else 1, rows, k, out)
    return out


def gemm_stage_f16(which: str, rows: int, k: int) -> np.ndarray:
    """The same operand as [rows, k] fp16 words (examples/src/gemm_sol.rs:1241-1249)."""
    out = np.empty((rows, k), dtype=np.uint16)
    _lib.fko_gemm_stage_f16(0 if which == "a" else 1, rows, k, out)
    return out


def to_f16(value: float) -> int:
    return _lib.fko_to_f16(value)


def exp2_approx(value: float) -> float:
    """The reference's polynomial 2^x (src/reg.rs:81-93), in its own operation order."""
    return float(_lib.fko_exp2_approx(value))


def bf16_add(held: int, added: int) -> int:
    """What a bf16 reduce-add leaves: the exact sum rounded once to bf16."""
    return _lib.fko_bf16_add(held, added)


def bf16_add_words(held: np.ndarray, added: np.ndarray) -> np.ndarray:
    """``bf16_add`` over arrays: exact sum in float64, one round-to-nearest-even to bf16."""
    total = bf16_to_f32(held).astype(np.float64) + bf16_to_f32(added).astype(np.float64)
    bits = total.view(np.uint64)
    sign = (bits >> np.uint64(63)).astype(np.uint32)
    exponent = ((bits >> np.uint64(52)) & np.uint64(0x7FF)).astype(np.int64) - 1023
    mantissa = bits & np.uint64((1 << 52) - 1)
    kept = (mantissa >> np.uint64(45)).astype(np.uint32)
    rest = mantissa & np.uint64((1 << 45) - 1)
    up = (rest > np.uint64(1 << 44)) | ((rest == np.uint64(1 << 44)) & ((kept & 1) == 1))
    combined = ((exponent + 127).astype(np.uint32) << 7) + kept + up.astype(np.uint32)  # a carry bumps the exponent
    out = (sign << 15) | combined
    out = np.where(total == 0.0, sign << 15, out)
    assert np.all((exponent >= -126) & (exponent <= 126) | (total == 0.0)), "outside the range this helper covers"
    return out.astype(np.uint16)


def gemm_check_c(observed: np.ndarray, m: int, n: int, k: int) -> tuple[int, float, int]:
    """(wrong elements, worst relative error, flat index of the first wrong element)."""
    worst = c_double(0.0)
    first = c_size_t(0)
    observed = np.ascontiguousarray(observed, dtype=np.uint16).reshape(m, n)
    wrong = _lib.fko_gemm_check_c(observed, m, n, k, ctypes.byref(worst), ctypes.byref(first))
    return int(wrong), float(worst.value), int(first.value)


def gemm_expected(row: int, column: int, k: int) -> int:
    return _lib.fko_gemm_expected(row, column, k)


def gemm_exact(m: int, n: int, k: int) -> np.ndarray:
    """The [m, n] fp32 values of the integer-operand product before their rounding (7 x 21 distinct cells)."""
    cells = np.array([[_lib.fko_gemm_exact(r, c, k) for c in range(21)] for r in range(7)], dtype=np.float32)
    return cells[np.arange(m)[:, None] % 7, np.arange(n)[None, :] % 21]


def gemm_rows(a: np.ndarray, b: np.ndarray, row0: int, rows: int, want_f64: bool = False):
    """Rows [row0, row0+rows) of C = A . B^T over bf16 words; returns (bf16 words, f64 or None)."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    n, k = b.shape
    assert a.shape[1] == k
    c = np.empty((rows, n), dtype=np.uint16)
    c64 = np.empty((rows, n), dtype=np.float64) if want_f64 else None
    _lib.fko_gemm_rows(a, b, n, k, row0, rows, c.ctypes.data, c64.ctypes.data if want_f64 else None)
    return c, c64


def flash_stage(which: str, sequence: int, heads: int) -> np.ndarray:
    """The reference's lattice operand ``q``, ``k`` or ``v`` as [heads, sequence, 128] bf16 words."""
    out = np.empty((heads, sequence, 128), dtype=np.uint16)
    _lib.fko_flash_stage({"q": 0, "k": 1, "v": 2}[which], sequence, heads, out)
    return out


def flash_rows(q: np.ndarray, k: np.ndarray, v: np.ndarray, row0: int, rows: int, scale: float,
               causal: bool):
    """f64 attention rows of one [sequence, 128] plane; returns (out [rows,128], lse [rows])."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    sequence = q.shape[0]
    out = np.empty((rows, 128), dtype=np.float64)
    lse = np.empty(rows, dtype=np.float64)
    _lib.fko_flash_rows(q, k, v, sequence, row0, rows, scale, int(causal), out, lse.ctypes.data)
    return out, lse


def softmax_stage(rows: int, planes: int) -> np.ndarray:
    """The reference's softmax seed as [planes, rows, 128] bf16 words (examples/src/softmax.rs:195-215)."""
    out = np.empty((planes, rows, 128), dtype=np.uint16)
    _lib.fko_softmax_stage(rows, planes, out)
    return out


def softmax_expected(plane: int, row: int, column: int) -> float:
    return _lib.fko_softmax_expected(plane, row, column)


def softmax_rows(x: np.ndarray) -> np.ndarray:
    """f64 base-2 softmax over the last axis (128) of bf16 words."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float64)
    _lib.fko_softmax_rows(x.reshape(-1, 128), x.size // 128, out.reshape(-1, 128))
    return out


def layernorm_stage(rows: int):
    """The reference's layernorm seed: (x [rows, 128], gamma [128], beta [128]) as bf16 words."""
    x = np.empty((rows, 128), dtype=np.uint16)
    gamma = np.empty(128, dtype=np.uint16)
    beta = np.empty(128, dtype=np.uint16)
    _lib.fko_layernorm_stage(rows, x, gamma, beta)
    return x, gamma, beta


def layernorm_rows(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, epsilon: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, 128)
    out = np.empty(x.shape, dtype=np.float64)
    _lib.fko_layernorm_rows(x, np.ascontiguousarray(gamma, dtype=np.uint16), np.ascontiguousarray(beta, dtype=np.uint16),
                            x.shape[0], epsilon, out)
    return out


def groupnorm_tiles(x: np.ndarray, epsilon: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, 128)
    out = np.empty(x.shape, dtype=np.float64)
    _lib.fko_groupnorm_tiles(x, x.shape[0], epsilon, out)
    return out


def flash_backward(q: np.ndarray, k: np.ndarray, v: np.ndarray, d_out: np.ndarray, scale: float, causal: bool):
    """f64 gradients (dq, dk, dv) of one [sequence, 128] plane of bf16 words."""
    q, k, v, d_out = (np.ascontiguousarray(x, dtype=np.uint16) for x in (q, k, v, d_out))
    sequence = q.shape[0]
    dq, dk, dv = (np.empty((sequence, 128), dtype=np.float64) for _ in range(3))
    _lib.fko_flash_backward(q, k, v, d_out, sequence, scale, int(causal), dq, dk, dv)
    return dq, dk, dv
