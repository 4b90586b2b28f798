"""bf16 GEMM ``C = A . B^T`` through the C ABI.

Host-side mirror of ``examples/src/gemm.rs``: ``tile_grid`` (:466-468), ``grid``
(:472-475) and ``run`` (:477-538) with torch tensors standing in for the
reference's device buffers. torch supplies memory and streams only.
"""
from __future__ import annotations

import torch

from ._lib import check, library
from .global_layout import GlobalLayout

BLOCK_M = 128
BLOCK_N = 256
BLOCK_K = 64
#: The traversal width the reference ships (examples/src/gemm.rs:138).
GROUP = 8
#: fp16 A and B (C stays bf16): the operand types of examples/src/gemm_sol.rs.
F16_OPERANDS = 1
#: C += A . B^T through the copy engine's reduce-add (src/shared.rs:974-1009).
ACCUMULATE = 2
#: max(x, 0) before the rounding (the `Relu` unary map, src/reg.rs:261).
RELU = 4


def tile_grid(m: int, n: int) -> tuple[int, int]:
    return m // (2 * BLOCK_M), n // BLOCK_N


def grid(m: int, n: int, sm_count: int = 148) -> int:
    return library().fk_gemm_grid(m, n, sm_count)


def _require_cuda_bf16(name: str, tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
        raise ValueError(f"{name} must be a contiguous bfloat16 tensor")


def new_status(device) -> torch.Tensor:
    """Zeroed device words for a launch; it writes the first four only if one of its waits gives up."""
    return torch.zeros(8, dtype=torch.int32, device=device)


def maps(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor):
    """The three tensor maps of a launch: A and B as loads, C as a store."""
    m, k = a.shape
    n = b.shape[0]
    a_map = GlobalLayout.packed(a.data_ptr(), [k, m]).tensor_map(BLOCK_M)
    b_map = GlobalLayout.packed(b.data_ptr(), [k, n]).tensor_map(BLOCK_N // 2)
    c_map = GlobalLayout.strided(c.data_ptr(), [n, m], [1, c.stride(0)]).tensor_map(32)
    return a_map, b_map, c_map


def launch(a_map, b_map, c_map, m: int, n: int, k: int, group: int = GROUP, status=None,
           stream=None) -> None:
    """Enqueue the kernel on ``stream`` (torch's current stream by default)."""
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    check(library().fk_gemm_bf16_launch(a_map.as_ptr(), b_map.as_ptr(), c_map.as_ptr(), m, n, k,
                                        group, handle, status.data_ptr() if status is not None else None))


def run(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None = None, group: int = GROUP,
        status: torch.Tensor | None = None, accumulate: bool = False, bias: torch.Tensor | None = None,
        relu: bool = False) -> torch.Tensor:
    """``C[m, n] (+)= map(sum_k A[m, k] * B[n, k] + bias[n])``; A is [m, k], B is [n, k], both bf16 or both fp16 on
    one GPU, C bf16. With ``accumulate`` the rounded product is added into ``c`` (in bf16, by the
    copy engine), which must then be given and hold values."""
    for name, tensor in (("a", a), ("b", b)):
        if not tensor.is_cuda:
            raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
        if tensor.dtype not in (torch.bfloat16, torch.float16) or not tensor.is_contiguous():
            raise ValueError(f"{name} must be a contiguous bfloat16 or float16 tensor")
    if a.dtype != b.dtype:
        raise ValueError("a and b must share one element type")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k:
        raise ValueError("a and b disagree on K")
    if c is None:
        if accumulate:
            raise ValueError("accumulating needs the C to add into")
        c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if not c.is_cuda:
        raise RuntimeError("c must live on a CUDA device: there is no CPU path")
    if c.dtype != torch.bfloat16 or c.dim() != 2 or c.stride(1) != 1 or c.shape != (m, n):
        raise ValueError("c must be an [m, n] bfloat16 tensor with unit column stride (rows may be padded)")
    if bias is not None and (not bias.is_cuda or bias.dtype != torch.bfloat16 or bias.shape != (n,)
                             or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous bfloat16 [n] tensor on the device")
    flags = ((F16_OPERANDS if a.dtype == torch.float16 else 0) | (ACCUMULATE if accumulate else 0)
             | (RELU if relu else 0))
    with torch.cuda.device(a.device):
        handle = torch.cuda.current_stream().cuda_stream
        check(library().fk_gemm_fused(a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                      bias.data_ptr() if bias is not None else None, m, n, k, c.stride(0), group,
                                      flags, handle, status.data_ptr() if status is not None else None))
    return c


def check_status(status: torch.Tensor) -> None:
    """Raise if the kernel recorded a stalled wait."""
    with torch.cuda.device(status.device):
        check(library().fk_status_check(status.data_ptr(), torch.cuda.current_stream().cuda_stream))


def run_host(a, b, c, m: int, n: int, k: int, group: int = GROUP) -> None:
    """The whole path from host buffers (numpy uint16 / pinned torch tensors): stage, launch, read back."""
    def address(x):
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
    check(library().fk_gemm_bf16_host(address(a), address(b), address(c), m, n, k, group))


def run_host_noalloc(a, b, c, m: int, n: int, k: int, group: int = GROUP) -> None:
    """``run_host`` for callers that must not reach the CUDA allocator: the staging lives in an
    array built into the library, so each of A, B and C is limited to 8 MiB."""
    def address(x):
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
    check(library().fk_gemm_bf16_host_noalloc(address(a), address(b), address(c), m, n, k, group))
