"""The memory-bound row kernels through the C ABI: base-2 softmax over rows, layernorm over rows,
whole-tile normalisation, all over rows of 128 bf16 columns.

Host-side mirror of ``examples/src/softmax.rs`` (``run`` :215-300, ``grid`` :193-195) and
``examples/src/layernorm.rs`` (``run`` :380-470, ``run_group`` :505-590). torch supplies memory and
streams only; there is no CPU path.
"""
from __future__ import annotations

import torch

from ._lib import check, library

ROWS = 128
COLUMNS = 128
#: examples/src/layernorm.rs:313
EPSILON = 1e-5


def _require(name: str, tensor: torch.Tensor, columns: int = COLUMNS) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous() or tensor.shape[-1] != columns:
        raise ValueError(f"{name} must be a contiguous bfloat16 tensor of {columns} columns")


def _launch(entry, x: torch.Tensor, out: torch.Tensor | None, status, *middle):
    _require("x", x)
    if out is None:
        out = torch.empty_like(x)
    _require("out", out)
    if out.shape != x.shape:
        raise ValueError("out must have x's shape")
    with torch.cuda.device(x.device):
        handle = torch.cuda.current_stream().cuda_stream
        check(entry(x, out, handle, status.data_ptr() if status is not None else None, *middle))
    return out


def softmax_rows(x: torch.Tensor, out: torch.Tensor | None = None, status=None) -> torch.Tensor:
    """``2^(x - max) / sum`` along the last axis of ``[..., rows, 128]``; rows % 128 == 0."""
    rows = x.shape[-2] if x.dim() >= 2 else 0
    planes = x.numel() // (rows * COLUMNS) if rows else 0
    return _launch(lambda a, b, h, s: library().fk_softmax_rows(a.data_ptr(), b.data_ptr(), rows, planes, h, s),
                   x, out, status)


def layernorm_rows(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, epsilon: float = EPSILON,
                   out: torch.Tensor | None = None, status=None) -> torch.Tensor:
    """``gamma * (x - mean) / sqrt(var + epsilon) + beta`` per row of ``[rows, 128]``."""
    _require("gamma", gamma)
    _require("beta", beta)
    rows = x.numel() // COLUMNS
    return _launch(lambda a, b, h, s: library().fk_layernorm_rows(a.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                                                 b.data_ptr(), rows, epsilon, h, s),
                   x, out, status)


def groupnorm_tile(x: torch.Tensor, epsilon: float = EPSILON, out: torch.Tensor | None = None,
                   status=None) -> torch.Tensor:
    """``(x - mean) / sqrt(var + epsilon)`` with the statistics of each [128, 128] tile of ``[rows, 128]``."""
    rows = x.numel() // COLUMNS
    return _launch(lambda a, b, h, s: library().fk_groupnorm_tile(a.data_ptr(), b.data_ptr(), rows, epsilon, h, s),
                   x, out, status)
