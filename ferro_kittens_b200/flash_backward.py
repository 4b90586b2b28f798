"""Flash-attention backward through the C ABI: ``(dq, dk, dv)`` from ``q, k, v, out, d_out`` and the
log-sum-exp ``flash_forward.run`` returned. torch supplies memory and streams only; there is no CPU
path and no autograd wrapper here.
"""
from __future__ import annotations

import torch

from ._lib import check, library

HEAD = 128


def _require(name: str, tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
        raise ValueError(f"{name} must be a contiguous bfloat16 tensor")


def run(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, d_out: torch.Tensor,
        lse: torch.Tensor, scale: float | None = None, causal: bool = False,
        status: torch.Tensor | None = None, workspace: torch.Tensor | None = None):
    """Gradients of ``softmax(scale * Q K^T [+ causal mask]) V`` with respect to q, k and v."""
    for name, tensor in (("q", q), ("k", k), ("v", v), ("out", out), ("d_out", d_out)):
        _require(name, tensor)
        if tensor.shape != q.shape:
            raise ValueError("q, k, v, out and d_out must share one [..., seq, 128] shape")
    if q.shape[-1] != HEAD:
        raise ValueError("the head dimension is 128")
    if lse.dtype != torch.float32 or not lse.is_contiguous() or lse.shape != q.shape[:-1]:
        raise ValueError("lse must be the contiguous float32 [..., seq] the forward returned")
    sequence = q.shape[-2]
    planes = q.numel() // (sequence * HEAD)
    if scale is None:
        scale = HEAD ** -0.5
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    floats = library().fk_flash_bwd_workspace_bytes(planes, sequence) // 4
    if workspace is None:
        workspace = torch.empty(floats, dtype=torch.float32, device=q.device)
    elif workspace.dtype != torch.float32 or workspace.numel() < floats or not workspace.is_cuda:
        raise ValueError(f"the workspace must be at least {floats} float32 on the device")
    with torch.cuda.device(q.device):
        handle = torch.cuda.current_stream().cuda_stream
        check(library().fk_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(),
                                     lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                     workspace.data_ptr(), planes, sequence, float(scale), int(causal), handle,
                                     status.data_ptr() if status is not None else None))
    return dq, dk, dv
