"""Flash-attention forward through the C ABI.

Host-side mirror of ``examples/src/flash_forward.rs``: ``grid`` (:444-446) and
``run`` (:457-568) with torch tensors standing in for the reference's device
buffers, widened to a batch of planes, a non-causal mode, bf16 output and LSE.
"""
from __future__ import annotations

import torch

from ._lib import check, library

QUERIES = 128
HEAD = 128
#: The reference's score scale (examples/src/flash_forward.rs:321).
SCALE = 0.125


def items(sequence: int, planes: int, causal: bool = False) -> int:
    """Work items of a launch: one per pair of 128-row query tiles per plane; under a causal
    mask a heavy and a light query block of one plane share an item, so half as many."""
    pairs = (sequence + 2 * QUERIES - 1) // (2 * QUERIES)
    return ((pairs + 1) // 2 if causal else pairs) * planes


def grid(sequence: int, planes: int, sm_count: int = 148, causal: bool = False) -> int:
    """CTAs of a launch: one persistent CTA per SM, fewer when there are fewer work entries. Without a
    mask the items left after the whole rounds are walked as two single tiles each when those fit one round."""
    count = items(sequence, planes, causal)
    tail = count % sm_count
    if not causal and tail and 2 * tail <= sm_count:
        count += tail
    return min(count, sm_count)


def _require(name: str, tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
        raise ValueError(f"{name} must be a contiguous bfloat16 tensor")


def run(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
        causal: bool = False, out_dtype: torch.dtype = torch.bfloat16,
        status: torch.Tensor | None = None):
    """``softmax(scale * Q K^T [+ causal mask]) V`` over ``[..., seq, 128]`` bf16 tensors.

    Leading dimensions (batch, heads) are flattened into planes. Returns
    ``(out, lse)``: ``out`` in ``out_dtype`` (bf16, or fp32 as the reference
    kernel writes it) and ``lse`` as fp32 natural-log normalisers ``[..., seq]``.
    """
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        _require(name, tensor)
    if q.shape != k.shape or q.shape != v.shape or q.shape[-1] != HEAD:
        raise ValueError("q, k and v must share one [..., seq, 128] shape")
    sequence = q.shape[-2]
    planes = q.numel() // (sequence * HEAD)
    if scale is None:
        scale = HEAD ** -0.5
    out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    lse = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        handle = torch.cuda.current_stream().cuda_stream
        check(library().fk_flash_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(),
            out.data_ptr() if out_dtype == torch.bfloat16 else None,
            out.data_ptr() if out_dtype == torch.float32 else None,
            lse.data_ptr(), planes, sequence, float(scale), int(causal), handle,
            status.data_ptr() if status is not None else None))
    return out, lse


def run_host(q, k, v, out, lse, planes: int, sequence: int, scale: float, causal: bool) -> None:
    """The whole path from host buffers: stage Q, K, V, launch, read O and LSE back."""
    def address(x):
        if x is None:
            return None
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
    check(library().fk_flash_fwd_host(address(q), address(k), address(v), address(out), address(lse),
                                      planes, sequence, float(scale), int(causal)))
