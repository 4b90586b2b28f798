"""Flash-attention backward against the f64 oracle (itself held to torch autograd in float64 on the
CPU, tests/test_oracle.py) and against fp32 autograd on the GPU at larger sizes, through the C ABI.
Inputs to the backward are what this library's own forward produced."""
import numpy as np
import pytest
import torch

import oracle
from ferro_kittens_b200 import FerroKittensError, flash_backward, flash_forward, gemm

pytestmark = pytest.mark.gpu


def _words(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _forward_backward(q, k, v, d_out, scale, causal):
    status = gemm.new_status(q.device)
    out, lse = flash_forward.run(q, k, v, scale=scale, causal=causal, status=status)
    dq, dk, dv = flash_backward.run(q, k, v, out, d_out, lse, scale=scale, causal=causal, status=status)
    torch.cuda.synchronize(q.device)
    gemm.check_status(status)
    return out, dq, dk, dv


def _inputs(planes, sequence, seed, device, spread=1.0):
    generator = torch.Generator(device="cpu").manual_seed(seed)
    return [(torch.randn((planes, sequence, 128), generator=generator) * spread).to(torch.bfloat16).to(device)
            for _ in range(4)]


# bf16 outputs (2^-9 relative each) on top of P and dS rounded to bf16 before their MMAs: the same
# error sources as the forward's 2^-8 gate, summed over a row. Bound relative to the largest entry.
TOLERANCE = 2e-2


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sequence", [128, 256, 384])
def test_against_the_f64_oracle(device, sequence, causal):
    planes, scale = 2, 0.125
    q, k, v, d_out = _inputs(planes, sequence, 40 + sequence, device)
    _, dq, dk, dv = _forward_backward(q, k, v, d_out, scale, causal)
    for plane in range(planes):
        expected = oracle.flash_backward(_words(q[plane]), _words(k[plane]), _words(v[plane]), _words(d_out[plane]),
                                         scale, causal)
        for name, got, want in zip(("dq", "dk", "dv"), (dq, dk, dv), expected):
            error = np.abs(got[plane].float().cpu().numpy().astype(np.float64) - want).max()
            assert error <= TOLERANCE * np.abs(want).max(), (name, plane, error, np.abs(want).max())


@pytest.mark.parametrize("causal", [False, True])
def test_against_fp32_autograd_at_a_longer_sequence(device, causal):
    planes, sequence, scale = 3, 2048, 128 ** -0.5
    q, k, v, d_out = _inputs(planes, sequence, 7, device)
    _, dq, dk, dv = _forward_backward(q, k, v, d_out, scale, causal)
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    scores = qf @ kf.transpose(1, 2) * scale
    if causal:
        hidden = torch.triu(torch.ones(sequence, sequence, dtype=torch.bool, device=device), 1)
        scores = scores.masked_fill(hidden, float("-inf"))
    (torch.softmax(scores, dim=-1) @ vf).backward(d_out.float())
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        error = (got.float() - want).abs().max().item()
        assert error <= TOLERANCE * want.abs().max().item(), (name, error, want.abs().max().item())


def test_sharp_rows_and_a_caller_workspace(device):
    """Scores spread wide enough that most of a row's weight sits on a few keys."""
    planes, sequence, scale = 2, 512, 0.125
    q, k, v, d_out = _inputs(planes, sequence, 3, device, spread=3.0)
    status = gemm.new_status(device)
    out, lse = flash_forward.run(q, k, v, scale=scale, causal=True, status=status)
    workspace = torch.empty(2 * planes * sequence, dtype=torch.float32, device=device)
    dq, dk, dv = flash_backward.run(q, k, v, out, d_out, lse, scale=scale, causal=True, status=status,
                                    workspace=workspace)
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    # The workspace holds -lse * log2(e) and -rowsum(dO * O): they enter the kernels as addends.
    assert torch.allclose(workspace.view(planes, 2, sequence)[:, 0], -lse * 1.4426950408889634, rtol=1e-6, atol=1e-6)
    delta = (out.float() * d_out.float()).sum(dim=-1)
    assert torch.allclose(workspace.view(planes, 2, sequence)[:, 1], -delta, rtol=1e-4, atol=1e-3)
    for plane in range(planes):
        expected = oracle.flash_backward(_words(q[plane]), _words(k[plane]), _words(v[plane]), _words(d_out[plane]),
                                         scale, True)
        for got, want in zip((dq, dk, dv), expected):
            error = np.abs(got[plane].float().cpu().numpy().astype(np.float64) - want).max()
            assert error <= TOLERANCE * np.abs(want).max()


def test_guards(device):
    q = torch.zeros((1, 192, 128), dtype=torch.bfloat16, device=device)
    lse = torch.zeros((1, 192), dtype=torch.float32, device=device)
    with pytest.raises(FerroKittensError, match="does not divide"):
        flash_backward.run(q, q, q, q, q, lse)
    q = torch.zeros((1, 128, 128), dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match="float32"):
        flash_backward.run(q, q, q, q, q, torch.zeros((1, 128), dtype=torch.float16, device=device))
    with pytest.raises(ValueError, match="workspace"):
        flash_backward.run(q, q, q, q, q, torch.zeros((1, 128), dtype=torch.float32, device=device),
                           workspace=torch.zeros(8, dtype=torch.float32, device=device))
