"""Launches under one wave with K split across the idle clusters (`fk_gemm_fused_workspace`): every
run of k-blocks adds its fp32 tile into the workspace, the last to arrive rounds once. Exact on the
reference's integer gate, where every partial sum is an integer fp32 holds, with the fused epilogue
and both operand types; the workspace comes back all zero, so it serves the next launch uncleared."""
import numpy as np
import pytest
import torch

import oracle
from ferro_kittens_b200 import FerroKittensError, gemm
from ferro_kittens_b200._lib import FK_ERR_TOO_LARGE, check, library

pytestmark = pytest.mark.gpu


def _device_words(words: np.ndarray, device, dtype) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16)).to(device).view(dtype)


def _words(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _run(a, b, workspace, **kwargs):
    status = gemm.new_status(a.device)
    c = gemm.run(a, b, status=status, workspace=workspace, **kwargs)
    torch.cuda.synchronize(a.device)
    gemm.check_status(status)
    return c


def test_which_shapes_split(device):
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    lib = library()
    assert lib.fk_gemm_workspace_bytes(256, 256, 32768, sms) >= 256 * 256 * 4
    assert lib.fk_gemm_workspace_bytes(512, 512, 65536, sms) >= 512 * 512 * 4
    assert lib.fk_gemm_workspace_bytes(16384, 16384, 16384, sms) == 0  # many waves
    assert lib.fk_gemm_workspace_bytes(1024, 1024, 32768, sms) == 0    # tiles enough for the cluster-sliced narrow kernel
    assert lib.fk_gemm_workspace_bytes(256, 256, 16384, sms) == 0      # too shallow to repay the fp32 round trip
    assert lib.fk_gemm_workspace_bytes(512, 256, 256, sms) == 0        # four k-blocks: nothing to cut
    assert lib.fk_gemm_workspace_bytes(500, 256, 256, sms) == 0        # not a shape at all
    assert gemm.workspace(16384, 16384, 16384, device) is None


# The reference's integer gate (examples/src/gemm.rs:434-440, 544-578) at depths that split: one tile
# cut sixteen ways, a two-tile strip, a K that does not divide into equal runs (513 k-blocks) under a
# ragged last row tile, and a square of four tiles.
@pytest.mark.parametrize("shape", [(256, 256, 32768), (256, 512, 32768), (768, 256, 32832), (512, 512, 32768)])
def test_exact_on_the_reference_gate_twice_with_one_workspace(device, shape):
    m, n, k = shape
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    workspace = gemm.workspace(m, n, k, device)
    assert workspace is not None
    for _ in range(2):
        c = _run(a, b, workspace)
        wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
        assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"
        assert int(workspace.count_nonzero().item()) == 0, "the launch did not leave its workspace zero"


def test_a_larger_workspace_serves_smaller_shapes_and_group_widths(device):
    workspace = gemm.workspace(512, 512, 32768, device)
    for (m, n, k), group in [((256, 512, 32768), 1), ((512, 256, 32768), 3), ((256, 256, 32768), 8),
                             ((1024, 1024, 512), 8)]:  # the last does not split and leaves the workspace alone
        a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
        b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
        c = _run(a, b, workspace, group=group)
        assert oracle.gemm_check_c(_words(c), m, n, k)[0] == 0
    assert int(workspace.count_nonzero().item()) == 0


@pytest.mark.parametrize("operands", ["bf16", "f16"])
def test_fused_epilogue_after_the_last_run(device, operands):
    """bias + ReLU + C += on the summed fp32 value, one rounding: the same cells as the one-launch path."""
    m, n, k = 512, 256, 32768
    stage = oracle.gemm_stage if operands == "bf16" else oracle.gemm_stage_f16
    dtype = torch.bfloat16 if operands == "bf16" else torch.float16
    a, b = _device_words(stage("a", m, k), device, dtype), _device_words(stage("b", n, k), device, dtype)
    bias_values = ((np.arange(n) * 3) % 13 - 6).astype(np.float32)
    bias = _device_words(oracle.f32_to_bf16(bias_values), device, torch.bfloat16)
    held = oracle.f32_to_bf16(np.full((m, n), 1.5, dtype=np.float32))
    c = _device_words(held.copy(), device, torch.bfloat16)
    workspace = gemm.workspace(m, n, k, device)
    assert workspace is not None
    _run(a, b, workspace, c=c, accumulate=True, bias=bias, relu=True)
    fused = oracle.f32_to_bf16(np.maximum(oracle.gemm_exact(m, n, k) + bias_values[None, :], np.float32(0.0)))
    assert np.array_equal(_words(c), oracle.bf16_add_words(held, fused))
    assert int(workspace.count_nonzero().item()) == 0


def test_seeded_random_within_tolerance_and_close_to_one_launch(device):
    m, n, k = 512, 512, 32768
    generator = torch.Generator(device="cpu").manual_seed(5)
    a = (torch.rand((m, k), generator=generator) * 2 - 1).to(torch.bfloat16).to(device)
    b = (torch.rand((n, k), generator=generator) * 2 - 1).to(torch.bfloat16).to(device)
    workspace = gemm.workspace(m, n, k, device)
    split = _run(a, b, workspace)
    whole = _run(a, b, None)
    reference = a.double() @ b.double().T
    # BASELINE's GEMM bound: 1e-2 * sqrt(K) * max|a| * max|b|.
    assert (split.double() - reference).abs().max().item() <= 1e-2 * k ** 0.5
    # the runs are summed in fp32 in another order: at most the last bf16 place differs
    assert (split.float() - whole.float()).abs().max().item() <= 2 ** -7 * reference.abs().max().item()


def test_a_short_workspace_is_refused_and_none_falls_back(device):
    m, n, k = 256, 512, 32768
    a = torch.zeros((m, k), dtype=torch.bfloat16, device=device)
    b = torch.zeros((n, k), dtype=torch.bfloat16, device=device)
    with pytest.raises(FerroKittensError, match="splits K over a workspace") as error:
        gemm.run(a, b, workspace=torch.zeros(1024, dtype=torch.uint8, device=device))
    assert error.value.code == FK_ERR_TOO_LARGE
    c = gemm.run(a, b, workspace=None)
    assert int(c.count_nonzero().item()) == 0
