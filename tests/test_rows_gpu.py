"""The row kernels against the oracle, through the C ABI: the reference's own gates
(examples/src/softmax.rs:215-300, examples/src/layernorm.rs:380-470, 505-590) with its seeds and
tolerances, then seeded random rows, in-place use, many tiles per CTA, and the shape guards."""
import numpy as np
import pytest
import torch

import oracle
from ferro_kittens_b200 import FerroKittensError, gemm, rows

pytestmark = pytest.mark.gpu


def _device(words: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16)).to(device).view(torch.bfloat16)


def _values(tensor: torch.Tensor) -> np.ndarray:
    return tensor.float().cpu().numpy().astype(np.float64)


def _checked(function, *args, **kwargs):
    status = gemm.new_status(args[0].device)
    out = function(*args, status=status, **kwargs)
    torch.cuda.synchronize(args[0].device)
    gemm.check_status(status)
    return out


def test_softmax_reference_gate(device):
    """CHECK_ROWS = 256 rows x CHECK_PLANES = 2, every output within 2^-8 relative of the closed form."""
    words = oracle.softmax_stage(256, 2)
    out = _values(_checked(rows.softmax_rows, _device(words, device)))
    expected = np.array([[[oracle.softmax_expected(p, r, c) for c in range(128)] for r in range(256)]
                         for p in range(2)])
    worst = np.abs(out / expected - 1).max()
    assert worst <= 1 / 256, worst
    assert np.abs(out / oracle.softmax_rows(words) - 1).max() <= 1 / 256


def test_layernorm_reference_gate(device):
    """CHECK_ROWS = 256, epsilon 1e-5, every output within 2^-7 relative (layernorm.rs:399, 434)."""
    x, gamma, beta = oracle.layernorm_stage(256)
    out = _values(_checked(rows.layernorm_rows, _device(x, device), _device(gamma, device), _device(beta, device),
                           rows.EPSILON))
    expected = oracle.layernorm_rows(x, gamma, beta, rows.EPSILON)
    worst = (np.abs(out - expected) / np.abs(expected)).max()
    assert worst <= 1 / 128, worst


def test_groupnorm_reference_gate(device):
    """The whole-tile statistic: absolute error within 1/64 (layernorm.rs:519, 568)."""
    x, _, _ = oracle.layernorm_stage(256)
    out = _values(_checked(rows.groupnorm_tile, _device(x, device), rows.EPSILON))
    expected = oracle.groupnorm_tiles(x, rows.EPSILON)
    worst = np.abs(out - expected).max()
    assert worst <= 1 / 64, worst
    # The two tiles have different statistics, so a kernel that normalised per row would differ.
    assert np.abs(oracle.layernorm_rows(x, np.full(128, oracle.to_bf16(1.0), np.uint16),
                                        np.zeros(128, np.uint16), rows.EPSILON) - expected).max() > 0.05


@pytest.mark.parametrize("tiles", [1, 5, 148, 149, 1000])
def test_seeded_random_rows(device, tiles):
    """One tile, fewer tiles than SMs, exactly one each, one CTA with two, and a ring that wraps."""
    generator = torch.Generator(device="cpu").manual_seed(20 + tiles)
    x = (torch.randn((tiles * 128, 128), generator=generator) * 3).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(128, generator=generator)).to(torch.bfloat16)
    beta = (0.5 * torch.randn(128, generator=generator)).to(torch.bfloat16)
    words = x.view(torch.int16).numpy().view(np.uint16)
    gw, bw = (t.view(torch.int16).numpy().view(np.uint16) for t in (gamma, beta))
    xd = x.to(device)
    soft = _values(_checked(rows.softmax_rows, xd))
    # bf16 output: half an ulp is 2^-9 relative; the ex2 unit and the fp32 sum add a little.
    assert np.abs(soft / oracle.softmax_rows(words) - 1).max() <= 1 / 256
    assert np.abs(soft.sum(axis=1) - 1).max() <= 2e-2
    layer = _values(_checked(rows.layernorm_rows, xd, gamma.to(device), beta.to(device), 1e-5))
    expected = oracle.layernorm_rows(words, gw, bw, 1e-5)
    assert np.abs(layer - expected).max() <= 1 / 128 * max(1.0, np.abs(expected).max())
    group = _values(_checked(rows.groupnorm_tile, xd, 1e-5))
    assert np.abs(group - oracle.groupnorm_tiles(words, 1e-5)).max() <= 1 / 64 * 4


def test_in_place_and_planes(device):
    words = oracle.softmax_stage(384, 3)
    x = _device(words, device)
    expected = _checked(rows.softmax_rows, x).clone()
    status = gemm.new_status(device)
    rows.softmax_rows(x, out=x, status=status)
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    assert torch.equal(x, expected)


def test_full_size_properties(device):
    """1 Gi elements in and out (2 GiB each way): every softmax row sums to one, every layernorm row
    has mean beta and unit spread under gamma = 1."""
    total_rows = 8 * 1024 * 1024 // 8  # 1 Mi rows x 128 = 128 Mi elements: larger than L2, seconds on the host
    generator = torch.Generator(device=device).manual_seed(7)
    x = (torch.randn((total_rows, 128), generator=generator, device=device) * 2).to(torch.bfloat16)
    soft = _checked(rows.softmax_rows, x)
    sums = soft.float().sum(dim=1)
    assert (sums - 1).abs().max().item() <= 2e-2
    ones = torch.ones(128, dtype=torch.bfloat16, device=device)
    zeros = torch.zeros(128, dtype=torch.bfloat16, device=device)
    layer = _checked(rows.layernorm_rows, x, ones, zeros, 1e-5).float()
    assert layer.mean(dim=1).abs().max().item() <= 2e-2
    assert (layer.var(dim=1, unbiased=False) - 1).abs().max().item() <= 5e-2
    sample = slice(total_rows - 256, total_rows)
    words = x[sample].view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.abs(_values(soft[sample]) / oracle.softmax_rows(words) - 1).max() <= 1 / 256


def test_shape_and_alignment_guards(device):
    x = torch.zeros((130, 128), dtype=torch.bfloat16, device=device)
    with pytest.raises(FerroKittensError, match="does not divide"):
        rows.softmax_rows(x)
    with pytest.raises(FerroKittensError, match="does not divide"):
        rows.groupnorm_tile(x)
    with pytest.raises(ValueError, match="128 columns"):
        rows.softmax_rows(torch.zeros((128, 64), dtype=torch.bfloat16, device=device))
    with pytest.raises(RuntimeError, match="no CPU path"):
        rows.softmax_rows(torch.zeros((128, 128), dtype=torch.bfloat16))
    big = torch.zeros((129, 128), dtype=torch.bfloat16, device=device)
    from ferro_kittens_b200._lib import check, library
    with pytest.raises(FerroKittensError, match="16-byte aligned"):
        check(library().fk_softmax_rows(big.data_ptr() + 2, big.data_ptr(), 128, 1,
                                        torch.cuda.current_stream().cuda_stream, None))
