"""GPU parity of the bf16 GEMM against the CPU oracle, through the C ABI.

The exact gates are the reference's own (examples/src/gemm.rs:422-430, 583-610):
integer operands, two sizes, four traversal widths, ``==`` on bf16 words. The
seeded random cases use the tolerance the task states:
``max|err| <= 1e-2 * sqrt(K) * max|a| * max|b|``.
"""
import math

import numpy as np
import pytest
import torch

import oracle
from ferro_kittens_b200 import FerroKittensError, gemm

pytestmark = pytest.mark.gpu


def _to_device(words: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16)).to(device).view(torch.bfloat16)


def _to_words(tensor: torch.Tensor) -> np.ndarray:
    return tensor.view(torch.int16).cpu().numpy().view(np.uint16)


def _run_checked(a, b, group=gemm.GROUP, tile="wide"):
    """These are the gates of the wide kernel (the replacement of `gemm_cg2_staged_x8x4`): small
    shapes would otherwise take the narrow tile, which has its own gates in test_gemm_variants_gpu.py."""
    status = gemm.new_status(a.device)
    c = gemm.run(a, b, group=group, status=status, tile=tile)
    gemm.check_status(status)
    return c


@pytest.mark.parametrize("shape", [(512, 256, 256), (4096, 4096, 256)])
@pytest.mark.parametrize("group", [8, 1, 3, 6])
def test_reference_integer_gate_is_exact(device, shape, group):
    m, n, k = shape
    a = _to_device(oracle.gemm_stage("a", m, k), device)
    b = _to_device(oracle.gemm_stage("b", n, k), device)
    c = _run_checked(a, b, group)
    wrong, worst, first = oracle.gemm_check_c(_to_words(c), m, n, k)
    assert wrong == 0, f"{wrong} of {m * n} elements wrong, first at flat index {first}"
    assert worst < 2 ** -8


@pytest.mark.parametrize("shape", [(256, 256, 64), (256, 256, 8192), (768, 1280, 1088)])
def test_integer_operands_other_shapes_exact(device, shape):
    """One tile and one k-block; a K deep enough to wrap the ring many times; ragged tile counts."""
    m, n, k = shape
    a = _to_device(oracle.gemm_stage("a", m, k), device)
    b = _to_device(oracle.gemm_stage("b", n, k), device)
    c = _run_checked(a, b, 3)
    # K past 256 leaves fp32 sums exact (|a*b| <= 30, K <= 8192 -> < 2^24).
    wrong, _, first = oracle.gemm_check_c(_to_words(c), m, n, k)
    assert wrong == 0, f"{wrong} wrong, first at {first}"


@pytest.mark.parametrize("tile", ["wide", None])
def test_config_1_uniform_1024_cubed(device, tile):
    """GEMM 1024^3, entries uniform[-1, 1) from seed 0, against the oracle over the same bf16 words:
    on the wide kernel, and as a launch this small runs when nothing is asked for (the narrow tile)."""
    m = n = k = 1024
    generator = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.rand((m, k), generator=generator) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand((n, k), generator=generator) * 2 - 1).to(torch.bfloat16)
    c = _run_checked(a.to(device), b.to(device), tile=tile)
    a_words, b_words = _to_words(a), _to_words(b)
    expected, exact = oracle.gemm_rows(a_words, b_words, 0, m, want_f64=True)
    got = oracle.bf16_to_f32(_to_words(c)).astype(np.float64)
    bound = 1e-2 * math.sqrt(k) * float(a.abs().max()) * float(b.abs().max())
    assert np.abs(got - exact).max() <= bound
    # Far tighter in practice: one bf16 rounding of an fp32-accumulated sum.
    assert np.abs(got - exact).max() <= np.abs(exact).max() * 2 ** -8 + 1e-3
    assert (np.abs(got - oracle.bf16_to_f32(expected)) <= np.abs(exact) * 2 ** -7 + 1e-3).all()


def test_leading_dimension_and_linearity(device):
    """C written into a wider buffer leaves the margin untouched; (2A).B == 2(A.B) exactly in bf16."""
    m, n, k = 512, 512, 512
    generator = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn((m, k), generator=generator).to(torch.bfloat16).to(device)
    b = torch.randn((n, k), generator=generator).to(torch.bfloat16).to(device)
    wide = torch.full((m, n + 64), 7.0, dtype=torch.bfloat16, device=device)
    status = gemm.new_status(device)
    from ferro_kittens_b200._lib import check, library
    check(library().fk_gemm_bf16(a.data_ptr(), b.data_ptr(), wide.data_ptr(), m, n, k, n + 64, 8,
                                 torch.cuda.current_stream().cuda_stream, status.data_ptr()))
    gemm.check_status(status)
    c = _run_checked(a, b)
    assert torch.equal(wide[:, :n], c)
    assert (wide[:, n:] == 7.0).all()
    doubled = _run_checked(a * 2, b)
    assert torch.equal(doubled, c * 2)


def test_shape_guards_reject_before_launch(device):
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device=device)
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device=device)
    with pytest.raises(FerroKittensError, match="traversal group width of 0"):
        gemm.run(a, b, group=0)
    with pytest.raises(FerroKittensError, match="does not divide"):
        gemm.run(a[:128].contiguous(), b)
    with pytest.raises(RuntimeError, match="no CPU path"):
        gemm.run(a.cpu(), b.cpu())


@pytest.mark.parametrize("shape", [(512, 256, 256), (4352, 512, 128)])
def test_host_buffer_entry_point(device, shape):
    """Host buffers in and out; the second shape is 17 row tiles, which the entry's pipeline cuts into
    eight blocks of two tiles and a last block of one."""
    m, n, k = shape
    a = oracle.gemm_stage("a", m, k)
    b = oracle.gemm_stage("b", n, k)
    c = np.zeros((m, n), dtype=np.uint16)
    gemm.run_host(a, b, c, m, n, k)
    wrong, _, _ = oracle.gemm_check_c(c, m, n, k)
    assert wrong == 0


def test_two_threads_calling_the_host_entry_on_one_device_take_turns(device):
    """The host-buffer entries share the device's staging buffers, streams and status words and hold
    the device's lock for the whole call: two threads with different shapes (the second outgrows the
    first's staging, which is freed and re-made) both get the exact answer."""
    import threading

    shapes = [(1024, 768, 256), (2048, 1280, 512), (512, 256, 1088)]
    results = {}

    def worker(index, shape):
        m, n, k = shape
        a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
        wrong = 0
        for _ in range(4):
            c = np.full((m, n), 0xFFFF, dtype=np.uint16)
            torch.cuda.set_device(device)
            gemm.run_host(a, b, c, m, n, k)
            wrong += oracle.gemm_check_c(c, m, n, k)[0]
        results[index] = wrong

    threads = [threading.Thread(target=worker, args=(index, shape)) for index, shape in enumerate(shapes)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert results == {0: 0, 1: 0, 2: 0}


@pytest.mark.parametrize("blocks", [1, 4])
def test_host_buffer_pipeline_over_row_blocks(device, blocks):
    """The multi-GPU host-buffer pipeline with a world of one (upload by row blocks, GEMM per block,
    read-back; the all-gather between upload and GEMM is the only step a single rank skips): exact on
    the reference's integer gate, twice in a row with the same buffers."""
    m, n, k = 2048, 768, 256
    a = torch.from_numpy(oracle.gemm_stage("a", m, k).view(np.int16)).view(torch.bfloat16).pin_memory()
    b = torch.from_numpy(oracle.gemm_stage("b", n, k).view(np.int16)).view(torch.bfloat16).pin_memory()
    c = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    plan = gemm.ShardedHostGemm(m, n, k, 1, 0, device, blocks=blocks)
    assert plan.bytes_per_step() == ((m * k + n * k) * 2, m * n * 2)
    for _ in range(2):
        c.zero_()
        plan.run(a, b, c)
        assert oracle.gemm_check_c(c.view(torch.int16).numpy().view(np.uint16), m, n, k)[0] == 0
    with pytest.raises(ValueError):
        plan.run(a[:1024], b, c)


@pytest.mark.parametrize("shape, seed, deviation", [((16384, 16384, 16384), 1, None), ((8192, 28672, 8192), 2, 0.02)])
def test_full_size_properties(device, shape, seed, deviation):
    """At the benchmark's sizes (the 16384-cubed case with N(0, 1)/sqrt(K) entries, the 8192 x 28672
    x 8192 up-projection shape with N(0, 0.02)): sampled rows against the oracle, and the whole matrix
    against a bf16 matmul by torch within one rounding."""
    m, n, k = shape
    generator = torch.Generator(device=device).manual_seed(seed)
    deviation = deviation if deviation is not None else 1.0 / math.sqrt(k)
    a = (torch.randn((m, k), generator=generator, device=device) * deviation).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=generator, device=device) * deviation).to(torch.bfloat16)
    c = _run_checked(a, b)
    rows = [0, 4097, m - 1]
    a_words = _to_words(a[rows].contiguous())
    b_words = _to_words(b)
    _, exact = oracle.gemm_rows(a_words, b_words, 0, len(rows), want_f64=True)
    got = oracle.bf16_to_f32(_to_words(c[rows].contiguous())).astype(np.float64)
    bound = 1e-2 * math.sqrt(k) * float(a.abs().max()) * float(b.abs().max())
    assert np.abs(got - exact).max() <= bound
    reference = a @ b.T
    difference = (c.float() - reference.float()).abs().max().item()
    assert difference <= 2 ** -7 * reference.float().abs().max().item()


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable(device):
    """Nothing is starved on purpose in the real kernels: a probe warp waits on a barrier nobody
    arrives on, with a short budget, through the same bounded wait both kernels use."""
    from ferro_kittens_b200._lib import FK_ERR_DEVICE_STALL, check, library

    status = gemm.new_status(device)
    check(library().fk_selftest_stall(torch.cuda.current_stream().cuda_stream, status.data_ptr(), 200_000))
    with pytest.raises(FerroKittensError, match="self-test wait") as error:
        gemm.check_status(status)
    assert error.value.code == FK_ERR_DEVICE_STALL
    words = status.tolist()
    assert words[0] == 0x301 and words[2] == 7 and words[3] == 0
    # The launch returned normally: the same context runs the exact gate right after.
    m, n, k = 512, 256, 256
    a = _to_device(oracle.gemm_stage("a", m, k), device)
    b = _to_device(oracle.gemm_stage("b", n, k), device)
    c = _run_checked(a, b)
    assert oracle.gemm_check_c(_to_words(c), m, n, k)[0] == 0
