"""The GEMM's two switches for the callers next to the path: fp16 operands (the operand types of
examples/src/gemm_sol.rs, checked the way its `check` does, :1382-1392) and `C += A.B^T` through the
copy engine's reduce-add (src/shared.rs:974-1009). All through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from ferro_kittens_b200 import FerroKittensError, gemm
from ferro_kittens_b200._lib import check, library

pytestmark = pytest.mark.gpu


def _device_words(words: np.ndarray, device, dtype) -> torch.Tensor:
    return torch.from_numpy(words.view(np.int16)).to(device).view(dtype)


def _words(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _run(a, b, c=None, accumulate=False):
    status = gemm.new_status(a.device)
    c = gemm.run(a, b, c, status=status, accumulate=accumulate)
    torch.cuda.synchronize(a.device)
    gemm.check_status(status)
    return c


# gemm_sol::check: every variant at 1024 x 1024 x 512, then the shallow-K gate (:1371-1380).
@pytest.mark.parametrize("shape", [(1024, 1024, 512), (2048, 2048, 256), (2560, 2048, 256), (5120, 2048, 256)])
def test_fp16_operands_are_exact_on_the_reference_gate(device, shape):
    m, n, k = shape
    a = _device_words(oracle.gemm_stage_f16("a", m, k), device, torch.float16)
    b = _device_words(oracle.gemm_stage_f16("b", n, k), device, torch.float16)
    c = _run(a, b)
    wrong, worst, first = oracle.gemm_check_c(_words(c), m, n, k)
    assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"


def test_fp16_operands_random_within_tolerance(device):
    m, n, k = 1024, 768, 1088
    generator = torch.Generator(device="cpu").manual_seed(11)
    a = (torch.rand((m, k), generator=generator) * 2 - 1).to(torch.float16).to(device)
    b = (torch.rand((n, k), generator=generator) * 2 - 1).to(torch.float16).to(device)
    c = _run(a, b)
    reference = a.double() @ b.double().T
    # BASELINE's GEMM bound: 1e-2 * sqrt(K) * max|a| * max|b|.
    assert (c.double() - reference).abs().max().item() <= 1e-2 * k ** 0.5


def test_mixed_operand_types_are_refused(device):
    a = torch.zeros((256, 64), dtype=torch.float16, device=device)
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match="share one element type"):
        gemm.run(a, b)


@pytest.mark.parametrize("operands", ["bf16", "f16"])
def test_accumulate_adds_the_rounded_product_in_bf16(device, operands):
    m, n, k = 1024, 512, 256
    if operands == "bf16":
        a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
        b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    else:
        a = _device_words(oracle.gemm_stage_f16("a", m, k), device, torch.float16)
        b = _device_words(oracle.gemm_stage_f16("b", n, k), device, torch.float16)
    product = np.array([[oracle.gemm_expected(r, c, k) for c in range(21)] for r in range(7)], dtype=np.uint16)
    product = product[np.arange(m)[:, None] % 7, np.arange(n)[None, :] % 21]
    rows, columns = np.meshgrid(np.arange(m), np.arange(n), indexing="ij")
    held = oracle.f32_to_bf16(((rows * 3 + columns * 5) % 37 - 18).astype(np.float32) * 0.75)
    c = _device_words(held.copy(), device, torch.bfloat16)
    _run(a, b, c, accumulate=True)
    once = oracle.bf16_add_words(held, product)
    assert np.array_equal(_words(c), once)
    _run(a, b, c, accumulate=True)
    assert np.array_equal(_words(c), oracle.bf16_add_words(once, product))
    # Spot-check the vectorised expectation against the scalar C restatement.
    for r, col in ((0, 0), (5, 20), (1023, 511), (512, 77)):
        assert once[r, col] == oracle.bf16_add(int(held[r, col]), int(product[r, col]))


def test_accumulate_respects_the_leading_dimension(device):
    m, n, k, ldc = 512, 256, 128, 384
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    whole = torch.full((m, ldc), 2.0, dtype=torch.bfloat16, device=device)
    _run(a, b, whole[:, :n], accumulate=True)
    assert torch.all(whole[:, n:] == 2.0)
    product = np.array([[oracle.gemm_expected(r, c, k) for c in range(21)] for r in range(7)], dtype=np.uint16)
    product = product[np.arange(m)[:, None] % 7, np.arange(n)[None, :] % 21]
    two = np.full((m, n), oracle.to_bf16(2.0), dtype=np.uint16)
    assert np.array_equal(_words(whole[:, :n]), oracle.bf16_add_words(two, product))


def test_unknown_flags_and_missing_c_are_refused(device):
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match="needs the C"):
        gemm.run(a, a, accumulate=True)
    c = torch.zeros((256, 256), dtype=torch.bfloat16, device=device)
    with pytest.raises(FerroKittensError, match="unknown GEMM flags"):
        check(library().fk_gemm(a.data_ptr(), a.data_ptr(), c.data_ptr(), 256, 256, 64, 256, 8, 128,
                                torch.cuda.current_stream().cuda_stream, None))


@pytest.mark.parametrize("with_bias, relu", [(True, False), (False, True), (True, True)])
def test_bias_and_relu_apply_before_the_one_rounding(device, with_bias, relu):
    """The fused epilogue on the integer operands: bias[n] added and max(x, 0) taken on the fp32 value,
    then one rounding -- exact against the oracle's unrounded cells."""
    m, n, k = 1024, 768, 256
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    bias_values = ((np.arange(n) * 7) % 23 - 11).astype(np.float32) * 0.5
    bias = _device_words(oracle.f32_to_bf16(bias_values), device, torch.bfloat16) if with_bias else None
    status = gemm.new_status(device)
    c = gemm.run(a, b, status=status, bias=bias, relu=relu)
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    expected = oracle.gemm_exact(m, n, k)
    if with_bias:
        expected = expected + bias_values[None, :]
    if relu:
        expected = np.maximum(expected, np.float32(0.0))
    assert np.array_equal(_words(c), oracle.f32_to_bf16(expected))
    if relu:
        assert (c.float() >= 0).all() and (c == 0).any()


def test_bias_relu_with_fp16_operands_and_accumulate(device):
    m, n, k = 512, 512, 128
    a = _device_words(oracle.gemm_stage_f16("a", m, k), device, torch.float16)
    b = _device_words(oracle.gemm_stage_f16("b", n, k), device, torch.float16)
    bias_values = ((np.arange(n) * 3) % 13 - 6).astype(np.float32)
    bias = _device_words(oracle.f32_to_bf16(bias_values), device, torch.bfloat16)
    held = oracle.f32_to_bf16(np.full((m, n), 1.5, dtype=np.float32))
    c = _device_words(held.copy(), device, torch.bfloat16)
    status = gemm.new_status(device)
    gemm.run(a, b, c, status=status, accumulate=True, bias=bias, relu=True)
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    fused = oracle.f32_to_bf16(np.maximum(oracle.gemm_exact(m, n, k) + bias_values[None, :], np.float32(0.0)))
    assert np.array_equal(_words(c), oracle.bf16_add_words(held, fused))


def test_bias_guards(device):
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError, match="bias must be"):
        gemm.run(a, a, bias=torch.zeros(128, dtype=torch.bfloat16, device=device))
    with pytest.raises(ValueError, match="bias must be"):
        gemm.run(a, a, bias=torch.zeros(256, dtype=torch.float32, device=device))


# ---- the narrow tile: one CTA per [128, 128] tile (the reference's entry for launches at or below
# ---- half a wave, examples/src/gemm_sol.rs:1063, 1335-1337), asked for by name and chosen by default

@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 256, 256), (1024, 768, 512), (768, 1280, 1088),
                                   (2048, 2048, 256), (4096, 4096, 256),
                                   (1024, 1024, 4096), (512, 768, 2048), (256, 256, 4096), (768, 512, 1088),
                                   (256, 512, 8192)])
def test_narrow_tile_is_exact_on_the_reference_gate(device, shape):
    """One k-block, a ring that wraps (17 k-blocks on 3 stages), more tiles than two CTAs per SM hold
    at once (1024 on 148 SMs); then the shapes whose few tiles are cut along K across a cluster
    (two CTAs for 1024 x 1024 x 4096, four for the 24-tile and the 4-tile launch, two ragged runs of
    9 and 8 k-blocks for K = 1088, four runs of 32 for K = 8192): `==` on bf16 words against the
    reference's integer check."""
    m, n, k = shape
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    status = gemm.new_status(device)
    c = gemm.run(a, b, status=status, tile="narrow")
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
    assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"
    wide = gemm.run(a, b, tile="wide")
    assert torch.equal(c, wide)


def test_narrow_tile_fused_epilogue_fp16_and_accumulate(device):
    m, n, k = 512, 512, 128
    a = _device_words(oracle.gemm_stage_f16("a", m, k), device, torch.float16)
    b = _device_words(oracle.gemm_stage_f16("b", n, k), device, torch.float16)
    bias_values = ((np.arange(n) * 3) % 13 - 6).astype(np.float32)
    bias = _device_words(oracle.f32_to_bf16(bias_values), device, torch.bfloat16)
    held = oracle.f32_to_bf16(np.full((m, n), 1.5, dtype=np.float32))
    c = _device_words(held.copy(), device, torch.bfloat16)
    status = gemm.new_status(device)
    gemm.run(a, b, c, status=status, accumulate=True, bias=bias, relu=True, tile="narrow")
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    fused = oracle.f32_to_bf16(np.maximum(oracle.gemm_exact(m, n, k) + bias_values[None, :], np.float32(0.0)))
    assert np.array_equal(_words(c), oracle.bf16_add_words(held, fused))


def test_narrow_tile_respects_the_leading_dimension(device):
    m, n, k, ldc = 512, 256, 256, 384
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    backing = torch.full((m, ldc), 7.0, dtype=torch.bfloat16, device=device)
    c = backing[:, :n]
    gemm.run(a, b, c, tile="narrow")
    torch.cuda.synchronize(device)
    assert oracle.gemm_check_c(_words(c), m, n, k)[0] == 0
    assert (backing[:, n:] == 7.0).all()


def test_small_shallow_launches_take_the_narrow_tile_by_default(device):
    """Both kernels accumulate a tile's k-blocks in the same order, so their results are equal bit for
    bit and the choice is not observable in the values; what is checked is that the default launch of
    a small, shallow problem is valid and equal to the forced ones, and that the flags are policed."""
    m, n, k = 1024, 1024, 512
    generator = torch.Generator(device="cpu").manual_seed(17)
    a = (torch.rand((m, k), generator=generator) * 2 - 1).to(torch.bfloat16).to(device)
    b = (torch.rand((n, k), generator=generator) * 2 - 1).to(torch.bfloat16).to(device)
    default, narrow, wide = gemm.run(a, b), gemm.run(a, b, tile="narrow"), gemm.run(a, b, tile="wide")
    reference = a.double() @ b.double().T
    for c in (default, narrow, wide):
        assert (c.double() - reference).abs().max().item() <= 1e-2 * k ** 0.5
    assert torch.equal(default, narrow)
    with pytest.raises(ValueError, match="tile is None"):
        gemm.run(a, b, tile="tall")
    with pytest.raises(FerroKittensError, match="both asked for"):
        check(library().fk_gemm(a.data_ptr(), b.data_ptr(), default.data_ptr(), m, n, k, n, 8, 8 | 16,
                                torch.cuda.current_stream().cuda_stream, None))


# ---- items narrower than 256 columns: the wide kernel's [512, 224] and [512, 192] items, which fill the
# ---- waves of launches whose [512, 256] tile count sits just past a whole number of waves

def _run_tiled(a, b, c, columns, flags=0, bias=None, group=gemm.GROUP):
    m, k = a.shape
    n = b.shape[0]
    status = gemm.new_status(a.device)
    maps = gemm.TiledMaps(a, b, c, columns=columns)
    gemm.launch_tiled(maps, m, n, k, group, status, flags=flags | gemm.TILE_WIDE, bias=bias)
    torch.cuda.synchronize(a.device)
    gemm.check_status(status)
    return c


@pytest.mark.parametrize("shape, columns", [((1024, 1792, 512), 224), ((768, 1792, 320), 224), ((1024, 1536, 512), 192),
                                            ((4096, 3584, 256), 224), ((2560, 1536, 256), 192), ((512, 5376, 1088), 224),
                                            ((4608, 5376, 128), 192), ((1024, 1792, 512), 256)])
@pytest.mark.parametrize("group", [8, 3])
def test_narrower_items_are_exact_on_the_reference_gate(device, shape, columns, group):
    """One item per cluster and several (the last one's passes are staged together), ragged tile rows,
    a K that wraps the ring: every width the launch can choose, forced here, on the integer gate."""
    m, n, k = shape
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    c = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=device)
    _run_tiled(a, b, c, columns, group=group)
    wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
    assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"


@pytest.mark.parametrize("columns", [224, 192])
def test_narrower_items_fused_epilogue_leading_dimension_and_accumulate(device, columns):
    """Bias (read per 32-column pass, never past column n), ReLU, a padded C whose margin stays
    untouched, fp16 operands, and the reduce-add through both store maps."""
    m, n, k = 1024, 5376, 256  # 21 x 256 = 24 x 224 = 28 x 192 columns
    a = _device_words(oracle.gemm_stage_f16("a", m, k), device, torch.float16)
    b = _device_words(oracle.gemm_stage_f16("b", n, k), device, torch.float16)
    bias_values = ((np.arange(n) * 7) % 23 - 11).astype(np.float32) * 0.5
    bias = _device_words(oracle.f32_to_bf16(bias_values), device, torch.bfloat16)
    wide = torch.full((m, n + 64), 7.0, dtype=torch.bfloat16, device=device)
    c = wide[:, :n]
    _run_tiled(a, b, c, columns, flags=gemm.F16_OPERANDS | gemm.RELU, bias=bias)
    fused = oracle.f32_to_bf16(np.maximum(oracle.gemm_exact(m, n, k) + bias_values[None, :], np.float32(0.0)))
    assert np.array_equal(_words(c), fused)
    assert (wide[:, n:] == 7.0).all()
    _run_tiled(a, b, c, columns, flags=gemm.F16_OPERANDS | gemm.RELU | gemm.ACCUMULATE, bias=bias)
    assert np.array_equal(_words(c), oracle.bf16_add_words(fused, fused))
    assert (wide[:, n:] == 7.0).all()


def test_the_launch_chooses_the_width_that_fills_its_waves(device):
    """8192 x 3584 is 224 tiles of [512, 256]: three waves of 74 clusters and two tiles over. The entries
    that build their own maps take 256 items of [512, 224] instead; same answer, bit for bit, as the
    256-column items give."""
    m, n, k = 8192, 3584, 256
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    if sms == 148:
        assert gemm.item_columns(m, n, k, device) == 224
        assert gemm.item_columns(m, 8 * n, k, device) == 256
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    c = _run(a, b)
    wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
    assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"
    generator = torch.Generator(device=device).manual_seed(3)
    a = (torch.randn((m, 1024), generator=generator, device=device) * 0.05).to(torch.bfloat16)
    b = (torch.randn((n, 1024), generator=generator, device=device) * 0.05).to(torch.bfloat16)
    chosen = _run(a, b)
    plain = _run_tiled(a, b, torch.empty_like(chosen), 256)
    assert torch.equal(chosen, plain)


def test_widths_the_kernel_does_not_have_are_refused(device):
    a = torch.zeros((1024, 64), dtype=torch.bfloat16, device=device)
    b = torch.zeros((1792, 64), dtype=torch.bfloat16, device=device)
    c = torch.zeros((1024, 1792), dtype=torch.bfloat16, device=device)
    maps = gemm.TiledMaps(a, b, c, columns=224)
    with pytest.raises(FerroKittensError, match="takes the narrow kernel"):
        gemm.launch_tiled(maps, 1024, 1792, 64)
    maps.columns = 208
    with pytest.raises(FerroKittensError, match="256, 224 or 192 columns wide"):
        gemm.launch_tiled(maps, 1024, 1792, 64, flags=gemm.TILE_WIDE)
    maps.columns = 192
    with pytest.raises(FerroKittensError, match="do not divide"):
        gemm.launch_tiled(maps, 1024, 1792, 64, flags=gemm.TILE_WIDE)
    maps.columns, maps.c_tail = 224, None
    with pytest.raises(FerroKittensError, match="a map of their own"):
        gemm.launch_tiled(maps, 1024, 1792, 64, flags=gemm.TILE_WIDE)


# ---- launches of more items than resident clusters: one cluster per item in the grid, handed out through
# ---- cluster launch control by the leader CTA's feed warp

@pytest.mark.parametrize("shape", [(8192, 8192, 64), (4352, 4096, 128), (2048, 14336, 192), (16384, 4096, 64),
                                   (8192, 8192, 2048)])
@pytest.mark.parametrize("group", [6, 1])
def test_items_handed_out_by_the_feed_are_exact(device, shape, group):
    """A k-block or two per item (the feed forced on launches it would not choose), so that a cluster
    runs through items as fast as the feed can claim them (512 to 1024 items on 74 clusters), a
    ragged last tile row, a width the launch chooses, and a launch that is fed unasked: every tile
    must be computed exactly once, whichever cluster took it."""
    m, n, k = shape
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    c = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=device)
    status = gemm.new_status(device)
    for _ in range(3):
        c.fill_(-3.0)
        gemm.run(a, b, c, group=group, status=status, tile="wide", order="feed" if k < 2048 else None)
        torch.cuda.synchronize(device)
        gemm.check_status(status)
        wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
        assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"


@pytest.mark.parametrize("columns", [224, 192])
def test_narrower_items_under_the_feed(device, columns):
    """Both choices at once: items of 224 / 192 columns handed out through cluster launch control,
    a ragged last tile row, twice in a row."""
    m, n, k = 7936, 5376, 128
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    c = torch.full((m, n), -3.0, dtype=torch.bfloat16, device=device)
    for _ in range(2):
        c.fill_(-3.0)
        _run_tiled(a, b, c, columns, flags=gemm.ORDER_FEED)
        wrong, _, first = oracle.gemm_check_c(_words(c), m, n, k)
        assert wrong == 0, f"{wrong} of {m * n} wrong, first at {first}"


def test_the_static_order_gives_the_same_words(device):
    m, n, k = 8192, 4096, 2048
    generator = torch.Generator(device=device).manual_seed(9)
    a = (torch.randn((m, k), generator=generator, device=device) * 0.05).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=generator, device=device) * 0.05).to(torch.bfloat16)
    fed = gemm.run(a, b, order="feed")
    static = gemm.run(a, b, order="static")
    assert torch.equal(fed, static)
    with pytest.raises(FerroKittensError, match="both asked for"):
        check(library().fk_gemm(a.data_ptr(), b.data_ptr(), fed.data_ptr(), m, n, k, n, 6, 96,
                                torch.cuda.current_stream().cuda_stream, None))


def test_fed_launches_back_to_back_stay_clean(device):
    """A few hundred fed launches in a row over three shapes (items of one k-block to 64): no wait runs
    out, and every C equals the static order's bit for bit."""
    cases = []
    for m, n, k in [(8192, 8192, 64), (4096, 8192, 1024), (8192, 4096, 4096)]:
        generator = torch.Generator(device=device).manual_seed(m + k)
        a = (torch.randn((m, k), generator=generator, device=device) / k ** 0.5).to(torch.bfloat16)
        b = (torch.randn((n, k), generator=generator, device=device) / k ** 0.5).to(torch.bfloat16)
        cases.append((a, b, gemm.run(a, b, tile="wide", order="static")))
    status = gemm.new_status(device)
    for _ in range(12):
        for a, b, expected in cases:
            c = torch.empty_like(expected)
            for _ in range(8):
                gemm.run(a, b, c, status=status, tile="wide", order="feed")
            gemm.check_status(status)
            assert torch.equal(c, expected)


def test_accumulate_under_the_feed_adds_every_tile_once(device):
    """C += A.B^T with more items than clusters: a tile taken twice, or dropped, shows in the sum."""
    m, n, k = 4096, 8192, 64
    a = _device_words(oracle.gemm_stage("a", m, k), device, torch.bfloat16)
    b = _device_words(oracle.gemm_stage("b", n, k), device, torch.bfloat16)
    c = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    status = gemm.new_status(device)
    gemm.run(a, b, c, status=status, accumulate=True, order="feed")
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    once = _words(c).copy()
    assert oracle.gemm_check_c(once, m, n, k)[0] == 0
    gemm.run(a, b, c, status=status, accumulate=True, order="feed")
    torch.cuda.synchronize(device)
    gemm.check_status(status)
    assert np.array_equal(_words(c), oracle.bf16_add_words(once, once))
