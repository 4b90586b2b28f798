"""The CPU oracle against the reference's known answers and the committed fixtures.

Known answers taken from the reference's own sources: the bf16 rounding rule
(examples/src/gemm.rs:444-447), the operand generators and their periods
(:434-440, 544-552), the two check sizes and that the CPU reference of them is
self-consistent under `check_c` (:422-430, 544-578), the attention lattice
(examples/src/flash_forward.rs:326-362) and the properties its seed is built for
(every value bf16-exact, V in [1, 3), outputs in [1, 3), a score ramp on the key axis).
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "golden.json").read_text())


def test_bf16_rounding_is_nearest_even():
    assert oracle.to_bf16(1.0) == 0x3F80
    assert oracle.to_bf16(1.00390625) == 0x3F80      # exactly half way: ties to even (down)
    assert oracle.to_bf16(1.01171875) == 0x3F82      # 1 + 3*2^-8: half way, ties to even (up)
    assert oracle.to_bf16(-2.5) == 0xC020
    for entry in GOLDEN["bf16"]:
        assert oracle.to_bf16(entry["value"]) == entry["bits"]
    values = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    vector = oracle.f32_to_bf16(values)
    assert all(vector[i] == oracle.to_bf16(float(values[i])) for i in range(0, 4096, 37))
    assert (oracle.bf16_to_f32(vector).view(np.uint32) & 0xFFFF == 0).all()


def test_gemm_operands_are_small_integers_with_the_documented_periods():
    a = oracle.bf16_to_f32(oracle.gemm_stage("a", 64, 64))
    b = oracle.bf16_to_f32(oracle.gemm_stage("b", 64, 64))
    assert a.min() == -3 and a.max() == 3 and b.min() == -10 and b.max() == 10
    assert (a == np.round(a)).all() and (b == np.round(b)).all()
    assert (a[7:14] == a[:7]).all() and (b[21:42] == b[:21]).all()
    assert oracle.gemm_a_value(2, 3) == (2 * 5 + 3 * 3) % 7 - 3
    assert oracle.gemm_b_value(5, 2) == (5 * 4 + 2 * 5) % 21 - 10


@pytest.mark.parametrize("k", [64, 256, 1088])
def test_gemm_cell_table_matches_the_fixture(k):
    cells = GOLDEN["gemm"][str(k)]
    for cell in range(7 * 21):
        assert oracle.gemm_expected(cell // 21, cell % 21, k) == cells["bf16"][cell]
        assert oracle.from_bf16(cells["bf16"][cell]) == pytest.approx(cells["exact"][cell], rel=2 ** -8)


@pytest.mark.parametrize("shape", [(512, 256, 256), (768, 1280, 1088)])
def test_gemm_reference_is_self_consistent_and_matches_the_fixture(shape):
    m, n, k = shape
    a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
    c, exact = oracle.gemm_rows(a, b, 0, m, want_f64=True)
    wrong, worst, _ = oracle.gemm_check_c(c, m, n, k)
    assert wrong == 0 and worst < 2 ** -8
    fixture = GOLDEN["gemm"][f"{m}x{n}x{k}"]
    assert hashlib.sha256(a.tobytes()).hexdigest() == fixture["a_sha256"]
    assert hashlib.sha256(b.tobytes()).hexdigest() == fixture["b_sha256"]
    assert hashlib.sha256(c.tobytes()).hexdigest() == fixture["c_sha256"]
    # Integer operands: the fp32 running sum is exact, so it equals the f64 one.
    assert (oracle.f32_to_bf16(exact.astype(np.float32)) == c).all()
    # check_c really is `==`: one flipped bit is one wrong element, found where it is.
    c[5, 9] ^= 1
    assert oracle.gemm_check_c(c, m, n, k)[::2] == (1, 5 * n + 9)


def test_gemm_rows_slab_equals_the_same_rows_of_the_whole():
    rng = np.random.default_rng(1)
    a = oracle.f32_to_bf16(rng.standard_normal((96, 320)).astype(np.float32))
    b = oracle.f32_to_bf16(rng.standard_normal((80, 320)).astype(np.float32))
    whole, whole64 = oracle.gemm_rows(a, b, 0, 96, want_f64=True)
    slab, slab64 = oracle.gemm_rows(a, b, 32, 16, want_f64=True)
    assert (slab == whole[32:48]).all() and (slab64 == whole64[32:48]).all()
    reference = oracle.bf16_to_f32(a).astype(np.float64) @ oracle.bf16_to_f32(b).astype(np.float64).T
    assert np.allclose(whole64, reference, rtol=1e-12, atol=1e-12)
    assert np.abs(oracle.bf16_to_f32(whole) - reference).max() <= np.abs(reference).max() * 2 ** -8 + 1e-4


def test_flash_lattice_has_the_properties_its_seed_is_built_for():
    sequence, heads = GOLDEN["flash"]["sequence"], GOLDEN["flash"]["heads"]
    tensors = {name: oracle.flash_stage(name, sequence, heads) for name in "qkv"}
    for name, words in tensors.items():
        assert hashlib.sha256(words.tobytes()).hexdigest() == GOLDEN["flash"]["inputs_sha256"][name]
    q, k, v = (oracle.bf16_to_f32(tensors[name]) for name in "qkv")
    assert (q[..., 0] == 2.0).all()
    assert (k[..., 0] == np.arange(sequence, dtype=np.float32) / 8.0).all()      # the score ramp
    assert v.min() >= 1.0 and v.max() < 3.0
    assert np.abs(q[..., 1:]).max() <= 1.0 and np.abs(k[..., 1:]).max() <= 1.0
    assert oracle._lib.fko_flash_permutation(2, 1, 5, 7) == (53 + 37 * 5 + (11 + 2 * ((5 + 34) % 63)) * 7 + 142) % 128


def test_flash_rows_match_the_fixture_and_stay_convex():
    sequence, heads, scale = (GOLDEN["flash"][key] for key in ("sequence", "heads", "scale"))
    q, k, v = (oracle.flash_stage(name, sequence, heads) for name in "qkv")
    for entry in GOLDEN["flash"]["rows"]:
        out, lse = oracle.flash_rows(q[entry["head"]], k[entry["head"]], v[entry["head"]], entry["row"], 1,
                                     scale, entry["causal"])
        assert np.allclose(out[0], entry["out"], rtol=1e-12, atol=0)
        assert lse[0] == pytest.approx(entry["lse"], abs=1e-10)
        assert out.min() >= 1.0 and out.max() < 3.0
    first, _ = oracle.flash_rows(q[0], k[0], v[0], 0, 1, scale, True)
    assert np.allclose(first[0], oracle.bf16_to_f32(v[0, 0]))  # row 0 attends key 0 only


def test_flash_rows_agree_with_a_dense_numpy_softmax():
    rng = np.random.default_rng(2)
    q, k, v = (oracle.f32_to_bf16(rng.standard_normal((192, 128)).astype(np.float32)) for _ in range(3))
    for causal in (False, True):
        out, lse = oracle.flash_rows(q, k, v, 0, 192, 128 ** -0.5, causal)
        scores = (oracle.bf16_to_f32(q).astype(np.float64) @ oracle.bf16_to_f32(k).astype(np.float64).T) * 128 ** -0.5
        if causal:
            scores = np.where(np.tril(np.ones_like(scores, dtype=bool)), scores, -np.inf)
        top = scores.max(axis=1, keepdims=True)
        weights = np.exp(scores - top)
        dense = weights @ oracle.bf16_to_f32(v).astype(np.float64) / weights.sum(axis=1, keepdims=True)
        assert np.allclose(out, dense, rtol=1e-10, atol=1e-12)
        assert np.allclose(lse, (top + np.log(weights.sum(axis=1, keepdims=True)))[:, 0], rtol=1e-12)


def test_fp16_rounding_known_answers():
    """`half::f16::from_f32` (examples/src/gemm_sol.rs:1245): round to nearest even, with the
    format's overflow and subnormal edges; and the whole operand range against numpy."""
    cases = {1.0: 0x3C00, -2.0: 0xC000, 65504.0: 0x7BFF, 65519.0: 0x7BFF, 65520.0: 0x7C00, 1e10: 0x7C00,
             2.0 ** -24: 0x0001, 2.0 ** -25: 0x0000, 1.5 * 2.0 ** -24: 0x0002, 2.0 ** -14: 0x0400,
             1.0 + 2.0 ** -11: 0x3C00, 1.0 + 3 * 2.0 ** -11: 0x3C02, 0.0: 0x0000}
    for value, bits in cases.items():
        assert oracle.to_f16(value) == bits, value
    values = np.arange(-10, 11, dtype=np.float32)
    assert [oracle.to_f16(float(v)) for v in values] == list(values.astype(np.float16).view(np.uint16))
    staged = oracle.gemm_stage_f16("b", 32, 64)
    expected = np.array([[oracle.gemm_b_value(r, d) for d in range(64)] for r in range(32)], dtype=np.float16)
    assert np.array_equal(staged, expected.view(np.uint16))


def test_bf16_add_rounds_the_exact_sum_once():
    """What a bf16 reduce-add leaves (src/shared.rs:974-1009): spacing at 256 is 2, ties go to even."""
    word = oracle.to_bf16
    assert oracle.bf16_add(word(1.0), word(1.0)) == word(2.0)
    assert oracle.bf16_add(word(256.0), word(1.0)) == word(256.0)   # 257 ties to the even 256
    assert oracle.bf16_add(word(256.0), word(3.0)) == word(260.0)   # 259 ties to the even 260
    assert oracle.bf16_add(word(258.0), word(1.0)) == word(260.0)
    assert oracle.bf16_add(word(-4.0), word(4.0)) == 0
    assert oracle.bf16_add(word(255.0), word(1.0)) == word(256.0)   # a carry into the exponent
    held = np.array([word(v) for v in (1.0, 256.0, 256.0, -4.0, 255.0, 0.75)], dtype=np.uint16)
    added = np.array([word(v) for v in (1.0, 1.0, 3.0, 4.0, 1.0, 1000.0)], dtype=np.uint16)
    scalar = [oracle.bf16_add(int(h), int(a)) for h, a in zip(held, added)]
    assert list(oracle.bf16_add_words(held, added)) == scalar


def test_row_kernel_seeds_have_the_properties_the_reference_states():
    """examples/src/softmax.rs:12-17 (every row a permutation of the multiples of 1/8 below 16, closed
    form of the answer), examples/src/layernorm.rs:309-312 (no row variance under 835) and :22-26
    (rows of different boost classes have different statistics, so the two norms differ)."""
    words = oracle.softmax_stage(256, 2)
    values = oracle.bf16_to_f32(words)
    for plane in range(2):
        for row in range(0, 256, 5):
            assert sorted(values[plane, row] * 8) == list(range(128))
    reference = oracle.softmax_rows(words)
    for plane, row, column in ((0, 0, 0), (1, 255, 127), (0, 128, 64), (1, 3, 9)):
        assert abs(reference[plane, row, column] / oracle.softmax_expected(plane, row, column) - 1) < 1e-12
    assert abs(reference.sum(axis=-1) - 1).max() < 1e-12
    # The closest pair of outputs of a row is 9.05 % apart (2^(1/8) - 1), far above the 2^-8 tolerance.
    ordered = np.sort(reference[0, 0])
    assert abs((ordered[1:] / ordered[:-1]).min() - 2 ** 0.125) < 1e-9

    x, gamma, beta = oracle.layernorm_stage(384)
    wide = oracle.bf16_to_f32(x).astype(np.float64)
    assert wide.var(axis=1).min() > 835
    assert oracle.from_bf16(int(gamma[64])) == 1.5 and oracle.from_bf16(int(beta[64])) == 3.0
    rows_ = oracle.layernorm_rows(x, gamma, beta, 1e-5)
    by_hand = (wide[7] - wide[7].mean()) / np.sqrt(wide[7].var() + 1e-5) * oracle.bf16_to_f32(gamma) + oracle.bf16_to_f32(beta)
    assert abs(rows_[7] - by_hand).max() < 1e-9
    tiles = oracle.groupnorm_tiles(x, 1e-5)
    for tile in range(3):
        block = wide[128 * tile:128 * tile + 128]
        assert abs(tiles[128 * tile:128 * tile + 128] - (block - block.mean()) / np.sqrt(block.var() + 1e-5)).max() < 1e-9


def test_attention_backward_oracle_matches_float64_autograd():
    """The backward oracle is the textbook derivative of the forward the reference checks against
    (examples/src/flash_forward.rs:419-440); an independent implementation (torch autograd in
    float64) pins it."""
    import torch

    generator = torch.Generator().manual_seed(0)
    for causal in (False, True):
        q, k, v, g = (torch.randn((160, 128), generator=generator).to(torch.bfloat16) for _ in range(4))
        words = lambda t: t.view(torch.int16).numpy().view(np.uint16)  # noqa: E731
        dq, dk, dv = oracle.flash_backward(words(q), words(k), words(v), words(g), 0.125, causal)
        qd, kd, vd = (t.double().requires_grad_() for t in (q, k, v))
        scores = qd @ kd.T * 0.125
        if causal:
            scores = scores.masked_fill(torch.triu(torch.ones(160, 160, dtype=torch.bool), 1), float("-inf"))
        (torch.softmax(scores, dim=-1) @ vd).backward(g.double())
        for mine, theirs in ((dq, qd), (dk, kd), (dv, vd)):
            assert np.abs(mine - theirs.grad.numpy()).max() < 1e-12


def test_exp2_polynomial_stays_inside_the_references_bound():
    """The reference's own test of `exp2_approx` (src/reg.rs:2047-2062) and its doc example (:75-79),
    on the restatement: relative error under 1e-4 from -125 to 125 in steps of 0.137, and the clamp
    that the masked-score sentinel depends on."""
    x = np.float32(-125.0)
    worst = 0.0
    while x <= 125.0:
        approx, exact = oracle.exp2_approx(float(x)), 2.0 ** float(x)
        worst = max(worst, abs((approx - exact) / exact))
        x = np.float32(x + np.float32(0.137))
    assert worst < 1.0e-4
    assert worst > 5.0e-5  # the stated maximum is 7.5e-5: a polynomial far better than that is not the reference's
    assert oracle.exp2_approx(-1.0e30) <= 2.0 ** -124
    assert abs(oracle.exp2_approx(3.5) / 2.0 ** 3.5 - 1.0) < 1.0e-4
