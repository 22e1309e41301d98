"""The oracle against the golden vectors produced by the reference's own
PyTorch restatements (tests/golden/make_golden.py), plus the properties the
reference's tests assert about these ops."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import load_triatt_golden, load_trimul_golden
from oracle import triangle_oracle as orc


@pytest.mark.parametrize("name", ["trimul_n7_c8.npz", "trimul_n12_c128.npz"])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_trimul_matches_reference_restatement(name, direction):
    params, x, mask, outs = load_trimul_golden(name)
    got = orc.triangle_multiplication(params, x, mask, direction, dtype="float64")
    # the reference accepts 2e-4 between its jnp path and this restatement
    np.testing.assert_allclose(got, outs[direction], rtol=2e-4, atol=2e-4)
    got32 = orc.triangle_multiplication(params, x, mask, direction, dtype="float32")
    np.testing.assert_allclose(got32, outs[direction], rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("name", ["triatt_n7_c8.npz", "triatt_n12_c128.npz"])
@pytest.mark.parametrize("starting", [True, False])
def test_triatt_matches_reference_restatement(name, starting):
    params, x, mask, outs = load_triatt_golden(name)
    # Rows of the attention with no valid key hold "-1e9 absorbed in fp32" garbage
    # in the reference (it depends on fp32 rounding of -1e9 + score), so they are
    # compared in fp32 only; everything else also against the fp64 truth.
    has_key = mask.any(axis=2) if starting else mask.any(axis=1)  # [B, N] per attention row
    valid = has_key[:, :, None] if starting else has_key[:, None, :]
    valid = np.broadcast_to(valid[..., None], outs[starting].shape)
    got = orc.triangle_attention(params, x, mask, starting=starting, dtype="float64")
    np.testing.assert_allclose(got[valid], outs[starting][valid], rtol=3e-4, atol=3e-4)
    got32 = orc.triangle_attention(params, x, mask, starting=starting, dtype="float32")
    np.testing.assert_allclose(got32, outs[starting], rtol=3e-4, atol=3e-4)


def test_directions_differ_on_unstructured_input():
    """A symmetric input hides a transposed contraction; the golden input is a
    seeded normal draw, so the two directions must disagree."""
    _, _, _, outs = load_trimul_golden("trimul_n12_c128.npz")
    assert np.abs(outs["outgoing"] - outs["incoming"]).max() > 1e-3


def test_ending_node_is_starting_node_on_transposed_input():
    params, x, mask, _ = load_triatt_golden("triatt_n7_c8.npz")
    end = orc.triangle_attention(params, x, mask, starting=False)
    start_t = orc.triangle_attention(params, np.swapaxes(x, 1, 2), np.swapaxes(mask, 1, 2), starting=True)
    np.testing.assert_allclose(end, np.swapaxes(start_t, 1, 2), rtol=1e-12, atol=1e-12)


def test_incoming_is_outgoing_of_transposed_operands():
    rng = np.random.default_rng(5)
    a = rng.standard_normal((6, 6, 4))
    b = rng.standard_normal((6, 6, 4))
    inc = orc.triangle_contraction(a, b, "incoming")
    out = orc.triangle_contraction(np.swapaxes(a, 0, 1), np.swapaxes(b, 0, 1), "outgoing")
    np.testing.assert_allclose(inc, out, rtol=1e-12, atol=1e-12)


def test_fully_masked_row_is_uniform_average():
    """XLA-path convention: the -1e9 constant absorbs the scores in fp32, so a
    row with no valid key becomes a uniform softmax over every key."""
    rng = np.random.default_rng(3)
    b, n, h, d = 1, 5, 2, 4
    q = rng.standard_normal((b, n, h, n, d)).astype(np.float32)
    k = rng.standard_normal((b, n, h, n, d)).astype(np.float32)
    v = rng.standard_normal((b, n, h, n, d)).astype(np.float32)
    tb = rng.standard_normal((b, 1, h, n, n)).astype(np.float32)
    mask = np.ones((b, n, n), dtype=np.float32)
    mask[0, 2, :] = 0.0
    mb = (np.float32(1e9) * (mask - 1.0))[:, :, None, None, :]
    out = orc.attention_core(q, k, v, tb, mb, dtype="float32")
    np.testing.assert_allclose(out[0, 2], np.broadcast_to(v[0, 2].mean(axis=-2, keepdims=True), out[0, 2].shape),
                               rtol=1e-5, atol=1e-5)


def test_bf16_emulation_stays_close_to_truth():
    rng = np.random.default_rng(0)
    n = 24
    params = orc.round_params(orc.random_trimul_params(rng, ln_noise=0.1), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = orc.pad_mask(n, 3)
    truth = orc.triangle_multiplication(params, x, mask, "outgoing", dtype="float64")
    emu = orc.triangle_multiplication(params, x, mask, "outgoing", dtype="bfloat16")
    err = orc.error_vs(truth, emu)
    # the reference's own bf16 path sits about 5e-3 (mean) from the fp64 truth
    assert err["max_abs_over_rms"] < 1e-1 and 1e-3 < err["mean_abs_over_rms"] < 1e-2, err


def test_layer_norm_rounds_before_affine_in_bf16():
    rng = np.random.default_rng(1)
    x = orc.round_bf16(rng.standard_normal((4, 128)).astype(np.float32))
    scale = orc.round_bf16(1.0 + 0.1 * rng.standard_normal(128).astype(np.float32))
    bias = orc.round_bf16(0.1 * rng.standard_normal(128).astype(np.float32))
    y = orc.layer_norm(x, scale, bias, 1e-5, dtype="bfloat16")
    assert np.array_equal(y, orc.round_bf16(y))  # output is representable in bf16
    y64 = orc.layer_norm(x, scale, bias, 1e-5, dtype="float64")
    assert np.abs(y - y64).max() < 0.05


def test_q_scale_division_equals_multiplication_by_the_rounded_reciprocal():
    """The projection kernel scales q by multiplying with fl(1 / bf16(sqrt 32)) instead of
    dividing; for every finite bf16 input both give the same bf16 result (the divisor is
    181/32, so an exact quotient is never within fp32 rounding error of a bf16 boundary)."""
    import ml_dtypes

    x = np.arange(0, 1 << 16, dtype=np.uint16).view(ml_dtypes.bfloat16).astype(np.float32)
    x = x[np.isfinite(x)]
    y = np.float32(np.float32(np.sqrt(np.float32(32.0))).astype(ml_dtypes.bfloat16))
    assert float(y) == 181.0 / 32.0
    inv = np.float32(1.0) / y
    div = (x / y).astype(np.float32).astype(ml_dtypes.bfloat16).view(np.uint16)
    mul = (x * inv).astype(np.float32).astype(ml_dtypes.bfloat16).view(np.uint16)
    assert np.array_equal(div, mul)


@pytest.mark.parametrize("dtype", ["float64", "bfloat16"])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_sampled_trimul_elements_equal_the_full_restatement(direction, dtype):
    """The element-sampling form used for the large GPU cases is the same arithmetic."""
    rng = np.random.default_rng(31)
    n = 40
    params = orc.round_params(orc.random_trimul_params(rng, ln_noise=0.1, std=0.05), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = orc.pad_mask(n, 3)
    full = orc.triangle_multiplication(params, x, mask, direction, dtype=dtype)[0]
    rows, cols = np.array([0, 17, 38]), np.array([1, 5, 22, 39])
    xt, mt = (x[0], mask[0]) if direction == "outgoing" else (x[0].transpose(1, 0, 2), mask[0].T)
    got = orc.triangle_multiplication_sampled(params, xt[rows], mt[rows], xt[cols], mt[cols],
                                              x[0][np.ix_(rows, cols)], dtype=dtype)
    ref = full[np.ix_(rows, cols)]
    if dtype == "float64":
        np.testing.assert_allclose(got, ref, rtol=1e-10, atol=1e-12)
    else:  # a different summation order inside BLAS may flip isolated bf16 roundings
        assert np.mean(got == ref) > 0.98
        np.testing.assert_allclose(got, ref, rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("dtype", ["float64", "bfloat16"])
@pytest.mark.parametrize("starting", [True, False])
def test_sampled_triatt_elements_equal_the_full_restatement(starting, dtype):
    rng = np.random.default_rng(32)
    n = 36
    params = orc.round_params(orc.random_triatt_params(rng, ln_noise=0.1, std=0.05), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = orc.pad_mask(n, 4)
    full = orc.triangle_attention(params, x, mask, starting=starting, dtype=dtype)[0]
    rows, cols = np.array([0, 9, 30]), np.array([2, 3, 19, 31])
    xt, mt = (x[0], mask[0]) if starting else (x[0].transpose(1, 0, 2), mask[0].T)
    got = orc.triangle_attention_sampled(params, xt[rows], mt[rows], xt[cols], cols, dtype=dtype)
    ref = full[np.ix_(rows, cols)] if starting else full[np.ix_(cols, rows)].transpose(1, 0, 2)
    if dtype == "float64":
        np.testing.assert_allclose(got, ref, rtol=1e-9, atol=1e-11)
    else:
        assert np.mean(got == ref) > 0.97
        np.testing.assert_allclose(got, ref, rtol=2e-2, atol=1e-3)


def test_block_variants_of_the_other_model_families():
    """pair_gate (Protenix), mask_transition (OpenFold3) and attention_first on the block
    restatement: the gate zeroes dropped pairs and gated tokens and, with a mask that is not an
    outer product, changes kept pairs too (a dropped pair's bias no longer reaches the rows that
    keep its key); the masked transition only changes dropped pairs; the order matters."""
    rng = np.random.default_rng(0)
    params = orc.random_pairformer_params(rng, c_s=48, heads_s=2, ln_noise=0.1)
    n = 12
    z = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    s = rng.standard_normal((1, n, 48)).astype(np.float32)
    pair_mask = orc.pad_mask(n, 3).copy()
    pair_mask[0, 1, 2] = 0.0
    pair_mask[0, 4, 0] = 0.0
    keep = pair_mask[0] == 1
    s0, z0 = orc.pairformer_layer(params, s, z, None, pair_mask, dtype="float32")
    s1, z1 = orc.pairformer_layer(params, s, z, None, pair_mask, dtype="float32", pair_gate=True)
    assert np.all(z1[0][~keep] == 0.0) and np.all(s1[0][n - 3:] == 0.0)
    assert np.abs(z1 - z0)[0][keep].max() > 1e-4
    _, z2 = orc.pairformer_layer(params, s, z, None, pair_mask, dtype="float32", mask_transition=True)
    assert np.abs(z2 - z0)[0][keep].max() == 0.0 and np.abs(z2 - z0)[0][~keep].max() > 1e-4
    _, z3 = orc.pairformer_layer(params, s, z, None, pair_mask, dtype="float32", attention_first=True)
    assert np.abs(z3 - z0).max() > 1e-4
    # with an all-ones mask the gate and the masked transition are no-ops
    ones = np.ones_like(pair_mask)
    a = orc.pairformer_layer(params, s, z, None, ones, dtype="float32")
    b = orc.pairformer_layer(params, s, z, None, ones, dtype="float32", pair_gate=True, mask_transition=True)
    assert np.array_equal(a[1], b[1]) and np.array_equal(a[0], b[0])
