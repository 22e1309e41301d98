"""The single-track attention oracle against the golden vectors produced by the
reference's own PyTorch restatement (tests/models/boltz2/
test_attention_checkpoint_parity.py:109-148, run by tests/golden/make_golden.py), at
the reference's tolerance of 2e-4."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import load_attention_pair_bias_golden
from oracle import triangle_oracle as orc


@pytest.mark.parametrize("name", ["attention_pair_bias_n7.npz", "attention_pair_bias_n12_c96.npz"])
def test_matches_reference_restatement(name):
    params, s, k_in, z, mask, out = load_attention_pair_bias_golden(name)
    got = orc.attention_pair_bias(params, s, z, mask, k_in=k_in, dtype="float64")
    np.testing.assert_allclose(got, out, rtol=2e-4, atol=2e-4)
    got32 = orc.attention_pair_bias(params, s, z, mask, k_in=k_in, dtype="float32")
    np.testing.assert_allclose(got32, out, rtol=2e-4, atol=2e-4)


def test_masked_keys_have_no_weight_and_k_in_defaults_to_s():
    rng = np.random.default_rng(2)
    params = orc.random_attention_pair_bias_params(rng, c_s=48, c_z=16, heads=2, std=0.3)
    s = rng.standard_normal((1, 6, 48))
    z = rng.standard_normal((1, 6, 6, 16))
    mask = np.array([[1, 1, 0, 1, 0, 1]], dtype=np.float64)
    base = orc.attention_pair_bias(params, s, z, mask)
    np.testing.assert_allclose(base, orc.attention_pair_bias(params, s, z, mask, k_in=s), rtol=0, atol=0)
    # changing a masked key's features or its pair bias column changes nothing
    k2 = s.copy()
    k2[0, 2] += 5.0
    z2 = z.copy()
    z2[0, :, 4] -= 3.0
    np.testing.assert_allclose(orc.attention_pair_bias(params, s, z2, mask, k_in=k2)[:, :, :], base, rtol=1e-9, atol=1e-9)


def test_has_no_bf16_mode():
    rng = np.random.default_rng(3)
    params = orc.random_attention_pair_bias_params(rng, c_s=24, c_z=8, heads=1)
    with pytest.raises(ValueError, match="float32 in the reference"):
        orc.attention_pair_bias(params, np.zeros((1, 2, 24)), np.zeros((1, 2, 2, 8)), np.ones((1, 2)), dtype="bfloat16")
