"""The transition oracle against the golden vectors produced by the reference's
own PyTorch module (tests/models/boltz2/test_transition_forward.py:11-33, run by
tests/golden/make_golden.py), at the reference's tolerance of 1e-5."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import load_transition_golden
from oracle import triangle_oracle as orc


@pytest.mark.parametrize("name", ["transition_d5_h11.npz", "transition_d128_h512.npz"])
def test_transition_matches_reference_module(name):
    params, x, outs = load_transition_golden(name)
    got = orc.transition(params, x, dtype="float64")
    np.testing.assert_allclose(got, outs["whole"], rtol=1e-5, atol=1e-5)
    # the reference's hidden-chunked accumulation is the same sum in another order
    np.testing.assert_allclose(got, outs["chunked"], rtol=2e-5, atol=2e-5)
    got32 = orc.transition(params, x, dtype="float32")
    np.testing.assert_allclose(got32, outs["whole"], rtol=2e-5, atol=2e-5)


def test_bf16_emulation_stays_close_to_truth():
    rng = np.random.default_rng(5)
    params = orc.round_params(orc.random_transition_params(rng, ln_noise=0.1), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((40, 128)).astype(np.float32))
    truth = orc.transition(params, x, dtype="float64")
    emu = orc.transition(params, x, dtype="bfloat16")
    err = orc.error_vs(truth, emu)
    assert err["mean_abs_over_rms"] < 5e-3 and err["max_abs_over_rms"] < 5e-2


def test_rows_are_independent():
    """The op is row-local (what lets a context-parallel rank run it on its own tile)."""
    rng = np.random.default_rng(6)
    params = orc.random_transition_params(rng)
    x = rng.standard_normal((3, 7, 128))
    whole = orc.transition(params, x)
    for i in range(3):
        np.testing.assert_allclose(orc.transition(params, x[i]), whole[i], rtol=1e-12, atol=1e-12)
