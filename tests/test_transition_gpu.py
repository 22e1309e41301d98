"""GPU parity of the pair transition against the oracle, through the C ABI.

bf16 tolerance as stated by the benchmark (conftest.assert_parity): mean-abs <=
2e-3 and max-abs <= 2e-2 of the output RMS against the oracle's bf16 emulation.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import assert_parity, load_transition_golden
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _case(seed, shape, std=0.05, ln_noise=0.1, hidden_mult=4):
    rng = np.random.default_rng(seed)
    params = orc.round_params(orc.random_transition_params(rng, expansion=hidden_mult, std=std, ln_noise=ln_noise), "bfloat16")
    x = orc.round_bf16(rng.standard_normal(shape + (128,)).astype(np.float32))
    return params, x


@pytest.mark.parametrize("shape", [(1, 1), (5, 7), (1, 128), (3, 200), (40, 40), (129, 130)])
def test_matches_bf16_emulation(cuda_device, shape):
    from foldjax_b200.transition import transition_forward
    from foldjax_b200 import _lib

    params, x = _case(sum(shape), shape)
    got = transition_forward(params, x)
    _lib.device_status()
    assert got.shape == x.shape and np.isfinite(got).all()
    ref = orc.transition(params, x, dtype="bfloat16")
    assert_parity(ref, got, label=f"transition {shape}")
    truth = orc.transition(params, x, dtype="float64")
    err = orc.error_vs(truth, got)
    assert err["mean_abs_over_rms"] < 6e-3, err


def test_golden_case_at_kernel_width(cuda_device):
    """The reference module's own output (fp32) for bf16-rounded inputs and weights."""
    from foldjax_b200.transition import transition_forward

    params, x, outs = load_transition_golden("transition_d128_h512.npz")
    params = orc.round_params(params, "bfloat16")
    xb = orc.round_bf16(x)
    got = transition_forward(params, xb)
    truth = orc.transition(params, xb, dtype="float64")
    err = orc.error_vs(truth, got)
    assert err["mean_abs_over_rms"] < 6e-3 and err["max_abs_over_rms"] < 6e-2, err
    # bf16 rounding of inputs and weights moves the fp32 golden output by less than this
    err_g = orc.error_vs(outs["whole"], got)
    assert err_g["mean_abs_over_rms"] < 2e-2, err_g


@pytest.mark.parametrize("hidden_mult", [1, 2, 4])
def test_other_hidden_widths(cuda_device, hidden_mult):
    from foldjax_b200.transition import transition_forward

    params, x = _case(90 + hidden_mult, (9, 33), hidden_mult=hidden_mult)
    got = transition_forward(params, x)
    assert_parity(orc.transition(params, x, dtype="bfloat16"), got, label=f"hidden {128 * hidden_mult}")


def test_fused_residual_in_place_and_determinism(cuda_device):
    from foldjax_b200.transition import transition_forward
    from foldjax_b200 import _device as dev

    params, x = _case(17, (20, 150))
    pd = dev.params_to_device(params)
    xd = dev.to_device(x, torch.bfloat16)
    upd = transition_forward(pd, xd)
    again = transition_forward(pd, xd)
    assert torch.equal(upd, again)
    expect = (xd.float() + upd.float()).to(torch.bfloat16)
    z = xd.clone()
    out = transition_forward(pd, z, residual=z, out=z)  # z += transition(z)
    assert out.data_ptr() == z.data_ptr()
    assert torch.equal(z, expect)


def test_large_case_properties(cuda_device):
    """512 x 512 pairs (larger than one wave of tiles): finite, rows independent of
    their position in the batch, same result as the same rows run alone."""
    from foldjax_b200.transition import transition_forward
    from foldjax_b200 import _device as dev

    params, x = _case(23, (512, 512), std=0.02, ln_noise=0.0)
    pd = dev.params_to_device(params)
    xd = dev.to_device(x, torch.bfloat16)
    full = transition_forward(pd, xd)
    assert torch.isfinite(full.float()).all()
    part = transition_forward(pd, xd[100:103].contiguous())
    assert torch.equal(part, full[100:103])
    ref = orc.transition(params, x[100:103], dtype="bfloat16")
    assert_parity(ref, part.float().cpu().numpy(), label="rows 100..102 of 512x512")


def test_masked_update(cuda_device):
    """mask= multiplies the update row by row before the residual add (OpenFold3's masked
    transition): dropped rows come back as the residual, kept rows as without a mask - bit for
    bit, since a 0/1 mask multiplies exactly."""
    from foldjax_b200.transition import transition_forward

    params, x = _case(17, (9, 150))
    rng = np.random.default_rng(3)
    mask = (rng.random((9, 150)) > 0.3).astype(np.float32)
    plain = transition_forward(params, x, residual=x)
    masked = transition_forward(params, x, residual=x, mask=mask)
    keep = mask.astype(bool)
    assert np.array_equal(masked[keep], plain[keep])
    assert np.array_equal(masked[~keep], x[~keep])
    update_only = transition_forward(params, x, mask=mask)
    assert np.all(update_only[~keep] == 0.0) and np.array_equal(update_only[keep], transition_forward(params, x)[keep])
    with pytest.raises(ValueError, match="one value per row"):
        transition_forward(params, x, mask=mask[:, :100])


def test_rejects_bad_arguments(cuda_device):
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.transition import transition_forward

    params, x = _case(3, (2, 2))
    with pytest.raises(ValueError, match="chunk_size must be positive"):
        transition_forward(params, x, chunk_size=0)
    with pytest.raises(ValueError, match="128-channel"):
        transition_forward(params, np.zeros((4, 64), dtype=np.float32))
    lib = _lib.load()
    xd = dev.to_device(x, torch.bfloat16)
    args = _lib.PairTransitionArgs(rows=4, channels=128, hidden=100, eps=1e-5, x=xd.data_ptr(), out=xd.data_ptr(),
                                   norm_scale=xd.data_ptr(), norm_bias=xd.data_ptr(), fc1=xd.data_ptr(),
                                   fc2=xd.data_ptr(), fc3=xd.data_ptr(), residual=None, workspace=xd.data_ptr(),
                                   workspace_bytes=1 << 30)
    assert lib.b200tri_pair_transition(C.byref(args), C.c_void_p(dev.stream_ptr())) == _lib.ERR_UNSUPPORTED
    assert b"multiple of 64" in lib.b200tri_last_error()
    args.hidden = 512
    args.workspace_bytes = 16
    assert lib.b200tri_pair_transition(C.byref(args), C.c_void_p(dev.stream_ptr())) == _lib.ERR_WORKSPACE
