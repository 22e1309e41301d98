"""float32 mode of the two triangle ops on the GPU, through the C ABI (dtype = F32).

Tolerance: the benchmark's float32 bar, max-abs error <= 1e-4, against the oracle in
float32 (the reference's float32 trunk) and in float64; and the reference's own torch
restatements (the golden vectors) at the tolerance its tests use for jnp == torch
(2e-4 for the multiplicative update, 3e-4 for the attention).
"""

from __future__ import annotations

import numpy as np
import pytest

from conftest import load_triatt_golden, load_trimul_golden
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

F32_TOL = 1e-4


def _max_abs(ref, got):
    return float(np.max(np.abs(np.asarray(ref, np.float64) - np.asarray(got, np.float64))))


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_config1_triangle_multiplication_fp32(cuda_device, direction):
    """Benchmark config 1: N = 256, c_z = c = 128, float32, all-ones mask, seed 0."""
    from foldjax_b200 import _lib
    from foldjax_b200.triangle import triangle_multiplication_forward

    rng = np.random.default_rng(0)
    n = 256
    params = orc.random_trimul_params(rng)
    x = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    mask = np.ones((1, n, n), np.float32)
    got = triangle_multiplication_forward(params, x, mask, direction, dtype="float32")
    _lib.device_status()
    assert got.dtype == np.float32 and got.shape == x.shape
    ref32 = orc.triangle_multiplication(params, x, mask, direction, dtype="float32")
    ref64 = orc.triangle_multiplication(params, x, mask, direction, dtype="float64")
    e32, e64 = _max_abs(ref32, got), _max_abs(ref64, got)
    print(f"tri-mult {direction} fp32 N=256: max-abs vs float32 oracle {e32:.2e}, vs float64 {e64:.2e}, "
          f"output rms {np.sqrt(np.mean(ref64 ** 2)):.3e}")
    assert e32 <= F32_TOL and e64 <= F32_TOL


@pytest.mark.parametrize("n,n_pad", [(40, 0), (100, 7), (192, 12)])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_triangle_multiplication_fp32_masked_and_ragged(cuda_device, n, n_pad, direction):
    from foldjax_b200.triangle import triangle_multiplication_forward

    rng = np.random.default_rng(n)
    params = orc.random_trimul_params(rng, ln_noise=0.1, std=0.05)
    x = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    mask = orc.pad_mask(n, n_pad) * (rng.random((1, n, n)) > 0.1)
    got = triangle_multiplication_forward(params, x, mask.astype(np.float32), direction, dtype="float32")
    ref = orc.triangle_multiplication(params, x, mask, direction, dtype="float64")
    # outputs here are O(1); the bar is relative to their scale
    scale = max(1.0, float(np.abs(ref).max()))
    assert _max_abs(ref, got) <= F32_TOL * scale, (_max_abs(ref, got), scale)
    res = triangle_multiplication_forward(params, x, mask.astype(np.float32), direction, dtype="float32", residual=x)
    np.testing.assert_allclose(res, x + got, rtol=0, atol=1e-6)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_trimul_golden_vectors_fp32(cuda_device, direction):
    from foldjax_b200.triangle import triangle_multiplication_forward

    params, x, mask, outs = load_trimul_golden("trimul_n12_c128.npz")
    got = triangle_multiplication_forward(params, x, mask, direction, dtype="float32")
    np.testing.assert_allclose(got, outs[direction], rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("starting", [True, False])
def test_triatt_golden_vectors_fp32(cuda_device, starting):
    from foldjax_b200.triangle_attention import triangle_attention_forward

    params, x, mask, outs = load_triatt_golden("triatt_n12_c128.npz")
    got = triangle_attention_forward(params, x, mask, starting=starting, dtype="float32")
    np.testing.assert_allclose(got, outs[starting], rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("n,n_pad", [(48, 0), (100, 9), (256, 32)])
@pytest.mark.parametrize("starting", [True, False])
def test_triangle_attention_fp32(cuda_device, n, n_pad, starting):
    from foldjax_b200 import _lib
    from foldjax_b200.triangle_attention import triangle_attention_forward

    rng = np.random.default_rng(300 + n)
    params = orc.random_triatt_params(rng, ln_noise=0.1, std=0.05)
    x = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    mask = orc.pad_mask(n, n_pad)
    got = triangle_attention_forward(params, x, mask, starting=starting, dtype="float32")
    _lib.device_status()
    ref = orc.triangle_attention(params, x, mask, starting=starting, dtype="float64")
    has_key = mask.any(axis=2) if starting else mask.any(axis=1)
    valid = has_key[:, :, None, None] if starting else has_key[:, None, :, None]
    valid = np.broadcast_to(valid, ref.shape)
    err = _max_abs(ref[valid], got[valid])
    print(f"tri-attn starting={starting} fp32 N={n}: max-abs vs float64 oracle {err:.2e}")
    assert err <= F32_TOL
    if n_pad:  # rows with no valid key: float32 absorbs the scores under -1e9 -> uniform average
        ref32 = orc.triangle_attention(params, x, mask, starting=starting, dtype="float32")
        assert _max_abs(ref32[~valid], got[~valid]) <= 1e-3


def test_float32_cuda_tensor_selects_the_mode_and_stays_on_device(cuda_device):
    from foldjax_b200 import _device as dev
    from foldjax_b200.triangle import triangle_multiplication_forward

    rng = np.random.default_rng(8)
    n = 64
    params = orc.random_trimul_params(rng)
    x = rng.standard_normal((n, n, 128)).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda_device)
    out = triangle_multiplication_forward(dev.params_to_device(params, torch.float32), xd, None, "outgoing")
    assert out.is_cuda and out.dtype == torch.float32 and out.shape == xd.shape
    ref = orc.triangle_multiplication(params, x[None], None, "outgoing", dtype="float64")[0]
    assert _max_abs(ref, out.cpu().numpy()) <= F32_TOL
    with pytest.raises(ValueError, match="Unsupported dtype"):
        triangle_multiplication_forward(params, x, None, "outgoing", dtype="float16")
