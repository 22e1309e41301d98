"""Parity at the benchmark's own sizes: N = 3072 with the last 60 tokens padded (the
per-block work of the 48-block trunk) and N = 1024 with the last 21 padded (the
one-block config), through the public operators.

The CPU restatement cannot produce a whole N = 3072 output in reasonable time, but an
output element (i, j) of either op depends on two rows of the input only (rows i and
j; columns for the incoming / ending variants), so a sample of elements is compared
against ``oracle.triangle_multiplication_sampled`` / ``triangle_attention_sampled``
(checked against the full restatement in tests/test_oracle.py). Tolerance: the
benchmark's bf16 budget (conftest.assert_parity).
"""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_parity
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _pair_case(cuda_device, n, n_pad, seed):
    gen = torch.Generator(device=cuda_device).manual_seed(seed)
    x = torch.randn(1, n, n, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    mask = torch.from_numpy(orc.pad_mask(n, n_pad)).to(cuda_device)
    return x, mask


def _sample(n, n_pad, seed, n_rows=3, n_cols=48):
    """Sampled rows and columns: mostly valid tokens, the first and the last valid one
    always included, plus two padded columns."""
    rng = np.random.default_rng(seed)
    valid = n - n_pad
    rows = np.unique(np.concatenate(([0, valid - 1], rng.integers(1, valid - 1, n_rows - 2))))
    cols = np.unique(np.concatenate(([0, valid - 1], rng.integers(1, valid - 1, n_cols - 4),
                                     [valid, n - 1] if n_pad else [1, 2])))
    return rows, cols


def _gather(x, mask, rows, cols, transposed):
    """(xi, mi, xj, mj, xij) as float32 NumPy arrays in the frame the oracle's sampled forms take."""
    x0, m0 = x[0], mask[0]
    r, c = torch.as_tensor(rows, device=x.device), torch.as_tensor(cols, device=x.device)
    if transposed:
        xi, xj = x0[:, r].transpose(0, 1), x0[:, c].transpose(0, 1)
        mi, mj = m0[:, r].transpose(0, 1), m0[:, c].transpose(0, 1)
    else:
        xi, xj, mi, mj = x0[r], x0[c], m0[r], m0[c]
    xij = x0[r][:, c]
    f = lambda t: t.float().cpu().numpy()
    return f(xi), f(mi), f(xj), f(mj), f(xij)


@pytest.mark.parametrize("n,n_pad", [(3072, 60), (1024, 21)])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_triangle_multiplication_sampled_elements(cuda_device, n, n_pad, direction):
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.triangle import triangle_multiplication_forward

    params_np = orc.round_params(orc.random_trimul_params(np.random.default_rng(3)), "bfloat16")
    x, mask = _pair_case(cuda_device, n, n_pad, seed=3)
    out = triangle_multiplication_forward(dev.params_to_device(params_np), x, mask, direction)
    _lib.device_status()
    rows, cols = _sample(n, n_pad, seed=n)
    xi, mi, xj, mj, xij = _gather(x, mask, rows, cols, transposed=direction == "incoming")
    ref = orc.triangle_multiplication_sampled(params_np, xi, mi, xj, mj, xij, dtype="bfloat16")
    got = out[0][torch.as_tensor(rows, device=cuda_device)][:, torch.as_tensor(cols, device=cuda_device)]
    print(assert_parity(ref, got.float().cpu().numpy(), label=f"tri-mult {direction} N={n} pad={n_pad} sampled"))
    del out
    dev.release_workspaces()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("n,n_pad", [(3072, 60), (1024, 21)])
@pytest.mark.parametrize("starting", [True, False])
def test_triangle_attention_sampled_elements(cuda_device, n, n_pad, starting):
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.triangle_attention import triangle_attention_forward

    params_np = orc.round_params(orc.random_triatt_params(np.random.default_rng(3)), "bfloat16")
    x, mask = _pair_case(cuda_device, n, n_pad, seed=4)
    out = triangle_attention_forward(dev.params_to_device(params_np), x, mask, starting=starting)
    _lib.device_status()
    rows, cols = _sample(n, n_pad, seed=n + 1)
    xi, mi, xj, _, _ = _gather(x, mask, rows, cols, transposed=not starting)
    ref = orc.triangle_attention_sampled(params_np, xi, mi, xj, cols, dtype="bfloat16")
    r, c = torch.as_tensor(rows, device=cuda_device), torch.as_tensor(cols, device=cuda_device)
    got = out[0][r][:, c] if starting else out[0][c][:, r].transpose(0, 1)
    print(assert_parity(ref, got.float().cpu().numpy(), label=f"tri-attn starting={starting} N={n} pad={n_pad} sampled"))
    del out
    dev.release_workspaces()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("n", [1024, 3072])
def test_pair_transition_sampled_rows(cuda_device, n):
    """The transition is row-local: whole sampled rows of the pair tensor against the oracle."""
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.transition import transition_forward

    params_np = orc.round_params(orc.random_transition_params(np.random.default_rng(5)), "bfloat16")
    x, _ = _pair_case(cuda_device, n, 0, seed=5)
    out = transition_forward(dev.params_to_device(params_np), x)
    _lib.device_status()
    rows = torch.as_tensor([0, n // 2 + 5, n - 1], device=cuda_device)
    ref = orc.transition(params_np, x[0][rows].float().cpu().numpy(), dtype="bfloat16")
    print(assert_parity(ref, out[0][rows].float().cpu().numpy(), label=f"pair transition N={n} sampled rows"))
    del out
    torch.cuda.empty_cache()


def test_attention_pair_bias_at_the_one_block_size(cuda_device):
    """Single-track attention with pair bias at N = 1024 with the last 21 tokens padded (the
    block config), full output against the fp64 oracle at the reference test's 2e-4."""
    from foldjax_b200 import _lib
    from foldjax_b200.attention import attention_pair_bias_forward

    n, heads = 1024, 16
    rng = np.random.default_rng(6)
    params = orc.round_params(orc.random_attention_pair_bias_params(rng, c_s=heads * 24, heads=heads), "bfloat16")
    s = rng.standard_normal((1, n, heads * 24)).astype(np.float32)
    z = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = np.ones((1, n), np.float32)
    mask[0, n - 21:] = 0.0
    got = attention_pair_bias_forward(params, s, z, mask)
    _lib.device_status()
    ref = orc.attention_pair_bias(params, s, z, mask, dtype="float64")
    np.testing.assert_allclose(got, ref, rtol=2e-4, atol=2e-4)
