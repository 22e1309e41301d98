"""The triangle ops at the shapes of their other call sites, through the C ABI's general
path (CUDA-core stages around the tensor-core contraction):

* the template stacks' c_z = 64 with c_hidden = 128, which the reference's fused
  cuEquivariance kernel rejects (src/foldjax/models/protenix/models/triangle/triangle.py:131-137);
* a 384-channel pair with 12 attention heads (the structural refiner,
  src/foldjax/models/opendde/structural_refiner.py:62);
* small widths and other head counts;
* leading batch axes beyond one, folded into B like the reference's fused wrappers do
  (src/foldjax/models/_cueq.py:89-121).

Tolerance: the benchmark's bf16 budget against the oracle's bf16 emulation
(conftest.assert_parity), and the float32 bar (1e-4) against the float64 oracle."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_parity
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("c_z,c_hidden", [(64, 128), (384, 384), (32, 32), (128, 64), (64, 200)])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_triangle_multiplication_other_widths_bf16(cuda_device, c_z, c_hidden, direction):
    from foldjax_b200 import _lib
    from foldjax_b200.triangle import triangle_multiplication_forward

    rng = np.random.default_rng(c_z + c_hidden)
    n = 72 if c_z < 384 else 40
    params = orc.round_params(orc.random_trimul_params(rng, c_z=c_z, c_hidden=c_hidden, std=0.05, ln_noise=0.1), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, c_z)).astype(np.float32))
    mask = orc.pad_mask(n, 5)
    got = triangle_multiplication_forward(params, x, mask, direction)
    _lib.device_status()
    emu = orc.triangle_multiplication(params, x, mask, direction, dtype="bfloat16")
    print(assert_parity(emu, got, label=f"trimul c_z={c_z} c_hidden={c_hidden} {direction}"))
    truth = orc.triangle_multiplication(params, x, mask, direction, dtype="float64")
    e_got, e_emu = orc.error_vs(truth, got), orc.error_vs(truth, emu)
    assert e_got["mean_abs_over_rms"] <= 1.25 * e_emu["mean_abs_over_rms"] + 1e-4, (e_got, e_emu)


@pytest.mark.parametrize("c_z,heads,head_dim", [(64, 4, 16), (384, 12, 32), (128, 8, 16), (128, 2, 64), (32, 4, 8)])
@pytest.mark.parametrize("starting", [True, False])
def test_triangle_attention_other_shapes_bf16(cuda_device, c_z, heads, head_dim, starting):
    from foldjax_b200 import _lib
    from foldjax_b200.triangle_attention import triangle_attention_forward

    rng = np.random.default_rng(c_z + heads)
    n = 70 if c_z < 384 else 40
    params = orc.round_params(orc.random_triatt_params(rng, c_z=c_z, heads=heads, c_hidden=head_dim, std=0.05, ln_noise=0.1),
                              "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, c_z)).astype(np.float32))
    mask = orc.pad_mask(n, 6)
    got = triangle_attention_forward(params, x, mask, starting=starting)
    _lib.device_status()
    emu = orc.triangle_attention(params, x, mask, starting=starting, dtype="bfloat16")
    has_key = mask.any(axis=2) if starting else mask.any(axis=1)
    valid = has_key[:, :, None, None] if starting else has_key[:, None, :, None]
    print(assert_parity(emu, got, where=np.broadcast_to(valid, emu.shape),
                        label=f"triatt c_z={c_z} {heads}x{head_dim} starting={starting}"))


def test_other_shapes_in_float32(cuda_device):
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200.triangle_attention import triangle_attention_forward

    rng = np.random.default_rng(77)
    n = 48
    pm = orc.random_trimul_params(rng, c_z=64, c_hidden=128)
    pa = orc.random_triatt_params(rng, c_z=64, heads=4, c_hidden=16)
    x = rng.standard_normal((1, n, n, 64)).astype(np.float32)
    mask = orc.pad_mask(n, 3)
    for direction in ("outgoing", "incoming"):
        got = triangle_multiplication_forward(pm, x, mask, direction, dtype="float32")
        ref = orc.triangle_multiplication(pm, x, mask, direction, dtype="float64")
        assert np.max(np.abs(got - ref)) <= 1e-4
    valid = np.broadcast_to(mask.any(axis=2)[:, :, None, None], x.shape)
    got = triangle_attention_forward(pa, x, mask, starting=True, dtype="float32")
    ref = orc.triangle_attention(pa, x, mask, starting=True, dtype="float64")
    assert np.max(np.abs(got - ref)[valid]) <= 1e-4


def test_leading_batch_axes_are_folded(cuda_device):
    from foldjax_b200 import _device as dev
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200.triangle_attention import triangle_attention_forward

    rng = np.random.default_rng(78)
    n = 40
    pm = dev.params_to_device(orc.random_trimul_params(rng))
    pa = dev.params_to_device(orc.random_triatt_params(rng))
    x = torch.randn(2, 3, n, n, 128, device=cuda_device).to(torch.bfloat16)
    mask = (torch.rand(2, 3, n, n, device=cuda_device) > 0.1).float()
    out = triangle_multiplication_forward(pm, x, mask, "outgoing")
    assert out.shape == x.shape
    flat = triangle_multiplication_forward(pm, x.reshape(6, n, n, 128), mask.reshape(6, n, n), "outgoing")
    assert torch.equal(out.reshape(6, n, n, 128), flat)
    single = triangle_multiplication_forward(pm, x[1, 2], mask[1, 2], "outgoing")
    assert single.shape == (n, n, 128) and torch.equal(single, out[1, 2])
    att = triangle_attention_forward(pa, x, mask, starting=False)
    assert att.shape == x.shape
    assert torch.equal(att[0, 1], triangle_attention_forward(pa, x[0, 1], mask[0, 1], starting=False))
