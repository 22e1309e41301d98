"""GPU parity of the single-track attention with pair bias against the oracle, through
the C ABI. The reference computes this op in float32 (s and z are promoted); here z
and the weights are bf16 (the trunk dtype) and all arithmetic is fp32, so the oracle is
evaluated in fp64 on the same bf16-rounded z and weights and the kernel must agree to
the reference test's own tolerance, 2e-4 (tests/models/boltz2/
test_attention_checkpoint_parity.py:47-52)."""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import load_attention_pair_bias_golden
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _case(seed, n, heads=16, keep=0.85, std=0.05):
    rng = np.random.default_rng(seed)
    params = orc.round_params(orc.random_attention_pair_bias_params(rng, c_s=heads * 24, heads=heads, std=std, ln_noise=0.1),
                              "bfloat16")
    s = rng.standard_normal((1, n, heads * 24)).astype(np.float32)
    k_in = rng.standard_normal((1, n, heads * 24)).astype(np.float32)
    z = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = (rng.random((1, n)) < keep).astype(np.float32)
    mask[0, 0] = 1.0
    return params, s, k_in, z, mask


@pytest.mark.parametrize("n,heads", [(1, 16), (5, 16), (64, 16), (100, 16), (257, 16), (96, 4)])
def test_matches_oracle(cuda_device, n, heads):
    from foldjax_b200 import _lib
    from foldjax_b200.attention import attention_pair_bias_forward

    params, s, k_in, z, mask = _case(n + heads, n, heads)
    got = attention_pair_bias_forward(params, s, z, mask, k_in=k_in)
    _lib.device_status()
    ref = orc.attention_pair_bias(params, s, z, mask, k_in=k_in, dtype="float64")
    assert got.shape == ref.shape and np.isfinite(got).all()
    np.testing.assert_allclose(got, ref, rtol=2e-4, atol=2e-4)
    # k_in defaults to s
    got_s = attention_pair_bias_forward(params, s, z, mask)
    np.testing.assert_allclose(got_s, orc.attention_pair_bias(params, s, z, mask, dtype="float64"), rtol=2e-4, atol=2e-4)


def test_golden_case_with_trunk_head_width(cuda_device):
    from foldjax_b200.attention import attention_pair_bias_forward

    params, s, k_in, z, mask, out = load_attention_pair_bias_golden("attention_pair_bias_n12_c96.npz")
    params = orc.round_params(params, "bfloat16")
    zb = orc.round_bf16(z)
    got = attention_pair_bias_forward(params, s, zb, mask, k_in=k_in)
    np.testing.assert_allclose(got, orc.attention_pair_bias(params, s, zb, mask, k_in=k_in), rtol=2e-4, atol=2e-4)
    # bf16 rounding of z and of the weights moves the reference module's fp32 output by less than this
    err = orc.error_vs(out, got)
    assert err["mean_abs_over_rms"] < 2e-2, err


def test_all_keys_masked_but_one_and_determinism(cuda_device):
    from foldjax_b200 import _device as dev
    from foldjax_b200.attention import attention_pair_bias_forward

    params, s, k_in, z, mask = _case(7, 70)
    mask[:] = 0.0
    mask[0, 13] = 1.0
    got = attention_pair_bias_forward(params, s, z, mask, k_in=k_in)
    ref = orc.attention_pair_bias(params, s, z, mask, k_in=k_in)
    np.testing.assert_allclose(got, ref, rtol=2e-4, atol=2e-4)
    pd = dev.params_to_device(params)
    sd, zd, md = dev.to_device(s, torch.float32), dev.to_device(z, torch.bfloat16), dev.to_device(mask, torch.float32)
    a = attention_pair_bias_forward(pd, sd, zd, md)
    b = attention_pair_bias_forward(pd, sd, zd, md)
    assert a.is_cuda and torch.equal(a, b)


def test_rejects_unsupported_shapes(cuda_device):
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.attention import attention_pair_bias_forward

    params, s, k_in, z, mask = _case(3, 4)
    with pytest.raises(ValueError, match="multiplicity"):
        attention_pair_bias_forward(params, s, z, mask, multiplicity=2)
    with pytest.raises(ValueError, match="shapes do not match"):
        attention_pair_bias_forward(params, s, z[:, :3], mask)
    lib = _lib.load()
    sd = dev.to_device(s, torch.float32)
    ptr = sd.data_ptr()
    args = _lib.AttentionPairBiasArgs(n=4, c_s=384, c_z=64, heads=16, eps=1e-5, inf=1e6, s=ptr, k_in=None, z=ptr, mask=ptr,
                                      proj_q=ptr, proj_q_bias=ptr, proj_k=ptr, proj_v=ptr, proj_g=ptr, proj_z_norm_scale=ptr,
                                      proj_z_norm_bias=ptr, proj_z=ptr, proj_o=ptr, out=ptr, workspace=ptr, workspace_bytes=1 << 30)
    assert lib.b200tri_attention_pair_bias(C.byref(args), C.c_void_p(dev.stream_ptr())) == _lib.ERR_UNSUPPORTED
    args.c_z, args.c_s = 128, 400
    assert lib.b200tri_attention_pair_bias(C.byref(args), C.c_void_p(dev.stream_ptr())) == _lib.ERR_UNSUPPORTED
    args.c_s, args.workspace_bytes = 384, 8
    assert lib.b200tri_attention_pair_bias(C.byref(args), C.c_void_p(dev.stream_ptr())) == _lib.ERR_WORKSPACE
