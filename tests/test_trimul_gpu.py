"""GPU parity of the triangle multiplicative update against the oracle.

Every call goes through the C ABI (ctypes -> libb200tri.so). bf16 tolerance as
stated by the benchmark: max-abs <= 2e-2 and mean-abs <= 2e-3 of the output RMS
(see conftest.assert_parity), measured against the oracle's bf16 emulation of
the reference's XLA path.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import assert_parity, load_trimul_golden
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _bf16(t):
    return t.to(torch.bfloat16)


def _chan_major(arr: np.ndarray, ld: int, device):
    """[n_o, n_t, 128] float -> bf16 device tensor [128, n_o, ld] (zero padded pitch)."""
    n_o, n_t, c = arr.shape
    buf = torch.zeros(c, n_o, ld, dtype=torch.bfloat16, device=device)
    buf[:, :, :n_t] = _bf16(torch.from_numpy(np.ascontiguousarray(arr.transpose(2, 0, 1)))).to(device)
    return buf


@pytest.mark.parametrize("n_i,n_j,n_k", [(128, 256, 64), (64, 64, 64), (200, 136, 72), (256, 512, 320)])
def test_contract_matches_einsum(cuda_device, n_i, n_j, n_k):
    from foldjax_b200 import _lib, _device as dev

    lib = _lib.load()
    rng = np.random.default_rng(n_i + n_j + n_k)
    a = orc.round_bf16(rng.standard_normal((n_i, n_k, 128)).astype(np.float32))
    b = orc.round_bf16(rng.standard_normal((n_j, n_k, 128)).astype(np.float32))
    ld_k = (n_k + 63) // 64 * 64
    ld_j = (n_j + 63) // 64 * 64
    ad = _chan_major(a, ld_k, cuda_device)
    bd = _chan_major(b, ld_k, cuda_device)
    out = torch.full((128, n_i, ld_j), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    args = _lib.TrimulContractArgs(
        n_i=n_i, n_j=n_j, n_k=n_k, n_src=1,
        a=ad.data_ptr(), a_ld=ld_k, a_chan_stride=n_i * ld_k, a_src_stride=0,
        b=bd.data_ptr(), b_ld=ld_k, b_chan_stride=n_j * ld_k, b_src_stride=0,
        acc_in=None, out_f32=None, out_bf16=out.data_ptr(), out_ld=ld_j, out_chan_stride=n_i * ld_j,
    )
    _lib.check(lib.b200tri_trimul_contract(C.byref(args), C.c_void_p(dev.stream_ptr())))
    _lib.device_status()
    got = out[:, :, :n_j].float().cpu().numpy().transpose(1, 2, 0)  # [i, j, d]
    ref = np.einsum("ikd,jkd->ijd", a.astype(np.float64), b.astype(np.float64), optimize=True)
    assert np.isfinite(got).all()
    # fp32 accumulation then one bf16 rounding: within one bf16 ulp of the exact value
    assert (np.abs(got - ref) <= 1.01 * 2.0 ** -8 * np.maximum(np.abs(ref), 1e-3) + 1e-3).all()
    # the pitch padding beyond n_j must be left untouched
    if ld_j > n_j:
        assert torch.isnan(out[:, :, n_j:].float()).all()


def test_contract_accumulates_over_sources_and_fp32(cuda_device):
    from foldjax_b200 import _lib, _device as dev

    lib = _lib.load()
    rng = np.random.default_rng(7)
    n_i, n_j, n_k, n_src = 96, 160, 64, 3
    a = orc.round_bf16(rng.standard_normal((n_src, n_i, n_k, 128)).astype(np.float32))
    b = orc.round_bf16(rng.standard_normal((n_src, n_j, n_k, 128)).astype(np.float32))
    ld = 64
    ad = torch.stack([_chan_major(a[s], ld, cuda_device) for s in range(n_src)])
    bd = torch.stack([_chan_major(b[s], ld, cuda_device) for s in range(n_src)])
    ld_j = 192
    acc = torch.randn(128, n_i, ld_j, dtype=torch.float32, device=cuda_device)
    out32 = torch.zeros_like(acc)
    args = _lib.TrimulContractArgs(
        n_i=n_i, n_j=n_j, n_k=n_k, n_src=n_src,
        a=ad.data_ptr(), a_ld=ld, a_chan_stride=n_i * ld, a_src_stride=128 * n_i * ld,
        b=bd.data_ptr(), b_ld=ld, b_chan_stride=n_j * ld, b_src_stride=128 * n_j * ld,
        acc_in=acc.data_ptr(), out_f32=out32.data_ptr(), out_bf16=None, out_ld=ld_j, out_chan_stride=n_i * ld_j,
    )
    _lib.check(lib.b200tri_trimul_contract(C.byref(args), C.c_void_p(dev.stream_ptr())))
    _lib.device_status()
    ref = np.einsum("sikd,sjkd->ijd", a.astype(np.float64), b.astype(np.float64), optimize=True)
    ref = ref + acc[:, :, :n_j].cpu().numpy().transpose(1, 2, 0)
    got = out32[:, :, :n_j].cpu().numpy().transpose(1, 2, 0)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-3)


def _run_forward(params, x, mask, direction, residual=None):
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200 import _lib

    out = triangle_multiplication_forward(params, x, mask, direction, residual=residual)
    _lib.device_status()
    return out


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_golden_case_through_the_plugin(cuda_device, direction):
    """The committed golden vector (reference's own torch restatement, fp32) at
    the kernels' width, run in bf16: error budget is the bf16 one."""
    params, x, mask, outs = load_trimul_golden("trimul_n12_c128.npz")
    params = orc.round_params(params, "bfloat16")
    xb = orc.round_bf16(x)
    emu = orc.triangle_multiplication(params, xb, mask, direction, dtype="bfloat16")
    got = _run_forward(params, xb, mask, direction)
    print(assert_parity(emu, got, label=f"golden {direction}"))
    # and the bf16 run stays within bf16 noise of the fp32 golden output
    err = orc.error_vs(outs[direction], got)
    assert err["mean_abs_over_rms"] < 2e-2, err


@pytest.mark.parametrize("n,n_pad", [(64, 0), (128, 5), (200, 13), (256, 0)])
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_forward_matches_oracle(cuda_device, n, n_pad, direction):
    rng = np.random.default_rng(100 + n)
    params = orc.round_params(orc.random_trimul_params(rng, ln_noise=0.1), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = orc.pad_mask(n, n_pad)
    emu = orc.triangle_multiplication(params, x, mask, direction, dtype="bfloat16")
    got = _run_forward(params, x, mask, direction)
    print(assert_parity(emu, got, label=f"trimul n={n} {direction}"))
    truth = orc.triangle_multiplication(params, x, mask, direction, dtype="float64")
    e_truth = orc.error_vs(truth, got)
    e_emu = orc.error_vs(truth, emu)
    # no further from the fp64 truth than the reference's own bf16 path (25 % slack)
    assert e_truth["mean_abs_over_rms"] <= 1.25 * e_emu["mean_abs_over_rms"] + 1e-4, (e_truth, e_emu)


def test_mask_none_equals_ones_and_residual_is_fused(cuda_device):
    rng = np.random.default_rng(3)
    n = 96
    params = orc.round_params(orc.random_trimul_params(rng), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    a = _run_forward(params, x, None, "outgoing")
    b = _run_forward(params, x, np.ones((1, n, n), np.float32), "outgoing")
    assert np.array_equal(a, b)
    c = _run_forward(params, x, None, "outgoing", residual=x)
    np.testing.assert_array_equal(c, orc.round_bf16(x + a))


def test_device_tensors_batch_and_determinism(cuda_device):
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200 import _device as dev

    rng = np.random.default_rng(4)
    n = 72
    params = dev.params_to_device(orc.random_trimul_params(rng))
    x = torch.randn(2, n, n, 128, device=cuda_device).to(torch.bfloat16)
    mask = (torch.rand(2, n, n, device=cuda_device) > 0.1).float()
    out1 = triangle_multiplication_forward(params, x, mask, "incoming")
    out2 = triangle_multiplication_forward(params, x, mask, "incoming")
    assert out1.is_cuda and out1.dtype == torch.bfloat16 and out1.shape == x.shape
    assert torch.equal(out1, out2)  # fixed reduction order: reruns are bit-identical
    single = triangle_multiplication_forward(params, x[1], mask[1], "incoming")
    assert torch.equal(single, out1[1])


def test_bad_arguments_are_rejected(cuda_device):
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200 import _lib

    rng = np.random.default_rng(5)
    params = orc.random_trimul_params(rng)
    x = np.zeros((1, 8, 8, 128), np.float32)
    with pytest.raises(ValueError, match="Unsupported triangle multiplication direction"):
        triangle_multiplication_forward(params, x, None, "sideways")
    with pytest.raises(ValueError, match="expected \\(64,\\)"):  # 64-channel input, 128-channel parameters
        triangle_multiplication_forward(params, np.zeros((1, 8, 8, 64), np.float32), None, "outgoing")
    with pytest.raises(ValueError, match="multiples of 8"):
        triangle_multiplication_forward(params, np.zeros((1, 8, 8, 60), np.float32), None, "outgoing")
    lib = _lib.load()
    args = _lib.TrimulArgs(n=8)
    assert lib.b200tri_trimul_forward(C.byref(args), None) == _lib.ERR_INVALID
    assert b"must not be null" in lib.b200tri_last_error()


def test_large_case_properties(cuda_device):
    """N = 1024 (the one-block benchmark size): the oracle is too slow for the full
    tensor, so check sampled output rows against it and the linearity of the
    contraction stage in `a`."""
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200 import _device as dev, _lib

    rng = np.random.default_rng(11)
    n = 1024
    params_np = orc.round_params(orc.random_trimul_params(rng), "bfloat16")
    params = dev.params_to_device(params_np)
    x = torch.randn(1, n, n, 128, device=cuda_device).to(torch.bfloat16)
    mask = torch.from_numpy(orc.pad_mask(n, 21)).to(cuda_device)
    out = triangle_multiplication_forward(params, x, mask, "outgoing")
    _lib.device_status()
    assert torch.isfinite(out.float()).all()
    # sampled rows: out[i, :, :] needs a[i, :, :] and all of b -> emulate on CPU for 3 rows
    xn = x[0].float().cpu().numpy()
    m = mask[0].cpu().numpy()
    rows = [0, 517, 1002]
    pr = orc._Prec("bfloat16")
    x_ln = orc.layer_norm(xn, params_np["norm_in"]["scale"], params_np["norm_in"]["bias"], 1e-5, "bfloat16")
    gate = pr.r(orc._sigmoid(orc._linear(x_ln, params_np["g_in"]["kernel"], pr)))
    proj = pr.r(pr.r(gate * orc._linear(x_ln, params_np["p_in"]["kernel"], pr)) * m[..., None])
    a, b = np.split(proj, 2, axis=-1)
    t = pr.r(np.einsum("ikd,jkd->ijd", a[rows], b, optimize=True))
    t = orc.layer_norm(t, params_np["norm_out"]["scale"], params_np["norm_out"]["bias"], 1e-5, "bfloat16")
    o = orc._linear(t, params_np["p_out"]["kernel"], pr)
    g = pr.r(orc._sigmoid(orc._linear(x_ln[rows], params_np["g_out"]["kernel"], pr)))
    ref = pr.r(o * g)
    got = out[0, rows].float().cpu().numpy()
    print(assert_parity(ref, got, label="trimul n=1024 sampled rows"))
