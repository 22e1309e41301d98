"""GPU parity of triangle attention against the oracle, through the C ABI.

Tolerance: the benchmark's bf16 budget (mean-abs <= 2e-3 and max-abs <= 2e-2 of the
output RMS, see conftest.assert_parity) against the oracle's bf16 emulation of the
reference's XLA path. Rows of the attention that have no valid key hold
"-1e9 absorbed in fp32" values in the reference; they are compared too (the kernel
reproduces the uniform average) but with the same budget.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import assert_parity, load_triatt_golden
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _run_forward(params, x, mask, starting, residual=None):
    from foldjax_b200 import _lib
    from foldjax_b200.triangle_attention import triangle_attention_forward

    out = triangle_attention_forward(params, x, mask, starting=starting, residual=residual)
    _lib.device_status()
    return out


def _valid_rows(mask, starting, shape):
    has_key = mask.any(axis=2) if starting else mask.any(axis=1)
    valid = has_key[:, :, None] if starting else has_key[:, None, :]
    return np.broadcast_to(valid[..., None], shape)


def test_projection_stage_matches_oracle(cuda_device):
    from foldjax_b200 import _device as dev, _lib

    lib = _lib.load()
    rng = np.random.default_rng(21)
    n = 136
    params = orc.round_params(orc.random_triatt_params(rng, ln_noise=0.1, std=0.05), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    _, parts = orc.triangle_attention(params, x, None, True, dtype="bfloat16", return_parts=True)
    P = dev.params_to_device(params)
    xd = dev.to_device(x, torch.bfloat16)[0]
    ld = (n + 63) // 64 * 64
    q = torch.empty(n, n, 128, dtype=torch.bfloat16, device=cuda_device)
    k = torch.empty_like(q)
    vt = torch.zeros(n, 128, ld, dtype=torch.float16, device=cuda_device)
    bias = torch.zeros(4, n, ld, dtype=torch.bfloat16, device=cuda_device)
    nb = lib.b200tri_triatt_project_workspace_bytes()
    ws = torch.empty(nb + 1024, dtype=torch.uint8, device=cuda_device)
    args = _lib.TriattProjectArgs(
        n_outer=n, n_inner=n, heads=4, head_dim=32, eps=1e-5,
        x=xd.data_ptr(), xs_outer=n * 128, xs_inner=128,
        norm_scale=P["layer_norm"]["scale"].data_ptr(), norm_bias=P["layer_norm"]["bias"].data_ptr(),
        w_q=P["mha"]["linear_q"]["kernel"].data_ptr(), w_k=P["mha"]["linear_k"]["kernel"].data_ptr(),
        w_v=P["mha"]["linear_v"]["kernel"].data_ptr(), w_bias=P["linear"]["kernel"].data_ptr(),
        q=q.data_ptr(), k=k.data_ptr(), vt=vt.data_ptr(), bias=bias.data_ptr(), ld=ld, bias_head_stride=n * ld,
        workspace=dev.aligned_ptr(ws), workspace_bytes=nb,
    )
    _lib.check(lib.b200tri_triatt_project(C.byref(args), C.c_void_p(dev.stream_ptr())))
    _lib.device_status()
    # oracle parts are [B, I, H, J, D]
    q_ref = parts["q"][0].transpose(0, 2, 1, 3).reshape(n, n, 128)
    k_ref = parts["k"][0].transpose(0, 2, 1, 3).reshape(n, n, 128)
    v_ref = parts["v"][0].transpose(0, 1, 3, 2).reshape(n, 128, n)
    b_ref = parts["tri_bias"][0, 0]
    print(assert_parity(q_ref, q.float().cpu().numpy(), label="q", mean_tol=2e-4))
    print(assert_parity(k_ref, k.float().cpu().numpy(), label="k", mean_tol=2e-4))
    print(assert_parity(v_ref, vt[:, :, :n].float().cpu().numpy(), label="vT", mean_tol=2e-4))
    print(assert_parity(b_ref, bias[:, :, :n].float().cpu().numpy(), label="bias", mean_tol=2e-4))


@pytest.mark.parametrize("n_i,n_j,n_k", [(4, 128, 64), (9, 200, 200), (16, 256, 320)])
def test_core_matches_dense_attention(cuda_device, n_i, n_j, n_k):
    """The attention-core operator on its own, with large biases so the running
    max moves (exercises the rescale), random key masks and one row with no
    valid key (uniform average in the XLA-path convention)."""
    from foldjax_b200 import _device as dev, _lib

    lib = _lib.load()
    rng = np.random.default_rng(n_i * 1000 + n_k)
    h, d = 4, 32
    q = orc.round_bf16(rng.normal(size=(n_i, n_j, h * d), scale=0.6).astype(np.float32))
    k = orc.round_bf16(rng.normal(size=(n_i, n_k, h * d), scale=0.6).astype(np.float32))
    v = orc.round_bf16(rng.normal(size=(n_i, n_k, h * d), scale=1.0).astype(np.float32))
    bias = orc.round_bf16(rng.normal(size=(h, n_j, n_k), scale=4.0).astype(np.float32))
    # keys sorted by a trend so later tiles raise the maximum
    bias += orc.round_bf16(np.linspace(-6, 6, n_k, dtype=np.float32))[None, None, :]
    bias = orc.round_bf16(bias)
    keep = rng.random((n_i, n_k)) > 0.2
    keep[:, 0] = True
    keep[n_i - 1, :] = False  # a row with no valid key
    mask = keep.astype(np.float32)
    # dense fp32 reference in the reference's operand order
    q5 = q.reshape(n_i, n_j, h, d).transpose(0, 2, 1, 3)[None]
    k5 = k.reshape(n_i, n_k, h, d).transpose(0, 2, 1, 3)[None]
    v5 = v.reshape(n_i, n_k, h, d).transpose(0, 2, 1, 3)[None]
    mb = (np.float32(1e9) * (mask - 1.0))[None, :, None, None, :]
    ref = orc.attention_core(q5, k5, v5, bias[None, None], mb, dtype="bfloat16")[0]  # [I,H,J,D]
    ref = ref.transpose(0, 2, 1, 3).reshape(n_i, n_j, h * d)

    ld = (n_k + 63) // 64 * 64
    qd = dev.to_device(q, torch.bfloat16)
    kd = dev.to_device(k, torch.bfloat16)
    vt = torch.zeros(n_i, h * d, ld, dtype=torch.float16, device=cuda_device)
    vt[:, :, :n_k] = torch.from_numpy(np.ascontiguousarray(v.transpose(0, 2, 1))).to(cuda_device).half()
    bd = torch.zeros(h, n_j, ld, dtype=torch.bfloat16, device=cuda_device)
    bd[:, :, :n_k] = torch.from_numpy(bias).to(cuda_device).bfloat16()
    md = dev.to_device(mask, torch.float32)
    o = torch.full((n_i, n_j, h * d), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    rmax = torch.zeros(n_i, h, n_j, dtype=torch.float32, device=cuda_device)
    rsum = torch.zeros_like(rmax)
    nb = lib.b200tri_triatt_core_workspace_bytes(n_i, n_k)
    ws = torch.empty(nb + 1024, dtype=torch.uint8, device=cuda_device)
    args = _lib.TriattCoreArgs(
        n_i=n_i, n_j=n_j, n_k=n_k, heads=h, head_dim=d,
        q=qd.data_ptr(), k=kd.data_ptr(), vt=vt.data_ptr(), v_ld=ld,
        bias=bd.data_ptr(), bias_ld=ld, bias_head_stride=n_j * ld,
        mask=md.data_ptr(), ms_i=n_k, ms_k=1, inf=1e9,
        o=o.data_ptr(), row_max=rmax.data_ptr(), row_sum=rsum.data_ptr(), unnormalized=0,
        workspace=dev.aligned_ptr(ws), workspace_bytes=nb,
    )
    _lib.check(lib.b200tri_triatt_core(C.byref(args), C.c_void_p(dev.stream_ptr())))
    _lib.device_status()
    got = o.float().cpu().numpy()
    print(assert_parity(ref, got, label=f"core {n_i}x{n_j}x{n_k}"))
    # softmax statistics: log-sum-exp of the scores per (i, h, j)
    s = np.einsum("ihjd,ihkd->ihjk", q5[0].astype(np.float64), k5[0].astype(np.float64))
    s = s + mb[0].astype(np.float64) + bias[None].astype(np.float64)
    lse_ref = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    lse_got = rmax.cpu().numpy().astype(np.float64) + np.log(rsum.cpu().numpy().astype(np.float64))
    valid = keep.any(axis=1)
    np.testing.assert_allclose(lse_got[valid], lse_ref[valid], rtol=0, atol=5e-3)


@pytest.mark.parametrize("starting", [True, False])
def test_golden_case_through_the_plugin(cuda_device, starting):
    params, x, mask, outs = load_triatt_golden("triatt_n12_c128.npz")
    params = orc.round_params(params, "bfloat16")
    xb = orc.round_bf16(x)
    emu = orc.triangle_attention(params, xb, mask, starting=starting, dtype="bfloat16")
    got = _run_forward(params, xb, mask, starting)
    valid = _valid_rows(mask, starting, emu.shape)
    print(assert_parity(emu, got, where=valid, label=f"golden starting={starting}"))
    err = orc.error_vs(outs[starting][valid], got[valid])
    assert err["mean_abs_over_rms"] < 3e-2, err


@pytest.mark.parametrize("n,n_pad", [(64, 0), (128, 8), (200, 13), (256, 64)])
@pytest.mark.parametrize("starting", [True, False])
def test_forward_matches_oracle(cuda_device, n, n_pad, starting):
    rng = np.random.default_rng(200 + n)
    params = orc.round_params(orc.random_triatt_params(rng, ln_noise=0.1, std=0.05), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask = orc.pad_mask(n, n_pad)
    emu = orc.triangle_attention(params, x, mask, starting=starting, dtype="bfloat16")
    got = _run_forward(params, x, mask, starting)
    valid = _valid_rows(mask, starting, emu.shape)
    print(assert_parity(emu, got, where=valid, label=f"triatt n={n} starting={starting}"))
    if n_pad:  # rows with no valid key: uniform average over all keys, like the XLA path
        print(assert_parity(emu, got, where=~valid, label="  fully masked rows", mean_tol=5e-3))
    truth = orc.triangle_attention(params, x, mask, starting=starting, dtype="float64")
    e_truth = orc.error_vs(truth[valid], got[valid])
    e_emu = orc.error_vs(truth[valid], emu[valid])
    assert e_truth["mean_abs_over_rms"] <= 1.25 * e_emu["mean_abs_over_rms"] + 1e-4, (e_truth, e_emu)


def test_config2_shape_and_ending_is_transposed_starting(cuda_device):
    """Benchmark config 2 (N=512, last 64 tokens padded, seed 1): ending node ==
    starting node on the transposed input, and sampled rows agree with the oracle."""
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.triangle_attention import triangle_attention_forward

    rng = np.random.default_rng(1)
    n = 512
    params_np = orc.round_params(orc.random_triatt_params(rng), "bfloat16")
    params = dev.params_to_device(params_np)
    x_np = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    mask_np = orc.pad_mask(n, 64)
    x = dev.to_device(x_np, torch.bfloat16)
    mask = dev.to_device(mask_np, torch.float32)
    end = triangle_attention_forward(params, x, mask, starting=False)
    start_t = triangle_attention_forward(params, x.transpose(1, 2).contiguous(), mask.transpose(1, 2).contiguous(),
                                         starting=True)
    _lib.device_status()
    assert torch.equal(end, start_t.transpose(1, 2))
    # starting node, sampled rows i against the oracle (rows are independent)
    start = triangle_attention_forward(params, x, mask, starting=True)
    rows = [0, 255, 447]
    emu, parts = orc.triangle_attention(params_np, x_np, mask_np, True, dtype="bfloat16", return_parts=True)
    got = start[0, rows].float().cpu().numpy()
    print(assert_parity(emu[0, rows], got, label="config 2 sampled rows"))


def test_attention_core_operator_signature(cuda_device):
    """core(q, k, v, tri_bias, mask_bias) with the reference's 5-D operands."""
    from foldjax_b200.triangle_attention import attention_core
    from foldjax_b200 import _lib

    rng = np.random.default_rng(9)
    b, n, h, d = 1, 96, 4, 32
    q = orc.round_bf16(rng.normal(size=(b, n, h, n, d), scale=0.5).astype(np.float32))
    k = orc.round_bf16(rng.normal(size=(b, n, h, n, d), scale=0.5).astype(np.float32))
    v = orc.round_bf16(rng.normal(size=(b, n, h, n, d)).astype(np.float32))
    tb = orc.round_bf16(rng.normal(size=(b, 1, h, n, n), scale=2.0).astype(np.float32))
    keep = rng.random((b, n, n)) > 0.15
    keep[..., 0] = True
    mb = np.where(keep[:, :, None, None, :], np.float32(0), np.float32(-1e9))
    ref = orc.attention_core(q, k, v, tb, mb, dtype="bfloat16")
    t = lambda a, dt: torch.from_numpy(a).to(cuda_device).to(dt)
    got = attention_core(t(q, torch.bfloat16), t(k, torch.bfloat16), t(v, torch.bfloat16), t(tb, torch.bfloat16),
                         t(mb, torch.float32))
    _lib.device_status()
    assert got.shape == ref.shape and got.dtype == torch.bfloat16
    print(assert_parity(ref, got.float().cpu().numpy(), label="attention_core operator"))


def test_mask_none_residual_and_determinism(cuda_device):
    rng = np.random.default_rng(6)
    n = 80
    params = orc.round_params(orc.random_triatt_params(rng), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    a = _run_forward(params, x, None, True)
    b = _run_forward(params, x, np.ones((1, n, n), np.float32), True)
    assert np.array_equal(a, b)
    c = _run_forward(params, x, None, True, residual=x)
    np.testing.assert_array_equal(c, orc.round_bf16(x + a))
    assert np.array_equal(a, _run_forward(params, x, None, True))


def test_core_resumes_across_key_tiles(cuda_device):
    """Ring-attention building block: the same softmax continued over three key
    tiles (running state in acc_o / row_max / row_sum) equals the one-shot core."""
    from foldjax_b200 import _device as dev, _lib

    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(5)
    n_i, n_j, h, d = 6, 200, 4, 32
    tiles = [136, 64, 120]
    n_k = sum(tiles)
    ld = (n_k + 63) // 64 * 64
    q = (torch.randn(n_i, n_j, h * d, generator=g) * 0.6).bfloat16().to(cuda_device)
    k = (torch.randn(n_i, n_k, h * d, generator=g) * 0.6).bfloat16().to(cuda_device)
    v = torch.randn(n_i, n_k, h * d, generator=g).bfloat16()
    bias = (torch.randn(h, n_j, n_k, generator=g) * 3.0 + torch.linspace(-5, 5, n_k)).bfloat16()
    mask = (torch.rand(n_i, n_k, generator=g) > 0.2).float()
    mask[:, 0] = 1.0
    mask[n_i - 1, :tiles[0]] = 0.0  # a row whose first key tile is fully masked
    mask = mask.to(cuda_device)

    def run(k_t, v_t, b_t, m_t, n_kt, out, **extra):
        ldt = (n_kt + 63) // 64 * 64
        vt = torch.zeros(n_i, h * d, ldt, dtype=torch.float16, device=cuda_device)
        vt[:, :, :n_kt] = v_t.transpose(1, 2).to(cuda_device).half()
        bd = torch.zeros(h, n_j, ldt, dtype=torch.bfloat16, device=cuda_device)
        bd[:, :, :n_kt] = b_t.to(cuda_device)
        kd = k_t.contiguous()
        md = m_t.contiguous()
        nb = lib.b200tri_triatt_core_workspace_bytes(n_i, n_kt)
        ws = torch.empty(nb + 1024, dtype=torch.uint8, device=cuda_device)
        args = _lib.TriattCoreArgs(
            n_i=n_i, n_j=n_j, n_k=n_kt, heads=h, head_dim=d, q=q.data_ptr(), k=kd.data_ptr(), vt=vt.data_ptr(),
            v_ld=ldt, bias=bd.data_ptr(), bias_ld=ldt, bias_head_stride=n_j * ldt, mask=md.data_ptr(), ms_i=n_kt,
            ms_k=1, inf=1e9, o=out.data_ptr(), workspace=dev.aligned_ptr(ws), workspace_bytes=nb, **extra)
        _lib.check(lib.b200tri_triatt_core(C.byref(args), C.c_void_p(dev.stream_ptr())))
        torch.cuda.synchronize()

    ref = torch.empty(n_i, n_j, h * d, dtype=torch.bfloat16, device=cuda_device)
    run(k, v, bias, mask, n_k, ref, row_max=None, row_sum=None, unnormalized=0)
    got = torch.full_like(ref, float("nan"))
    acc = torch.zeros(n_i, n_j, h * d, dtype=torch.float32, device=cuda_device)
    rmax = torch.zeros(n_i, h, n_j, dtype=torch.float32, device=cuda_device)
    rsum = torch.zeros_like(rmax)
    k0 = 0
    for t, n_kt in enumerate(tiles):
        sl = slice(k0, k0 + n_kt)
        run(k[:, sl], v[:, sl], bias[:, :, sl], mask[:, sl], n_kt, got, row_max=rmax.data_ptr(),
            row_sum=rsum.data_ptr(), acc_o=acc.data_ptr(), resume=int(t > 0), unnormalized=int(t < len(tiles) - 1))
        k0 += n_kt
    _lib.device_status()
    print(assert_parity(ref.float().cpu().numpy(), got.float().cpu().numpy(), label="resumed core", mean_tol=2e-4))


def test_attention_core_scale_argument_and_mixed_mask_bias(cuda_device):
    """The cuEquivariance calling convention (unscaled q plus ``scale``,
    src/foldjax/models/_cueq.py:66-121) and an additive mask bias that mixes soft entries
    with the -1e9 constant and -inf: the bias is added as given, not rebuilt from a 0/1 mask."""
    from foldjax_b200.triangle_attention import attention_core
    from foldjax_b200 import _lib

    rng = np.random.default_rng(10)
    lead, n_i, n_j, n_k, h, d = (2,), 7, 130, 90, 4, 32
    shape = lambda n: lead + (n_i, h, n, d)
    q = orc.round_bf16(rng.normal(size=shape(n_j), scale=2.5).astype(np.float32))
    k = orc.round_bf16(rng.normal(size=shape(n_k), scale=0.5).astype(np.float32))
    v = orc.round_bf16(rng.normal(size=shape(n_k)).astype(np.float32))
    tb = orc.round_bf16(rng.normal(size=lead + (1, h, n_j, n_k), scale=2.0).astype(np.float32))
    kind = rng.integers(0, 10, size=lead + (n_i, n_k))
    mb = np.zeros(lead + (n_i, n_k), np.float32)
    mb[kind == 0] = -1e9
    mb[kind == 1] = -np.inf
    soft = kind == 2
    mb[soft] = -rng.random(soft.sum()).astype(np.float32) * 3.0  # soft biases beside the hard ones
    mb[..., 0] = 0.0  # every row keeps at least one key
    mb5 = mb[:, :, None, None, :]
    scale = 1.0 / np.sqrt(d)
    q_scaled = orc.round_bf16(q * orc.round_bf16(np.float32(scale)))
    ref = orc.attention_core(q_scaled, k, v, tb, np.maximum(mb5, np.float32(-1e9)), dtype="bfloat16")
    t = lambda a, dt: torch.from_numpy(a).to(cuda_device).to(dt)
    got = attention_core(t(q, torch.bfloat16), t(k, torch.bfloat16), t(v, torch.bfloat16), t(tb, torch.bfloat16),
                         t(mb5, torch.float32), scale=scale)
    _lib.device_status()
    assert got.shape == ref.shape and got.dtype == torch.bfloat16
    print(assert_parity(ref, got.float().cpu().numpy(), label="attention_core scale= and mixed mask bias"))
    # the soft entries matter: dropping them changes the result by far more than the tolerance
    ref_nosoft = orc.attention_core(q_scaled, k, v, tb, np.where(soft[:, :, None, None, :], 0, np.maximum(mb5, -1e9)),
                                    dtype="bfloat16")
    assert orc.error_vs(ref_nosoft, got.float().cpu().numpy())["mean_abs_over_rms"] > 1e-2


def test_core_walks_several_key_tiles_in_one_launch(cuda_device):
    """b200tri_triatt_core_multi: one launch over key tiles that live in separate buffers
    equals the one-shot core over the concatenated keys; and the context-parallel pattern -
    own tile first (unnormalized), then every peer tile in one resumed launch - does too."""
    from foldjax_b200 import _device as dev, _lib

    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(15)
    n_i, n_j, h, d, n_kt, n_t = 5, 200, 4, 32, 128, 3
    n_k = n_kt * n_t
    q = (torch.randn(n_i, n_j, h * d, generator=g) * 0.6).bfloat16().to(cuda_device)
    k = (torch.randn(n_i, n_k, h * d, generator=g) * 0.6).bfloat16().to(cuda_device)
    v = torch.randn(n_i, n_k, h * d, generator=g).bfloat16().to(cuda_device)
    bias = (torch.randn(h, n_j, n_k, generator=g) * 3.0 + torch.linspace(-5, 5, n_k)).bfloat16().to(cuda_device)
    mask = (torch.rand(n_i, n_k, generator=g) > 0.2).float()
    mask[:, 0] = 1.0
    mask[n_i - 1, :n_kt] = 0.0
    mask = mask.to(cuda_device)
    keep = []  # buffers stay alive until the launches have run

    def tile_args(sl, n_keys, **common):
        vt = v[:, sl].transpose(1, 2).contiguous().half()
        bd = bias[:, :, sl].contiguous()
        kd = k[:, sl].contiguous()
        md = mask[:, sl].contiguous()
        keep.extend([vt, bd, kd, md])
        return dict(n_i=n_i, n_j=n_j, n_k=n_keys, heads=h, head_dim=d, q=q.data_ptr(), k=kd.data_ptr(),
                    vt=vt.data_ptr(), v_ld=n_keys, bias=bd.data_ptr(), bias_ld=n_keys, bias_head_stride=n_j * n_keys,
                    mask=md.data_ptr(), ms_i=n_keys, ms_k=1, inf=1e9, **common)

    def launch(arg_dicts):
        n = len(arg_dicts)
        nb = lib.b200tri_triatt_core_multi_workspace_bytes(n_i, arg_dicts[0]["n_k"], n)
        ws = torch.empty(nb + 1024, dtype=torch.uint8, device=cuda_device)
        keep.append(ws)
        arr = (_lib.TriattCoreArgs * n)(*[
            _lib.TriattCoreArgs(workspace=dev.aligned_ptr(ws), workspace_bytes=nb, **a) for a in arg_dicts])
        _lib.check(lib.b200tri_triatt_core_multi(arr, n, C.c_void_p(dev.stream_ptr())))

    ref = torch.empty(n_i, n_j, h * d, dtype=torch.bfloat16, device=cuda_device)
    launch([tile_args(slice(0, n_k), n_k, o=ref.data_ptr())])
    tiles = [slice(t * n_kt, (t + 1) * n_kt) for t in range(n_t)]
    one = torch.full_like(ref, float("nan"))
    launch([tile_args(sl, n_kt, o=one.data_ptr()) for sl in tiles])
    acc = torch.zeros(n_i, n_j, h * d, dtype=torch.float32, device=cuda_device)
    rmax = torch.zeros(n_i, h, n_j, dtype=torch.float32, device=cuda_device)
    rsum = torch.zeros_like(rmax)
    state = dict(row_max=rmax.data_ptr(), row_sum=rsum.data_ptr(), acc_o=acc.data_ptr())
    two = torch.full_like(ref, float("nan"))
    launch([tile_args(tiles[1], n_kt, o=two.data_ptr(), unnormalized=1, **state)])  # "own" tile first
    launch([tile_args(sl, n_kt, o=two.data_ptr(), resume=1, **state) for sl in (tiles[2], tiles[0])])
    # the grouped pattern of a four-tile ring: own tile, then one tile, then two tiles in a launch
    # that resumes AND leaves the state unnormalised in the middle (64-key tiles here)
    n_q4 = n_k // 6
    quarter = [slice(t * n_q4, (t + 1) * n_q4) for t in range(6)]
    three = torch.full_like(ref, float("nan"))
    acc.zero_(); rmax.zero_(); rsum.zero_()
    launch([tile_args(quarter[2], n_q4, o=three.data_ptr(), unnormalized=1, **state)])
    launch([tile_args(quarter[3], n_q4, o=three.data_ptr(), resume=1, unnormalized=1, **state)])
    launch([tile_args(sl, n_q4, o=three.data_ptr(), resume=1, unnormalized=1, **state) for sl in (quarter[4], quarter[5])])
    launch([tile_args(sl, n_q4, o=three.data_ptr(), resume=1, **state) for sl in (quarter[0], quarter[1])])
    torch.cuda.synchronize()
    _lib.device_status()
    r = ref.float().cpu().numpy()
    print(assert_parity(r, one.float().cpu().numpy(), label="three key tiles, one launch", mean_tol=2e-4))
    print(assert_parity(r, two.float().cpu().numpy(), label="own tile + resumed multi-tile launch", mean_tol=2e-4))
    print(assert_parity(r, three.float().cpu().numpy(), label="own tile + grouped resumed launches", mean_tol=2e-4))
    # too many tiles, or ragged tiles, are refused
    bad = (_lib.TriattCoreArgs * 8)()
    assert lib.b200tri_triatt_core_multi(bad, 8, None) == _lib.ERR_INVALID
