"""The whole Pairformer block and a stack of blocks as ONE library call
(b200tri_pairformer_forward), against the oracle's restatement of
pairformer_layer_forward and against the per-op entry points.

Tolerance: the pair tensor in the benchmark's bf16 budget (conftest.assert_parity)
against the oracle's bf16 emulation; the float32 single track at mean-abs <= 2e-3 and
max-abs <= 2e-2 of its RMS (it reads the bf16 pair tensor through the pair-bias
projection, so it inherits the pair track's rounding differences)."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_parity
from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _case(seed, n, n_pad, ln_noise=0.1, std=0.03):
    rng = np.random.default_rng(seed)
    params = orc.round_params(orc.random_pairformer_params(rng, std=std, ln_noise=ln_noise), "bfloat16")
    z = orc.round_bf16(rng.standard_normal((1, n, n, 128)).astype(np.float32))
    s = rng.standard_normal((1, n, 384)).astype(np.float32)
    pair_mask = orc.pad_mask(n, n_pad)
    mask = np.ones((1, n), np.float32)
    if n_pad:
        mask[0, n - n_pad:] = 0.0
    return params, s, z, mask, pair_mask


@pytest.mark.parametrize("n,n_pad", [(64, 0), (136, 9)])
def test_block_matches_the_oracle(cuda_device, n, n_pad):
    from foldjax_b200 import _lib
    from foldjax_b200.pairformer import pairformer_layer_forward

    params, s, z, mask, pair_mask = _case(n, n, n_pad)
    s_got, z_got = pairformer_layer_forward(params, s, z, mask, pair_mask)
    _lib.device_status()
    s_ref, z_ref = orc.pairformer_layer(params, s, z, mask, pair_mask, dtype="bfloat16")
    valid = (pair_mask[0].any(axis=1)[:, None] & pair_mask[0].any(axis=0)[None, :])[None, :, :, None]
    print(assert_parity(z_ref, z_got, where=np.broadcast_to(valid, z_ref.shape), label=f"block z N={n}"))
    tok = mask[0].astype(bool)
    err = orc.error_vs(s_ref[0][tok], s_got[0][tok])
    print(f"block s N={n}: {err}")
    assert err["mean_abs_over_rms"] < 2e-3 and err["max_abs_over_rms"] < 2e-2, err
    # the update of s is not a no-op, and z really went through the block
    assert orc.error_vs(s[0][tok], s_got[0][tok])["mean_abs_over_rms"] > 1e-2
    assert not np.array_equal(z_got, z)


def test_trunk_call_equals_block_by_block_and_stacked_leaves(cuda_device):
    """Three blocks in one call == three one-block calls, bit for bit; stacked [L, ...] leaves
    (what the reference's scan carries) == a list of per-block mappings."""
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.pairformer import pairformer_forward

    n, blocks = 72, 3
    rng = np.random.default_rng(5)
    layers = [orc.round_params(orc.random_pairformer_params(rng, std=0.03, ln_noise=0.1), "bfloat16")
              for _ in range(blocks)]
    _, s, z, mask, pair_mask = _case(6, n, 5)
    sd, zd = dev.to_device(s, torch.float32), dev.to_device(z, torch.bfloat16)
    md, pmd = dev.to_device(mask, torch.float32), dev.to_device(pair_mask, torch.float32)
    s_all, z_all = pairformer_forward(layers, sd, zd, md, pmd)
    s_it, z_it = sd, zd
    for layer in layers:
        s_it, z_it = pairformer_forward([layer], s_it, z_it, md, pmd)
    _lib.device_status()
    assert torch.equal(z_all, z_it) and torch.equal(s_all, s_it)

    def stack(nodes):
        if isinstance(nodes[0], dict):
            return {k: stack([node[k] for node in nodes]) for k in nodes[0]}
        return np.stack(nodes)

    s_st, z_st = pairformer_forward(stack(layers), sd, zd, md, pmd, num_blocks=blocks)
    assert torch.equal(z_st, z_all) and torch.equal(s_st, s_all)
    assert torch.equal(zd, dev.to_device(z, torch.bfloat16))  # inputs untouched


def test_pair_track_only_equals_the_per_op_block(cuda_device):
    from foldjax_b200 import _device as dev
    from foldjax_b200.block import triangle_block_forward
    from foldjax_b200.pairformer import pairformer_forward

    params, _, z, _, pair_mask = _case(9, 80, 6)
    zd, pmd = dev.to_device(z, torch.bfloat16), dev.to_device(pair_mask, torch.float32)
    pd = dev.params_to_device(params)
    s_none, z_one = pairformer_forward([params], None, zd, None, pmd)
    assert s_none is None
    assert torch.equal(z_one, triangle_block_forward(pd, zd, pmd))


@pytest.mark.parametrize("variant,flags", [
    ("protenix", dict(pair_gate=True)),
    ("openfold3", dict(mask_transition=True)),
    ("boltz2", dict(attention_first=True)),
])
def test_block_variants_match_the_oracle(cuda_device, variant, flags):
    """The block orders of the other model families: Protenix's pair gate (with a mask that is
    NOT an outer product, so the gate before the first update matters), OpenFold3's masked
    transition, and attention before multiplication."""
    from foldjax_b200 import _lib
    from foldjax_b200.pairformer import pairformer_forward

    params, s, z, mask, pair_mask = _case(21, 72, 7)
    pair_mask = pair_mask.copy()
    rng = np.random.default_rng(5)
    drop = rng.random(pair_mask.shape) < 0.05
    drop[0, np.arange(72), np.arange(72)] = False  # the diagonal (the token gate) stays as padded
    pair_mask[drop] = 0.0
    kw = dict(attention_first=True) if "attention_first" in flags else {}
    s_got, z_got = pairformer_forward([params], s, z, mask, pair_mask, variant=variant, **kw)
    _lib.device_status()
    s_ref, z_ref = orc.pairformer_layer(params, s, z, mask, pair_mask, dtype="bfloat16", **flags)
    rows_ok = pair_mask[0].any(axis=1)
    valid = (rows_ok[:, None] & pair_mask[0].any(axis=0)[None, :])[None, :, :, None]
    # attention first puts the op with the largest rounding noise (fp16 P, 5e-4 of RMS) in front
    # of three more ops: the chained mean error triples (1.1e-3, still inside 2e-3) and one
    # element in half a million passes 2e-2 of RMS, so the max-abs bound is 3e-2 for that order
    print(assert_parity(z_ref, z_got, where=np.broadcast_to(valid, z_ref.shape), label=f"block z, {variant} {flags}",
                        max_tol=3e-2 if "attention_first" in flags else 2e-2))
    tok = mask[0].astype(bool)
    err = orc.error_vs(s_ref[0][tok], s_got[0][tok])
    print(f"block s, {variant}: {err}")
    assert err["mean_abs_over_rms"] < 2e-3 and err["max_abs_over_rms"] < 2e-2, err
    if variant == "protenix":
        assert np.all(z_got[0][pair_mask[0] == 0] == 0.0) and np.all(s_got[0][~tok] == 0.0)
    # the variant does change the result
    _, z_plain = pairformer_forward([params], s, z, mask, pair_mask)
    assert not np.array_equal(z_plain, z_got)


def test_streamed_host_blocks_equal_one_call_each(cuda_device):
    """stream_host_blocks (copies of neighbouring items overlapped with the kernels) gives, item
    by item, exactly what triangle_block_forward gives for that item alone; five different
    items, so both device slots are reused while their neighbours are still in flight."""
    from foldjax_b200 import _device as dev
    from foldjax_b200.block import triangle_block_forward, triangle_block_forward_stream

    params, _, z, _, pair_mask = _case(11, 136, 5)
    pd = dev.params_to_device(params)
    gen = torch.Generator().manual_seed(3)
    items = []
    for k in range(5):
        zk = (torch.from_numpy(z).float() + 0.25 * k * torch.randn(z.shape, generator=gen)).bfloat16().pin_memory()
        mk = torch.from_numpy(pair_mask).float().clone()
        if k % 2:
            mk[:, :, : 3 + k] = 0.0
        items.append((zk, mk.pin_memory()))
    outs = triangle_block_forward_stream(pd, items)
    assert len(outs) == 5
    for (zk, mk), got in zip(items, outs):
        want = triangle_block_forward(pd, zk.cuda(), mk.cuda()).cpu()
        assert torch.equal(got, want)
    assert not torch.equal(outs[0], outs[2])


def test_bad_arguments_are_rejected(cuda_device):
    from foldjax_b200 import _lib
    from foldjax_b200.pairformer import pairformer_forward, pairformer_layer_forward

    params, s, z, mask, pair_mask = _case(2, 16, 0)
    with pytest.raises(ValueError, match="Unsupported triangle_backend"):
        pairformer_layer_forward(params, s, z, mask, pair_mask, triangle_backend="pallas")
    with pytest.raises(ValueError, match="does not match"):
        pairformer_forward([params], s[:, :8], z, mask, pair_mask)
    with pytest.raises(ValueError, match="at least one block"):
        pairformer_forward([], s, z, mask, pair_mask)
    lib = _lib.load()
    assert lib.b200tri_pairformer_forward(None, None) == _lib.ERR_INVALID
