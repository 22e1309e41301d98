"""Host-side argument checks that run before any kernel launch (no GPU needed).

The operators hand raw pointers to the kernels, so a result buffer of the wrong
size, dtype or layout must be refused in Python: on the device it would be a write
past the allocation."""

from __future__ import annotations

import pytest

torch = pytest.importorskip("torch")

from foldjax_b200 import _device as dev


def test_out_buffer_must_match_the_input_exactly():
    like = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="shape"):
        dev.check_out(torch.zeros(1, 7, 8, 128, dtype=torch.bfloat16), like)
    with pytest.raises(ValueError, match="bfloat16"):
        dev.check_out(torch.zeros(1, 8, 8, 128, dtype=torch.float32), like)
    with pytest.raises(ValueError, match="contiguous"):
        dev.check_out(torch.zeros(1, 8, 128, 8, dtype=torch.bfloat16).transpose(2, 3), like)
    with pytest.raises(ValueError, match="torch tensor"):
        dev.check_out([1, 2, 3], like)
    # right shape, dtype and layout, but host memory: the kernels cannot write there
    with pytest.raises(ValueError, match="CUDA tensor"):
        dev.check_out(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16), like)


def test_residual_shape_is_compared_with_the_input():
    like = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="residual shape"):
        dev.check_same_shape(torch.zeros(1, 4, 4, 128), like, "residual")
    assert dev.check_same_shape(like, like, "residual") is like


def test_workspace_reuse_accounts_for_the_alignment_slack(monkeypatch):
    """A cached buffer is reused only if it still covers the request after the pointer
    has been rounded up to 1 KiB."""
    real_empty = torch.empty

    def fake_empty(n, dtype=None, device=None):
        return real_empty(int(n), dtype=torch.uint8)

    monkeypatch.setattr(dev.torch, "empty", fake_empty)
    monkeypatch.setattr(dev.torch.cuda, "current_device", lambda: 0)
    dev.release_workspaces()
    a = dev.workspace(4096, "t")
    assert a.numel() == 4096 + 1024
    assert dev.workspace(4096, "t") is a
    assert dev.workspace(3000, "t") is a
    b = dev.workspace(4097, "t")  # 4097 + 1024 > 5120: the old buffer no longer covers it
    assert b is not a and b.numel() == 4097 + 1024
    dev.release_workspaces()


def test_streamed_blocks_refuse_mismatched_host_buffers():
    """stream_host_blocks checks its host buffers before it touches a device."""
    from foldjax_b200.block import stream_host_blocks

    z = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16)
    run = lambda zd, md: zd + 1  # never reached
    assert stream_host_blocks(run, []) == []
    with pytest.raises(ValueError, match="bfloat16"):
        stream_host_blocks(run, [(z.float(), None)], [z.clone()])
    with pytest.raises(ValueError, match="same shape"):
        stream_host_blocks(run, [(z, None), (z[:, :4].contiguous(), None)], [z.clone(), z.clone()])
    with pytest.raises(ValueError, match="float32"):
        stream_host_blocks(run, [(z, torch.ones(1, 8, 8, dtype=torch.float64))], [z.clone()])
    with pytest.raises(ValueError, match="1 items but 2"):
        stream_host_blocks(run, [(z, None)], [z.clone(), z.clone()])
    with pytest.raises(ValueError, match="outputs must be"):
        stream_host_blocks(run, [(z, None)], [z.float()])


def test_block_variant_names_are_checked_before_any_device_work():
    from foldjax_b200.pairformer import VARIANTS, pairformer_forward

    assert set(VARIANTS) == {"boltz2", "protenix", "openfold3"}
    z = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Unsupported pairformer variant"):
        pairformer_forward([{}], None, z, None, None, variant="alphafold2")
