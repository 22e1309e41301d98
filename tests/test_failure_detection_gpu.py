"""A bounded device wait that runs out is reported to the host and leaves the GPU usable.

No kernel is hung or faulted here: ``b200tri_selftest_wait`` enqueues a one-warp kernel that
waits, through the library's ordinary bounded wait, on a barrier nothing arrives at, with a
limit of about a millisecond. The kernel gives up by itself, records its role code in the
device status word and returns."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import triangle_oracle as orc

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_expired_wait_is_reported_and_the_context_stays_usable(cuda_device):
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.transition import transition_forward

    lib = _lib.load()
    assert lib.b200tri_device_status() == 0
    _lib.check(lib.b200tri_selftest_wait(2_000_000, dev.stream_ptr()))  # ~1 ms of SM clock
    with pytest.raises(_lib.B200TriError) as info:
        _lib.device_status()
    assert info.value.code == _lib.ERR_TIMEOUT
    assert "B200TRI_ERR_TIMEOUT" in str(info.value) and "110" in str(info.value)
    assert lib.b200tri_device_status() == 0  # reading the word cleared it
    # the next real kernel runs and is right
    rng = np.random.default_rng(1)
    params = orc.round_params(orc.random_transition_params(rng), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((4, 40, 128)).astype(np.float32))
    got = transition_forward(params, x)
    ref = orc.transition(params, x, dtype="bfloat16")
    assert orc.error_vs(ref, got)["mean_abs_over_rms"] < 2e-3
    assert lib.b200tri_device_status() == 0


def test_host_path_raises_when_a_kernel_gave_up(cuda_device):
    """The operators read the status word where they synchronise anyway (the copy back to
    host memory), so a timeout is an exception there instead of a silently partial result."""
    from foldjax_b200 import _device as dev, _lib
    from foldjax_b200.transition import transition_forward

    lib = _lib.load()
    rng = np.random.default_rng(2)
    params = orc.round_params(orc.random_transition_params(rng), "bfloat16")
    x = orc.round_bf16(rng.standard_normal((2, 16, 128)).astype(np.float32))
    _lib.check(lib.b200tri_selftest_wait(1_000_000, dev.stream_ptr()))
    with pytest.raises(_lib.B200TriError, match="B200TRI_ERR_TIMEOUT"):
        transition_forward(params, x)  # host array in -> copy back -> status check
    assert lib.b200tri_device_status() == 0
    transition_forward(params, x)


def test_selftest_rejects_unbounded_limits(cuda_device):
    from foldjax_b200 import _lib

    lib = _lib.load()
    assert lib.b200tri_selftest_wait(0, None) == _lib.ERR_INVALID
    assert lib.b200tri_selftest_wait(10**12, None) == _lib.ERR_INVALID
