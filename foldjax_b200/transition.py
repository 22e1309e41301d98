"""Pair transition (SwiGLU feed-forward) on B200 - host side.

Mirrors ``transition_forward`` of the reference
(src/foldjax/models/boltz2/models/primitives/transition.py:41-127): same argument
names, same parameter mapping (``norm``/``fc1``/``fc2``/``fc3``, kernels stored
``[in, out]``), same error text for a bad ``chunk_size``. The arithmetic runs in
libb200tri (one fused sm_100a kernel per call); nothing here falls back to
another implementation.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Mapping

import numpy as np
import torch

from . import _device as dev
from . import _lib
from .triangle import C_Z, _leaf, _ptr


def transition_forward(
    params: Mapping[str, Mapping[str, Any]],
    x: Any,
    chunk_size: int | None = None,
    eps: float = 1e-5,
    row_chunk_size: int | None = None,
    glu_backend: str = "b200",
    *,
    residual: Any | None = None,
    out: torch.Tensor | None = None,
    mask: Any | None = None,
):
    """Boltz Transition block: ``(silu(LN(x) @ fc1) * (LN(x) @ fc2)) @ fc3``.

    ``x`` is ``[..., 128]`` in bf16 (the pair tensor ``[B, N, N, 128]``, a tile of
    it, or any other stack of 128-channel rows). Device tensor in -> device
    tensor out; NumPy / CPU tensor in -> copied to the GPU and back.

    ``chunk_size`` (hidden-dimension chunks) and ``row_chunk_size`` (outer-row
    blocks) exist in the reference to bound the widened ``[..., 1024]``
    intermediate; the fused kernel never materialises it, so both are validated
    and otherwise ignored, the way the reference ignores them for its fused GLU
    backend. ``residual`` (optional, may be ``x`` itself) fuses the caller's
    ``z + update``; ``out`` may alias ``x`` only if it also is the residual. ``mask`` (optional,
    one value per row, i.e. the shape of ``x`` without its channel axis) multiplies the update
    before the residual add: OpenFold3's masked transition
    (src/foldjax/models/openfold3/models/primitives.py:133-150).
    """
    if chunk_size is not None and chunk_size <= 0:
        raise ValueError(f"chunk_size must be positive, got {chunk_size}")
    dev.require_cuda()
    lib = _lib.load()
    host_in = dev.is_host_array(x)
    numpy_in = isinstance(x, np.ndarray)
    xd = dev.to_device(x, torch.bfloat16)
    if xd.dim() < 1 or xd.shape[-1] != C_Z:
        raise ValueError(f"libb200tri is built for {C_Z}-channel rows; got shape {tuple(xd.shape)}")
    rows = xd.numel() // C_Z
    rd = None
    if residual is not None:
        rd = xd if residual is x else dev.to_device(residual, torch.bfloat16)
        if rd.shape != xd.shape:
            raise ValueError(f"residual shape {tuple(rd.shape)} does not match x {tuple(xd.shape)}")
    if out is None:
        out = torch.empty_like(xd)
    else:
        dev.check_out(out, xd)
    if out.data_ptr() == xd.data_ptr() and (rd is None or rd.data_ptr() != xd.data_ptr()):
        raise ValueError("out may alias x only when x is also the residual")
    leaves = {
        "norm_scale": _leaf(params, "norm", "scale"),
        "norm_bias": _leaf(params, "norm", "bias"),
        "fc1": _leaf(params, "fc1", "kernel"),
        "fc2": _leaf(params, "fc2", "kernel"),
        "fc3": _leaf(params, "fc3", "kernel"),
    }
    hidden = leaves["fc1"].shape[-1]
    if (tuple(leaves["fc1"].shape) != (C_Z, hidden) or tuple(leaves["fc2"].shape) != (C_Z, hidden)
            or tuple(leaves["fc3"].shape) != (hidden, C_Z)):
        raise ValueError(
            f"transition kernels must be fc1/fc2 [{C_Z}, hidden] and fc3 [hidden, {C_Z}]; got "
            f"{tuple(leaves['fc1'].shape)}, {tuple(leaves['fc2'].shape)}, {tuple(leaves['fc3'].shape)}")
    if rows == 0:
        return out
    md = None
    if mask is not None:
        md = dev.to_device(mask, torch.float32)
        if md.numel() != rows:
            raise ValueError(f"mask shape {tuple(md.shape)} does not give one value per row of x {tuple(xd.shape)}")
    nbytes = lib.b200tri_pair_transition_workspace_bytes(hidden)
    ws = dev.workspace(nbytes, "pair_transition")
    args = _lib.PairTransitionArgs(
        rows=rows, channels=C_Z, hidden=hidden, eps=float(eps),
        x=xd.data_ptr(), residual=_ptr(rd), out=out.data_ptr(),
        workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes, row_mask=_ptr(md),
        **{k: v.data_ptr() for k, v in leaves.items()},
    )
    _lib.check(lib.b200tri_pair_transition(C.byref(args), C.c_void_p(dev.stream_ptr())))
    if host_in:
        host = out.float().cpu() if numpy_in else out.cpu()
        dev.check_device_status()
        return host.numpy() if numpy_in else host
    return out
