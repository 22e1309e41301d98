"""Triangle multiplicative update on B200 - host side.

Mirrors ``triangle_multiplication_forward`` of the reference
(src/foldjax/models/boltz2/models/triangle/triangle.py:33-129): same argument
names and meaning, same parameter mapping, same error text for a bad direction.
The arithmetic runs in libb200tri (hand-written sm_100a kernels); nothing here
falls back to another implementation.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Mapping

import numpy as np
import torch

from . import _device as dev
from . import _lib

C_Z = 128  # channel width of the tensor-core specialisation (other widths run the general path)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check_pair(x: torch.Tensor) -> tuple[torch.Tensor, Any]:
    """-> (the pair tensor as [B, N, N, C], the caller's leading shape). A missing batch axis is
    added and leading axes beyond one are folded into B, the way the reference's fused
    wrappers do it (src/foldjax/models/_cueq.py:89-121); the second item is what to restore."""
    lead = tuple(x.shape[:-3])
    if x.dim() < 3 or x.shape[-2] != x.shape[-3]:
        raise ValueError(f"expected a pair tensor [B, N, N, C], got shape {tuple(x.shape)}")
    if x.shape[-1] % 8 or x.shape[-1] > 1024:
        raise ValueError(f"libb200tri takes channel counts that are multiples of 8 up to 1024; got {x.shape[-1]} channels")
    return x.reshape((-1,) + tuple(x.shape[-3:])), lead


def _unfold(t: torch.Tensor, lead: tuple) -> torch.Tensor:
    return t.reshape(tuple(lead) + tuple(t.shape[1:]))


def _leaf(params: Mapping, *path: str, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    node: Any = params
    for key in path:
        node = node[key]
    if not isinstance(node, torch.Tensor) or not node.is_cuda or node.dtype != dtype:
        node = dev.to_device(node, dtype)
    return node.contiguous()


def resolve_dtype(x: Any, dtype: str | None) -> tuple[torch.dtype, int]:
    """Trunk dtype of a call: ``dtype`` if given ("bfloat16" / "float32"), else float32 for a
    float32 CUDA tensor and bfloat16 for everything else (host arrays are float32 containers
    of either trunk, so they say nothing). Returns (torch dtype, the C ABI's dtype code)."""
    if dtype is None:
        dtype = "float32" if isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32 else "bfloat16"
    name = {"bf16": "bfloat16", "fp32": "float32"}.get(str(dtype), str(dtype))
    if name == "bfloat16":
        return torch.bfloat16, _lib.DTYPE_BF16
    if name == "float32":
        return torch.float32, _lib.DTYPE_F32
    raise ValueError(f"Unsupported dtype: {dtype!r} (expected 'bfloat16' or 'float32')")


def triangle_multiplication_forward(
    params: Mapping[str, Mapping[str, Any]],
    x: Any,
    mask: Any,
    direction: str,
    eps: float = 1e-5,
    chunk_size: int = 128,
    glu_backend: str = "xla",
    contraction_precision: str = "float32",
    *,
    residual: Any | None = None,
    out: torch.Tensor | None = None,
    dtype: str | None = None,
):
    """Boltz triangle multiplication, outgoing or incoming.

    ``x`` is ``[B, N, N, 128]`` (or ``[N, N, 128]``), ``mask`` is ``[B, N, N]`` or None.
    ``dtype`` selects the trunk: "bfloat16" (default; bf16 storage, fp32 accumulation) or
    "float32" (every step in float32, the contraction as split-bf16 products on the tensor
    cores; the reference's float32 trunk, 1e-4). A float32 CUDA tensor selects float32 by
    itself. Device tensors in -> device tensor out; NumPy / CPU
    tensors in -> the inputs are copied to the GPU, the result is copied back and
    returned as the same kind of array (the end-to-end path).

    ``chunk_size``, ``glu_backend`` and ``contraction_precision`` are accepted for
    signature compatibility: a fused backend has nothing to chunk, and the
    contraction always accumulates in fp32 on the tensor cores (the reference's
    default "float32" mode).  ``residual`` (optional) fuses the caller's
    ``z + update``.
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"Unsupported triangle multiplication direction: {direction!r}")
    if contraction_precision not in ("float32", "bf16"):
        raise ValueError(f"Unsupported contraction_precision: {contraction_precision!r}")
    dev.require_cuda()
    lib = _lib.load()
    host_in = dev.is_host_array(x)
    numpy_in = isinstance(x, np.ndarray)
    tdt, code = resolve_dtype(x, dtype)
    xd, lead = _check_pair(dev.to_device(x, tdt))
    b, n, c_z = xd.shape[0], xd.shape[1], xd.shape[3]
    md = None
    if mask is not None:
        md = dev.to_device(mask, torch.float32)
        if md.dim() < 2 or tuple(md.shape[-2:]) != (n, n) or md.numel() != b * n * n:
            raise ValueError(f"mask shape {tuple(md.shape)} does not match pair tensor {tuple(x.shape)}")
        md = md.reshape(b, n, n)
    rd = None
    if residual is not None:
        rd, _ = _check_pair(dev.to_device(residual, tdt))
        dev.check_same_shape(rd, xd, "residual")
    if out is None:
        out = torch.empty_like(xd)
    else:
        if isinstance(out, torch.Tensor) and out.numel() == xd.numel() and out.is_contiguous():
            out = out.view(xd.shape) if tuple(out.shape[-3:]) == tuple(xd.shape[-3:]) else out
        dev.check_out(out, xd)
    leaves = {
        "norm_in_scale": _leaf(params, "norm_in", "scale", dtype=tdt),
        "norm_in_bias": _leaf(params, "norm_in", "bias", dtype=tdt),
        "p_in": _leaf(params, "p_in", "kernel", dtype=tdt),
        "g_in": _leaf(params, "g_in", "kernel", dtype=tdt),
        "norm_out_scale": _leaf(params, "norm_out", "scale", dtype=tdt),
        "norm_out_bias": _leaf(params, "norm_out", "bias", dtype=tdt),
        "p_out": _leaf(params, "p_out", "kernel", dtype=tdt),
        "g_out": _leaf(params, "g_out", "kernel", dtype=tdt),
    }
    c_hidden = leaves["p_out"].shape[0]
    want = {"norm_in_scale": (c_z,), "norm_in_bias": (c_z,), "p_in": (c_z, 2 * c_hidden), "g_in": (c_z, 2 * c_hidden),
            "norm_out_scale": (c_hidden,), "norm_out_bias": (c_hidden,), "p_out": (c_hidden, c_z), "g_out": (c_z, c_z)}
    for name, shape in want.items():
        if tuple(leaves[name].shape) != shape:
            raise ValueError(f"triangle multiplication parameter {name} has shape {tuple(leaves[name].shape)}, "
                             f"expected {shape} for c_z = {c_z}, c_hidden = {c_hidden}")
    if c_hidden % 8 or c_hidden > 1024:
        raise ValueError(f"libb200tri takes hidden widths that are multiples of 8 up to 1024; got {c_hidden}")
    nbytes = lib.b200tri_trimul_workspace_bytes_shape(n, code, c_z, c_hidden)
    ws = dev.workspace(nbytes, "trimul")
    for bi in range(b):
        args = _lib.TrimulArgs(
            n=n, incoming=int(direction == "incoming"), eps=float(eps),
            x=xd[bi].data_ptr(), mask=_ptr(md[bi]) if md is not None else None,
            residual=_ptr(rd[bi]) if rd is not None else None, out=out[bi].data_ptr(),
            workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes, dtype=code, c_z=c_z, c_hidden=c_hidden,
            **{k: v.data_ptr() for k, v in leaves.items()},
        )
        _lib.check(lib.b200tri_trimul_forward(C.byref(args), C.c_void_p(dev.stream_ptr())))
    result = _unfold(out, lead)
    if host_in:
        host = result.float().cpu() if numpy_in else result.cpu()
        dev.check_device_status()  # the copy synchronised: a kernel that gave up on a wait shows here
        return host.numpy() if numpy_in else host
    return result
