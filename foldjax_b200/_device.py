"""Device-memory plumbing for the host layer.

PyTorch is used here for exactly three things: owning device buffers, naming the
current CUDA stream, and (in ``cp``) ``torch.distributed``. No torch operator
runs on the data path; all arithmetic happens inside libb200tri.
"""

from __future__ import annotations

from typing import Any, Mapping

import numpy as np
import torch

_workspaces: dict[tuple[int, str], torch.Tensor] = {}


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("foldjax_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def workspace(nbytes: int, tag: str = "default") -> torch.Tensor:
    """A cached, grow-only scratch buffer per (device, tag); 1 KiB aligned."""
    dev = torch.cuda.current_device()
    key = (dev, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < int(nbytes) + 1024:  # callers round the pointer up by up to 1023 B
        _workspaces.pop(key, None)
        buf = torch.empty(int(nbytes) + 1024, dtype=torch.uint8, device=f"cuda:{dev}")
        _workspaces[key] = buf
    return buf


def aligned_ptr(buf: torch.Tensor, align: int = 1024) -> int:
    p = buf.data_ptr()
    return (p + align - 1) // align * align


def check_out(out: torch.Tensor, like: torch.Tensor, name: str = "out") -> torch.Tensor:
    """The caller's result buffer goes to the kernels as a raw pointer, so it must be
    exactly what they write: a contiguous CUDA bf16 tensor of the input's shape on the
    input's device. Anything else would be a write past the buffer, not a Python error."""
    if not isinstance(out, torch.Tensor):
        raise ValueError(f"{name} must be a torch tensor, got {type(out).__name__}")
    if out.dtype != like.dtype:
        raise ValueError(f"{name} must be {like.dtype}, got {out.dtype}")
    if tuple(out.shape) != tuple(like.shape):
        raise ValueError(f"{name} shape {tuple(out.shape)} does not match the input {tuple(like.shape)}")
    if not out.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if not out.is_cuda or out.device != like.device:
        raise ValueError(f"{name} must be a CUDA tensor on the input's device ({like.device}), got {out.device}")
    return out


def check_same_shape(t: torch.Tensor, like: torch.Tensor, name: str) -> torch.Tensor:
    if tuple(t.shape) != tuple(like.shape):
        raise ValueError(f"{name} shape {tuple(t.shape)} does not match the input {tuple(like.shape)}")
    return t


def check_device_status() -> None:
    """Read (and clear) the device status word at a point where the host synchronises
    anyway; raises if a kernel gave up on a bounded wait since the last check."""
    from . import _lib

    _lib.device_status()


def release_workspaces() -> None:
    _workspaces.clear()


def to_device(x: Any, dtype: torch.dtype | None = None, device: torch.device | None = None) -> torch.Tensor:
    """numpy / torch (any device) -> contiguous CUDA tensor of `dtype`."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    if isinstance(x, np.ndarray):
        if x.dtype.name == "bfloat16":  # ml_dtypes
            t = torch.from_numpy(x.view(np.uint16).copy()).view(torch.bfloat16)
        else:
            t = torch.from_numpy(np.ascontiguousarray(x))
    elif isinstance(x, torch.Tensor):
        t = x
    else:
        t = torch.as_tensor(np.asarray(x))
    t = t.to(device=device, dtype=dtype or t.dtype, non_blocking=True)
    return t.contiguous()


def params_to_device(params: Mapping, dtype: torch.dtype = torch.bfloat16, device=None):
    """Move a nested parameter mapping to the device in the trunk dtype."""
    if isinstance(params, Mapping):
        return {k: params_to_device(v, dtype, device) for k, v in params.items()}
    return to_device(params, dtype, device)


def is_host_array(x: Any) -> bool:
    return isinstance(x, np.ndarray) or (isinstance(x, torch.Tensor) and not x.is_cuda)
