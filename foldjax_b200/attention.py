"""Single-representation attention with pair bias on B200 - host side.

Mirrors ``attention_pair_bias_forward`` of the reference
(src/foldjax/models/boltz2/models/primitives/attention.py:19-140): same argument
names and parameter mapping (``proj_q`` with bias, ``proj_k``, ``proj_v``, ``proj_g``,
``proj_z_norm``, ``proj_z``, ``proj_o``; kernels stored ``[in, out]``). The
arithmetic runs in libb200tri; nothing here falls back to another implementation.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Mapping

import numpy as np
import torch

from . import _device as dev
from . import _lib
from .triangle import C_Z, _leaf

HEAD_DIM = 24  # head width the token-attention kernel is built for


def attention_pair_bias_forward(
    params: Mapping[str, Mapping[str, Any]],
    s: Any,
    z: Any,
    mask: Any,
    k_in: Any | None = None,
    multiplicity: int = 1,
    inf: float = 1e6,
    eps: float = 1e-5,
    chunk_size: int | None = None,
    attention_backend: str = "b200",
):
    """Boltz AttentionPairBias: ``s [B, N, c_s]`` (fp32, already layer-normed by the
    caller), ``z [B, N, N, 128]`` (read as bf16, the trunk dtype), ``mask [B, N]``.
    Returns the fp32 update ``[B, N, c_s]``; device tensors in -> device tensor out,
    NumPy / CPU tensors in -> copied to the GPU and back.

    ``chunk_size`` (query blocking) bounds a score tensor the fused path never
    materialises: accepted and ignored. ``multiplicity`` other than 1 (the diffusion
    module's use) is not supported.
    """
    if multiplicity != 1:
        raise ValueError("multiplicity != 1 is not supported by the b200 backend")
    dev.require_cuda()
    lib = _lib.load()
    host_in = dev.is_host_array(s)
    numpy_in = isinstance(s, np.ndarray)
    sd = dev.to_device(s, torch.float32)
    kd = sd if k_in is None else dev.to_device(k_in, torch.float32)
    zd = dev.to_device(z, torch.bfloat16)
    md = dev.to_device(mask, torch.float32)
    if sd.dim() != 3 or zd.dim() != 4 or md.dim() != 2:
        raise ValueError(f"expected s [B,N,c_s], z [B,N,N,c_z], mask [B,N]; got {tuple(sd.shape)}, {tuple(zd.shape)}, {tuple(md.shape)}")
    b, n, c_s = sd.shape
    if tuple(zd.shape) != (b, n, n, C_Z) or tuple(md.shape) != (b, n) or kd.shape != sd.shape:
        raise ValueError(f"shapes do not match: s {tuple(sd.shape)}, k_in {tuple(kd.shape)}, z {tuple(zd.shape)}, mask {tuple(md.shape)}")
    lv = {
        "proj_q": _leaf(params, "proj_q", "kernel"), "proj_q_bias": _leaf(params, "proj_q", "bias"),
        "proj_k": _leaf(params, "proj_k", "kernel"), "proj_v": _leaf(params, "proj_v", "kernel"),
        "proj_g": _leaf(params, "proj_g", "kernel"),
        "proj_z_norm_scale": _leaf(params, "proj_z_norm", "scale"), "proj_z_norm_bias": _leaf(params, "proj_z_norm", "bias"),
        "proj_z": _leaf(params, "proj_z", "kernel"), "proj_o": _leaf(params, "proj_o", "kernel"),
    }
    heads = lv["proj_z"].shape[-1]
    if c_s != heads * HEAD_DIM or tuple(lv["proj_q"].shape) != (c_s, c_s) or tuple(lv["proj_z"].shape) != (C_Z, heads):
        raise ValueError(f"libb200tri is built for heads of width {HEAD_DIM} and c_z = {C_Z}; got c_s {c_s}, {heads} heads")
    out = torch.empty_like(sd)
    nbytes = lib.b200tri_attention_pair_bias_workspace_bytes(n, c_s, heads)
    ws = dev.workspace(nbytes, "attention_pair_bias")
    for bi in range(b):
        args = _lib.AttentionPairBiasArgs(
            n=n, c_s=c_s, c_z=C_Z, heads=heads, eps=float(eps), inf=float(inf),
            s=sd[bi].data_ptr(), k_in=kd[bi].data_ptr(), z=zd[bi].data_ptr(), mask=md[bi].data_ptr(),
            out=out[bi].data_ptr(), workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes,
            **{k: v.data_ptr() for k, v in lv.items()},
        )
        _lib.check(lib.b200tri_attention_pair_bias(C.byref(args), C.c_void_p(dev.stream_ptr())))
    if host_in:
        host = out.cpu()
        return host.numpy() if numpy_in else host
    return out
