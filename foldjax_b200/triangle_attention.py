"""Triangle attention (starting / ending node) on B200 - host side.

Mirrors ``triangle_attention_forward`` of the reference
(src/foldjax/models/boltz2/models/triangle/triangle_attention.py:79-162) and the
attention-core operator its fused backends implement
(``pallas_attention_core``, triangle_attention_pallas.py:180; ``cueq_attention_core``,
src/foldjax/models/_cueq.py:66). Same argument names and meaning; chunking knobs
are accepted and ignored, as the reference's fused backends do.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Mapping

import numpy as np
import torch

from . import _device as dev
from . import _lib
from .triangle import C_Z, _check_pair, _leaf, _ptr, _unfold, resolve_dtype

HEADS = 4
HEAD_DIM = 32


def triangle_attention_forward(
    params: Mapping[str, Any],
    x: Any,
    mask: Any | None = None,
    starting: bool = True,
    inf: float = 1e9,
    eps: float = 1e-5,
    chunk_size: int = 128,
    q_chunk_size: int | None = None,
    matmul_precision: str = "highest",
    triangle_backend: str = "b200",
    *,
    residual: Any | None = None,
    out: torch.Tensor | None = None,
    dtype: str | None = None,
):
    """Boltz TriangleAttention, starting or ending node.

    ``x`` is ``[B, N, N, 128]`` (or ``[N, N, 128]``), ``mask`` ``[B, N, N]`` or None (= ones).
    ``dtype`` selects the trunk: "bfloat16" (default) or "float32" (every step in float32 on
    the CUDA cores, the reference's float32 trunk, 1e-4); a float32 CUDA tensor selects
    float32 by itself. ``params`` is the reference's mapping ``{"layer_norm": {scale,
    bias}, "linear": {kernel [128, 4]}, "mha": {"linear_q" | "linear_k" |
    "linear_v" | "linear_g" | "linear_o": {kernel [128, 128]}}}``. Device tensors in
    -> device tensor out; NumPy / CPU tensors in -> copied to the GPU and back.
    """
    if triangle_backend != "b200":
        raise ValueError(f"Unsupported triangle_backend: {triangle_backend!r}")
    if matmul_precision.lower() not in ("highest", "float32", "fp32", "default", "tensorfloat32", "tf32"):
        raise ValueError(f"Unsupported matmul_precision: {matmul_precision!r}")
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
        "norm_scale": _leaf(params, "layer_norm", "scale", dtype=tdt),
        "norm_bias": _leaf(params, "layer_norm", "bias", dtype=tdt),
        "w_bias": _leaf(params, "linear", "kernel", dtype=tdt),
        "w_q": _leaf(params, "mha", "linear_q", "kernel", dtype=tdt),
        "w_k": _leaf(params, "mha", "linear_k", "kernel", dtype=tdt),
        "w_v": _leaf(params, "mha", "linear_v", "kernel", dtype=tdt),
        "w_g": _leaf(params, "mha", "linear_g", "kernel", dtype=tdt),
        "w_o": _leaf(params, "mha", "linear_o", "kernel", dtype=tdt),
    }
    heads = leaves["w_bias"].shape[-1]
    width = leaves["w_g"].shape[-1]
    head_dim = width // max(heads, 1)
    want = {"norm_scale": (c_z,), "norm_bias": (c_z,), "w_bias": (c_z, heads), "w_q": (c_z, width), "w_k": (c_z, width),
            "w_v": (c_z, width), "w_g": (c_z, width), "w_o": (width, c_z)}
    for name, shape in want.items():
        if tuple(leaves[name].shape) != shape:
            raise ValueError(f"triangle attention parameter {name} has shape {tuple(leaves[name].shape)}, expected "
                             f"{shape} for c_z = {c_z}, {heads} heads x {head_dim}")
    if heads * head_dim != width or head_dim not in (8, 16, 24, 32, 48, 64):
        raise ValueError(f"libb200tri takes head widths 8, 16, 24, 32, 48 and 64; got {heads} heads over {width} channels")
    nbytes = lib.b200tri_triatt_workspace_bytes_shape(n, code, c_z, heads, head_dim)
    ws = dev.workspace(nbytes, "triatt")
    for bi in range(b):
        args = _lib.TriattArgs(
            n=n, starting=int(bool(starting)), heads=heads, head_dim=head_dim, inf=float(inf), eps=float(eps),
            x=xd[bi].data_ptr(), mask=_ptr(md[bi]) if md is not None else None,
            residual=_ptr(rd[bi]) if rd is not None else None, out=out[bi].data_ptr(),
            workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes, dtype=code, c_z=c_z,
            **{k: v.data_ptr() for k, v in leaves.items()},
        )
        _lib.check(lib.b200tri_triatt_forward(C.byref(args), C.c_void_p(dev.stream_ptr())))
    result = _unfold(out, lead)
    if host_in:
        host = result.float().cpu() if numpy_in else result.cpu()
        dev.check_device_status()  # the copy synchronised: a kernel that gave up on a wait shows here
        return host.numpy() if numpy_in else host
    return result


def attention_core(q, k, v, tri_bias, mask_bias, scale: float | None = None):
    """The attention-core operator: ``core(q, k, v, tri_bias, mask_bias[, scale]) -> out``.

    q/k/v ``[B, I, H, J, D]`` device tensors (q pre-scaled unless ``scale`` is given, the
    cuEquivariance convention of src/foldjax/models/_cueq.py:66-121: q is then multiplied by
    ``scale`` cast to q's dtype and the product rounded to that dtype, as the reference's
    Protenix path does, triangle.py:563,792), ``tri_bias [B, 1, H, J, K]``, ``mask_bias
    [B, I, 1, 1, K]`` additive fp32 (0, a soft bias, -1e9 or -inf). Returns ``[B, I, H, J, D]``
    in ``v.dtype``. Leading axes beyond five are folded into B.

    The additive mask bias goes to the kernel as it is (no round trip through a 0/1 mask), so
    soft and hard entries can be mixed; a row with no kept key comes out as the uniform average
    over its keys, the convention of the finite -1e9 mask (triangle_attention.py:138-142), not as
    the zeros of the reference's 2-D ring (src/foldjax/models/_cp_attention.py:380-385).
    Enqueue-only: nothing here waits for the device. The operands are re-laid out for the
    kernel with torch copies (q,k -> [I,J,H*D], v -> [I,H*D,K] fp16, bias -> [H,J,K]); the
    module-level forward avoids those copies by producing that layout directly.
    """
    dev.require_cuda()
    lib = _lib.load()
    lead = q.shape[:-4]
    qf = q.reshape((-1,) + tuple(q.shape[-4:]))
    kf = k.reshape((-1,) + tuple(k.shape[-4:]))
    vf = v.reshape((-1,) + tuple(v.shape[-4:]))
    bf = tri_bias.reshape((-1,) + tuple(tri_bias.shape[-4:]))
    mf = mask_bias.reshape((-1,) + tuple(mask_bias.shape[-4:]))
    bsz, n_i, h, n_j, d = qf.shape
    n_k = kf.shape[-2]
    if (h, d) != (HEADS, HEAD_DIM):
        raise ValueError(f"libb200tri is built for 4 heads x 32; got {h} x {d}")
    if tuple(mf.shape[1:]) != (n_i, 1, 1, n_k) or tuple(bf.shape[1:]) != (1, h, n_j, n_k):
        raise ValueError(f"mask_bias {tuple(mask_bias.shape)} / tri_bias {tuple(tri_bias.shape)} do not match "
                         f"q {tuple(q.shape)} and k {tuple(k.shape)}")
    qf = qf.to(torch.bfloat16)
    if scale is not None:
        qf = qf * torch.tensor(float(scale), dtype=torch.bfloat16, device=qf.device)  # one bf16 rounding
    ld = (n_k + 63) // 64 * 64
    out = torch.empty((bsz, n_i, h, n_j, d), dtype=v.dtype, device=v.device)
    nbytes = lib.b200tri_triatt_core_workspace_bytes(n_i, n_k)
    ws = dev.workspace(nbytes, "triatt_core")
    for bi in range(bsz):
        q2 = qf[bi].permute(0, 2, 1, 3).reshape(n_i, n_j, h * d).contiguous()
        k2 = kf[bi].permute(0, 2, 1, 3).reshape(n_i, n_k, h * d).to(torch.bfloat16).contiguous()
        v2 = torch.zeros(n_i, h * d, ld, dtype=torch.float16, device=v.device)
        v2[:, :, :n_k] = vf[bi].permute(0, 1, 3, 2).reshape(n_i, h * d, n_k).to(torch.float16)
        b2 = torch.zeros(h, n_j, ld, dtype=torch.bfloat16, device=v.device)
        b2[:, :, :n_k] = bf[bi, 0].to(torch.bfloat16)
        mb = mf[bi, :, 0, 0, :].float().contiguous()
        o2 = torch.empty(n_i, n_j, h * d, dtype=torch.bfloat16, device=v.device)
        args = _lib.TriattCoreArgs(
            n_i=n_i, n_j=n_j, n_k=n_k, heads=h, head_dim=d,
            q=q2.data_ptr(), k=k2.data_ptr(), vt=v2.data_ptr(), v_ld=ld,
            bias=b2.data_ptr(), bias_ld=ld, bias_head_stride=n_j * ld,
            mask=mb.data_ptr(), ms_i=n_k, ms_k=1, inf=0.0, mask_additive=1,
            o=o2.data_ptr(), row_max=None, row_sum=None, unnormalized=0,
            workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes,
        )
        _lib.check(lib.b200tri_triatt_core(C.byref(args), C.c_void_p(dev.stream_ptr())))
        out[bi] = o2.reshape(n_i, n_j, h, d).permute(0, 2, 1, 3).to(v.dtype)
    return out.reshape(tuple(lead) + tuple(out.shape[1:]))
