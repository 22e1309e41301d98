"""One Pairformer block, or a stack of them, as a single library call - host side.

Mirrors ``pairformer_layer_forward`` of the reference
(src/foldjax/models/boltz2/models/trunk_blocks/pairformer.py:100-206: same argument names,
same parameter mapping ``tri_mul_out`` / ``tri_mul_in`` / ``tri_att_start`` /
``tri_att_end`` / ``transition_z`` / ``pre_norm_s`` / ``attention`` / ``transition_s``,
returns ``(s, z)``) and the scan over stacked layers around it (pairformer.py:30-100).
The whole block - pair track in bf16 on the tensor cores, single track in float32 - is ONE
call of ``b200tri_pairformer_forward``; a list of per-layer mappings, or one mapping whose
leaves carry a leading layer axis (what the reference's scan carries, _stacking.py), runs
the whole stack in one call.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Mapping, Sequence

import numpy as np
import torch

from . import _device as dev
from . import _lib
from .triangle import C_Z

_TRIMUL = {"norm_in_scale": ("norm_in", "scale"), "norm_in_bias": ("norm_in", "bias"), "p_in": ("p_in", "kernel"),
           "g_in": ("g_in", "kernel"), "norm_out_scale": ("norm_out", "scale"), "norm_out_bias": ("norm_out", "bias"),
           "p_out": ("p_out", "kernel"), "g_out": ("g_out", "kernel")}
_TRIATT = {"norm_scale": ("layer_norm", "scale"), "norm_bias": ("layer_norm", "bias"), "w_bias": ("linear", "kernel"),
           "w_q": ("mha", "linear_q", "kernel"), "w_k": ("mha", "linear_k", "kernel"),
           "w_v": ("mha", "linear_v", "kernel"), "w_g": ("mha", "linear_g", "kernel"),
           "w_o": ("mha", "linear_o", "kernel")}
_TRANS = {"norm_scale": ("norm", "scale"), "norm_bias": ("norm", "bias"), "fc1": ("fc1", "kernel"),
          "fc2": ("fc2", "kernel"), "fc3": ("fc3", "kernel")}
_ATT = {"proj_q": ("proj_q", "kernel"), "proj_q_bias": ("proj_q", "bias"), "proj_k": ("proj_k", "kernel"),
        "proj_v": ("proj_v", "kernel"), "proj_g": ("proj_g", "kernel"),
        "proj_z_norm_scale": ("proj_z_norm", "scale"), "proj_z_norm_bias": ("proj_z_norm", "bias"),
        "proj_z": ("proj_z", "kernel"), "proj_o": ("proj_o", "kernel")}


def _get(node: Any, path: tuple[str, ...]) -> Any:
    for key in path:
        node = node[key]
    return node


class _Packed:
    """Device copies of one block's (or one stack's) parameters and the C struct pointing at them."""

    def __init__(self, params: Mapping[str, Any], single: bool):
        self.keep: list[torch.Tensor] = []
        self.struct = _lib.PairformerBlockParams()

        def ptr(node: Any) -> int:
            t = node if isinstance(node, torch.Tensor) and node.is_cuda and node.dtype == torch.bfloat16 else \
                dev.to_device(node, torch.bfloat16)
            t = t.contiguous()
            self.keep.append(t)
            return t.data_ptr()

        def fill(dst, table, src):
            for field_name, path in table.items():
                setattr(dst, field_name, ptr(_get(src, path)))

        fill(self.struct.tri_mul_out, _TRIMUL, params["tri_mul_out"])
        fill(self.struct.tri_mul_in, _TRIMUL, params["tri_mul_in"])
        fill(self.struct.tri_att_start, _TRIATT, params["tri_att_start"])
        fill(self.struct.tri_att_end, _TRIATT, params["tri_att_end"])
        fill(self.struct.transition_z, _TRANS, params["transition_z"])
        self.struct.transition_z.hidden = int(np.shape(_get(params["transition_z"], ("fc1", "kernel")))[-1])
        self.heads_s = 0
        if single:
            self.struct.pre_norm_s_scale = ptr(params["pre_norm_s"]["scale"])
            self.struct.pre_norm_s_bias = ptr(params["pre_norm_s"]["bias"])
            fill(self.struct.attention, _ATT, params["attention"])
            fill(self.struct.transition_s, _TRANS, params["transition_s"])
            self.struct.transition_s.hidden = int(np.shape(_get(params["transition_s"], ("fc1", "kernel")))[-1])
            self.heads_s = int(np.shape(_get(params["attention"], ("proj_z", "kernel")))[-1])


#: what distinguishes the block of each model family at the level of this driver
VARIANTS = {
    "boltz2": {"pair_gate": False, "mask_transition": False},
    "protenix": {"pair_gate": True, "mask_transition": False},
    "openfold3": {"pair_gate": False, "mask_transition": True},
}


def pairformer_forward(
    params: Mapping[str, Any] | Sequence[Mapping[str, Any]],
    s: Any | None,
    z: Any,
    mask: Any | None,
    pair_mask: Any | None,
    eps: float = 1e-5,
    *,
    num_blocks: int | None = None,
    tri_inf: float = 1e9,
    att_inf: float = 1e6,
    variant: str = "boltz2",
    pair_gate: bool | None = None,
    mask_transition: bool | None = None,
    attention_first: bool = False,
):
    """Run a stack of Pairformer blocks in one library call and return ``(s, z)``.

    ``params``: a sequence of per-block mappings, or ONE mapping with stacked leaves
    ``[num_blocks, ...]`` (pass ``num_blocks``). ``s`` ``[B, N, c_s]`` float32 or None (pair
    track only), ``z`` ``[B, N, N, 128]`` bf16, ``mask`` ``[B, N]``, ``pair_mask`` ``[B, N, N]``.
    Device tensors in -> device tensors out (the inputs are not modified); host arrays in ->
    copied to the GPU and back.

    ``variant`` picks the block order of a model family: "boltz2" (default), "protenix" (the
    pair tensor is multiplied by the pair mask before the first update and after every update,
    the single track by the token mask, which defaults to the pair mask's diagonal:
    protenix/models/trunk_blocks/pairformer.py:71-180) or "openfold3" (the pair transition's
    update is multiplied by the pair mask: openfold3/models/pair_block.py:174-183).
    ``pair_gate`` / ``mask_transition`` override the variant's choice; ``attention_first`` runs
    the attention updates before the multiplications (OpenFold3's ``tri_mul_first=False``).
    The arithmetic inside the ops is the Boltz-2 one either way (rounding points, layer norm)."""
    if variant not in VARIANTS:
        raise ValueError(f"Unsupported pairformer variant: {variant!r} (expected one of {sorted(VARIANTS)})")
    gate = VARIANTS[variant]["pair_gate"] if pair_gate is None else bool(pair_gate)
    mask_trans = VARIANTS[variant]["mask_transition"] if mask_transition is None else bool(mask_transition)
    dev.require_cuda()
    lib = _lib.load()
    host_in = dev.is_host_array(z)
    numpy_in = isinstance(z, np.ndarray)
    zd = dev.to_device(z, torch.bfloat16)
    squeeze = zd.dim() == 3
    if squeeze:
        zd = zd.unsqueeze(0)
    if zd.dim() != 4 or zd.shape[1] != zd.shape[2] or zd.shape[3] != C_Z:
        raise ValueError(f"expected a pair tensor [B, N, N, {C_Z}], got shape {tuple(zd.shape)}")
    b, n = zd.shape[0], zd.shape[1]
    single = s is not None
    sd = None
    if single:
        sd = dev.to_device(s, torch.float32)
        sd = sd.unsqueeze(0) if sd.dim() == 2 else sd
        if sd.dim() != 3 or tuple(sd.shape[:2]) != (b, n):
            raise ValueError(f"s shape {tuple(sd.shape)} does not match the pair tensor {tuple(zd.shape)}")
    pmd = None
    if pair_mask is not None:
        pmd = dev.to_device(pair_mask, torch.float32)
        pmd = pmd.unsqueeze(0) if pmd.dim() == 2 else pmd
        if tuple(pmd.shape) != (b, n, n):
            raise ValueError(f"pair_mask shape {tuple(pmd.shape)} does not match the pair tensor {tuple(zd.shape)}")
    md = None
    if mask is not None:
        md = dev.to_device(mask, torch.float32)
        md = md.unsqueeze(0) if md.dim() == 1 else md
        if tuple(md.shape) != (b, n):
            raise ValueError(f"mask shape {tuple(md.shape)} does not match the pair tensor {tuple(zd.shape)}")
    if gate and md is None and pmd is not None and single:
        md = torch.diagonal(pmd, dim1=-2, dim2=-1).contiguous()  # single_valid = diag(pair_valid)
    if isinstance(params, Mapping):
        stacked, blocks = 1, int(num_blocks or 1)
        packed = [_Packed(params, single)]
    else:
        stacked, blocks = 0, len(params)
        packed = [_Packed(p, single) for p in params]
        if blocks == 0:
            raise ValueError("pairformer_forward needs at least one block of parameters")
    structs = (_lib.PairformerBlockParams * len(packed))(*[p.struct for p in packed])
    c_s = sd.shape[2] if single else 0
    heads_s = packed[0].heads_s
    if single and c_s != heads_s * 24:
        raise ValueError(f"libb200tri is built for single-track heads of width 24; got c_s {c_s}, {heads_s} heads")
    hidden_z = packed[0].struct.transition_z.hidden
    hidden_s = packed[0].struct.transition_s.hidden if single else 0
    nbytes = lib.b200tri_pairformer_workspace_bytes(n, c_s, heads_s, hidden_z, hidden_s)
    ws = dev.workspace(nbytes, "pairformer")
    z_out = torch.empty_like(zd)
    s_out = torch.empty_like(sd) if single else None
    for bi in range(b):
        args = _lib.PairformerArgs(
            n=n, c_s=c_s, heads_s=heads_s, n_blocks=blocks, stacked=stacked, eps=float(eps), tri_inf=float(tri_inf),
            att_inf=float(att_inf), params=structs, z_in=zd[bi].data_ptr(), z_out=z_out[bi].data_ptr(),
            s_in=sd[bi].data_ptr() if single else None, s_out=s_out[bi].data_ptr() if single else None,
            pair_mask=pmd[bi].data_ptr() if pmd is not None else None, mask=md[bi].data_ptr() if md is not None else None,
            workspace=dev.aligned_ptr(ws), workspace_bytes=nbytes,
            pair_gate=int(gate), mask_transition=int(mask_trans), attention_first=int(bool(attention_first)))
        _lib.check(lib.b200tri_pairformer_forward(C.byref(args), C.c_void_p(dev.stream_ptr())))
    if squeeze:
        z_out = z_out[0]
        s_out = s_out[0] if single and np.ndim(s) == 2 else s_out
    if host_in:
        zh = z_out.float().cpu() if numpy_in else z_out.cpu()
        sh = s_out.cpu() if single else None
        dev.check_device_status()
        if numpy_in:
            return (sh.numpy() if single else None), zh.numpy()
        return sh, zh
    return s_out, z_out


def pairformer_layer_forward(
    params: Mapping[str, Any],
    s: Any,
    z: Any,
    mask: Any,
    pair_mask: Any,
    eps: float = 1e-5,
    chunk_size: int = 128,
    triangle_attention_chunk: int | None = None,
    triangle_attention_q_chunk: int | None = None,
    transition_hidden_chunk: int | None = None,
    matmul_precision: str = "highest",
    attention_backend: str = "b200",
    triangle_backend: str = "b200",
    glu_backend: str = "b200",
):
    """One Boltz PairformerLayer in eval mode (no dropout): returns ``(s, z)``. The chunking
    and precision knobs of the reference signature are accepted and ignored (a fused backend
    has nothing to chunk)."""
    for name, value in (("attention_backend", attention_backend), ("triangle_backend", triangle_backend),
                        ("glu_backend", glu_backend)):
        if value != "b200":
            raise ValueError(f"Unsupported {name}: {value!r}")
    return pairformer_forward([params], s, z, mask, pair_mask, eps)
