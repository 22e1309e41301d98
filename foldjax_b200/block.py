"""The pair track of one Pairformer block: the four triangle updates and the pair
transition in the reference's order, each with its residual add fused into the
kernel.

Mirrors the pair-stack part of ``pairformer_layer_forward``
(src/foldjax/models/boltz2/models/trunk_blocks/pairformer.py:126-180):

    z = z + tri_mul_out(z);  z = z + tri_mul_in(z)
    z = z + tri_att_start(z);  z = z + tri_att_end(z)
    z = z + transition_z(z)

``params`` uses the reference's names for these sub-modules: ``tri_mul_out``,
``tri_mul_in``, ``tri_att_start``, ``tri_att_end`` and (optional) ``transition_z``;
without the last key only the four triangle updates run.
"""

from __future__ import annotations

from typing import Any, Mapping

import numpy as np
import torch

from . import _device as dev
from .transition import transition_forward
from .triangle import triangle_multiplication_forward
from .triangle_attention import triangle_attention_forward

OPS = ("tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end")


def block_flops(n: int) -> float:
    """Algorithmic flops of the four triangle ops of one block (c_z = c = 128, 4 heads x 32)."""
    return 2.0 * (256.0 * n**3 + 196608.0 * n**2) + 2.0 * (512.0 * n**3 + 164864.0 * n**2)


def transition_flops(n: int, c_z: int = 128, hidden: int = 512) -> float:
    """Algorithmic flops of the pair transition: three c_z x hidden products per pair."""
    return 2.0 * n * n * 3 * c_z * hidden


def triangle_block_forward(params: Mapping[str, Any], z: Any, mask: Any | None, *, out: Any | None = None):
    """Apply the four triangle updates (and the pair transition, if ``params`` has
    ``transition_z``) of one block to the pair tensor.

    Device tensors: ``z`` is updated out of place and the new pair tensor is
    returned (``out`` may alias nothing). Host tensors (NumPy arrays or CPU torch
    tensors, ideally pinned): ``z`` and ``mask`` are copied to the GPU, the block
    runs, and the result is copied back into ``out`` (allocated if None) - the
    end-to-end path.
    """
    dev.require_cuda()
    host_in = dev.is_host_array(z)
    zd = dev.to_device(z, torch.bfloat16)
    md = None if mask is None else dev.to_device(mask, torch.float32)
    # Two work buffers, used alternately; the caller's tensor is never written.
    work = (torch.empty_like(zd), torch.empty_like(zd))
    cur = zd
    for step, name in enumerate(OPS):
        nxt = work[step & 1]
        if name.startswith("tri_mul"):
            direction = "outgoing" if name.endswith("out") else "incoming"
            triangle_multiplication_forward(params[name], cur, md, direction, residual=cur, out=nxt)
        else:
            triangle_attention_forward(params[name], cur, md, starting=name.endswith("start"), residual=cur, out=nxt)
        cur = nxt
    if "transition_z" in params:
        transition_forward(params["transition_z"], cur, residual=cur, out=cur)  # row-local: safe in place
    if not host_in:
        return cur
    if out is None:
        out = torch.empty(cur.shape, dtype=torch.bfloat16, pin_memory=True)
    if isinstance(out, np.ndarray):
        out[...] = cur.float().cpu().numpy()
    else:
        out.copy_(cur, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    dev.check_device_status()  # raises if a kernel of the block gave up on a bounded wait
    return out
