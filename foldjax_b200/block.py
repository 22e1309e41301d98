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


def stream_host_blocks(run_block, items, outs=None):
    """Run ``run_block(z_device, mask_device) -> z_device`` over a sequence of HOST inputs
    with the transfers overlapped: while the kernels of item k run, item k+1 is copied to
    the GPU and the result of item k-1 is copied back (three streams, two device input slots,
    PCIe in both directions at once).

    ``items``: a sequence of ``(z, mask)`` CPU torch tensors, bf16 ``z`` and float32 ``mask``
    (or None), all of one shape; pinned memory lets the copies run asynchronously. ``outs``:
    optional list of pinned CPU bf16 tensors to receive the results (allocated if None).
    Returns the list of outputs after everything has finished. This is the end-to-end form
    for a stream of complexes (or of trunk recycles whose inputs live on the host); a single
    call of ``triangle_block_forward`` on host arrays cannot overlap its own two copies with
    anything, because the first op needs the whole pair tensor and the last one produces it.
    """
    items = list(items)
    if not items:
        return []
    for z, mask in items:
        if not (isinstance(z, torch.Tensor) and not z.is_cuda and z.dtype == torch.bfloat16 and z.is_contiguous()):
            raise ValueError("stream_host_blocks takes contiguous CPU bfloat16 tensors for z")
        if z.shape != items[0][0].shape:
            raise ValueError("stream_host_blocks: every item must have the same shape")
        if mask is not None and not (isinstance(mask, torch.Tensor) and not mask.is_cuda and mask.dtype == torch.float32):
            raise ValueError("stream_host_blocks takes CPU float32 tensors (or None) for mask")
    if outs is None:
        dev.require_cuda()
        outs = [torch.empty(z.shape, dtype=torch.bfloat16, pin_memory=True) for z, _ in items]
    if len(outs) != len(items):
        raise ValueError(f"stream_host_blocks: {len(items)} items but {len(outs)} output buffers")
    for o, (z, _) in zip(outs, items):
        if not (isinstance(o, torch.Tensor) and not o.is_cuda and o.dtype == torch.bfloat16 and o.is_contiguous()
                and o.shape == z.shape):
            raise ValueError("stream_host_blocks: outputs must be contiguous CPU bfloat16 tensors of the inputs' shape")
    dev.require_cuda()
    compute = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    z0, m0 = items[0]
    z_slot = [torch.empty(z0.shape, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    m_slot = [None if m0 is None else torch.empty(m0.shape, dtype=torch.float32, device="cuda") for _ in range(2)]
    loaded = [torch.cuda.Event() for _ in range(2)]     # slot filled (copy_in)
    consumed = [torch.cuda.Event() for _ in range(2)]   # slot no longer read (compute)
    start = torch.cuda.Event()
    start.record(compute)
    copy_in.wait_event(start)   # nothing of this call overtakes the caller's earlier work
    copy_out.wait_event(start)
    for k, (z, mask) in enumerate(items):
        slot = k & 1
        with torch.cuda.stream(copy_in):
            if k >= 2:
                copy_in.wait_event(consumed[slot])
            z_slot[slot].copy_(z, non_blocking=True)
            if mask is not None:
                m_slot[slot].copy_(mask, non_blocking=True)
            loaded[slot].record(copy_in)
        compute.wait_event(loaded[slot])
        # the block writes its own work buffers; the input slot is free once its last reader ran
        res = run_block(z_slot[slot], m_slot[slot])
        if res.data_ptr() == z_slot[slot].data_ptr():
            raise RuntimeError("run_block must not return its input buffer")
        done = torch.cuda.Event()
        done.record(compute)
        consumed[slot].record(compute)
        res.record_stream(copy_out)  # the allocator may not reuse it before the copy below has run
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            outs[k].copy_(res, non_blocking=True)
        del res
    finish = torch.cuda.Event()
    finish.record(copy_out)
    compute.wait_event(finish)
    copy_in.synchronize()
    copy_out.synchronize()
    compute.synchronize()
    dev.check_device_status()
    return outs


def triangle_block_forward_stream(params: Mapping[str, Any], items, outs=None):
    """``triangle_block_forward`` over a sequence of host ``(z, mask)`` pairs with the copies of
    neighbouring items overlapped with the kernels (see ``stream_host_blocks``)."""
    return stream_host_blocks(lambda zd, md: triangle_block_forward(params, zd, md), items, outs)
