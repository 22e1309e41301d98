"""2-D context-parallel triangle ops: one process per GPU, tiles exchanged over
NVLink with NCCL point-to-point calls (``torch.distributed``), the arithmetic in
libb200tri's stage kernels.

Option surface of the reference kept: ``context_parallel(cp_devices, layout=)``
(src/foldjax/models/_cp.py:259) and the ``cp_devices`` / ``cp_layout`` knobs; the
grid is R x C with C a multiple of R, so the 1x2 and 2x4 grids of one 8-GPU box
work next to the square grids the reference is limited to (_cp.py:182-187).

Each rank holds the tile z[I_r, J_c] of the pair tensor (bf16, contiguous
``[n_r, n_c, 128]``) and the whole ``[N, N]`` mask (it is 1/256 of the pair
tensor; replicating it removes one exchange per op). The schedules are the
message lists of ``cp_plan``: tiles are fetched directly from their owners
(NVSwitch gives every pair the same bandwidth) in a rotated order, posted before
the first local kernel starts, so transfers run beside the tile compute; the
attention core continues one softmax across the key tiles (running state in
fp32), which is what the reference's ring does with its two passes
(src/foldjax/models/_cp_attention.py:290-386).
"""

from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Any, Mapping

import torch
import torch.distributed as dist

from . import _device as dev
from . import _lib
from .cp_plan import (
    Grid,
    Msg,
    grid_for,
    key_order,
    padded_tokens,
    triatt_ending_msgs,
    triatt_starting_msgs,
    trimul_incoming_msgs,
    trimul_outgoing_msgs,
)
from .triangle import _leaf

# SMs left to NCCL's send/recv kernels while a tile exchange is in flight (B200TRI_COMM_SMS overrides).
# Measured on 1x2 and 2x4 grids of B200s: reserving none is 1-2 % faster than reserving 8 or 32 (the
# point-to-point transfers of one box do not need SMs of their own), so the default is 0.
COMM_SMS = int(os.environ.get("B200TRI_COMM_SMS", "0"))


@dataclass
class CPContext:
    grid: Grid
    rank: int
    group: Any = None

    @property
    def coords(self) -> tuple[int, int]:
        return self.grid.coords(self.rank)


def context_parallel(cp_devices: int | None = None, layout: str | None = None, group=None) -> CPContext:
    """Grid over the ranks of ``group`` (default: the world). ``layout`` "1d" is not
    offered: the 2-D tiling is the only sharded form of this backend."""
    if not dist.is_initialized():
        raise RuntimeError("context_parallel needs an initialised torch.distributed process group")
    world = dist.get_world_size(group)
    n = cp_devices or world
    if n != world:
        raise ValueError(f"cp_devices={n} but the process group has {world} ranks")
    if layout in ("auto", "2d"):
        layout = None
    if layout == "1d":
        raise ValueError("cp_layout='1d' is not supported by the b200 backend; use '2d' (or 'RxC')")
    return CPContext(grid_for(n, layout), dist.get_rank(group), group)


def shard_pair(ctx: CPContext, z: torch.Tensor) -> torch.Tensor:
    """This rank's tile of a full [N, N, ...] tensor (host-side helper for tests and benchmarks)."""
    n = z.shape[0]
    n_r, n_c = ctx.grid.tile_shape(n)
    r, c = ctx.coords
    return z[r * n_r:(r + 1) * n_r, c * n_c:(c + 1) * n_c].contiguous()


def pad_pair(grid: Grid, z: torch.Tensor, mask: torch.Tensor | None):
    """Pad a full ``[N, N, C]`` pair tensor and its ``[N, N]`` mask to a token count
    the grid tiles evenly: zero pairs, and mask 0 on the added rows and columns, so
    the added tokens are dropped as keys and contribute nothing to the contraction
    (the reference's padding, triangle.py:165-172, _cp_attention.py:265-279). The
    caller crops the result back to ``[:N, :N]``. With mask None an all-ones mask of
    the original size is made, because the padding must be masked."""
    n = z.shape[0]
    n_pad = padded_tokens(n, grid)
    if mask is None:
        mask = torch.ones(n, n, dtype=torch.float32, device=z.device)
    if n_pad == n:
        return z, mask
    zp = torch.zeros((n_pad, n_pad) + tuple(z.shape[2:]), dtype=z.dtype, device=z.device)
    zp[:n, :n] = z
    mp = torch.zeros(n_pad, n_pad, dtype=mask.dtype, device=mask.device)
    mp[:n, :n] = mask
    return zp, mp


# ------------------------------------------------------------------ exchange
def _post(ctx: CPContext, msgs: list[Msg], views) -> list:
    """Post the P2P operations of this rank's messages. ``views(msg, side)`` returns the
    list of contiguous tensors that make up the message on the "send" or "recv"
    side. Local messages are copied. Returns the NCCL work handles."""
    ops = []
    for msg in msgs:
        if msg.src == msg.dst == ctx.rank:
            for s, d in zip(views(msg, "send"), views(msg, "recv")):
                if s.data_ptr() != d.data_ptr():
                    d.copy_(s, non_blocking=True)
        elif msg.src == ctx.rank:
            ops += [dist.P2POp(dist.isend, t, msg.dst, ctx.group) for t in views(msg, "send")]
        elif msg.dst == ctx.rank:
            ops += [dist.P2POp(dist.irecv, t, msg.src, ctx.group) for t in views(msg, "recv")]
    return dist.batch_isend_irecv(ops) if ops else []


def _wait(works) -> None:
    for w in works:
        w.wait()


def _call(fn, args) -> None:
    _lib.check(fn(C.byref(args), C.c_void_p(dev.stream_ptr())))


def _bf16_buf(tag: str, *shape: int) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    raw = dev.workspace(2 * n + 1024, tag)
    off = dev.aligned_ptr(raw) - raw.data_ptr()
    return raw[off:off + 2 * n].view(torch.bfloat16).view(*shape)


def _buf(tag: str, dtype: torch.dtype, *shape: int) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    raw = dev.workspace(nbytes + 1024, tag)
    off = dev.aligned_ptr(raw) - raw.data_ptr()
    return raw[off:off + nbytes].view(dtype).view(*shape)


def _ws(tag: str, nbytes: int) -> tuple[int, int]:
    raw = dev.workspace(nbytes + 1024, tag)
    return dev.aligned_ptr(raw), nbytes


# ------------------------------------------------------------------ tri-mult
def triangle_multiplication_cp(
    ctx: CPContext,
    params: Mapping[str, Mapping[str, Any]],
    x: torch.Tensor,
    mask: torch.Tensor | None,
    direction: str,
    eps: float = 1e-5,
    *,
    residual: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Triangle multiplication on this rank's tile ``x [n_r, n_c, 128]`` of the pair
    tensor; ``mask`` is the whole ``[N, N]`` mask (or None). Returns the tile of the
    update (plus ``residual`` if given). Replaces the 2-D branch of
    triangle_multiplication_forward (triangle.py:104-110, _cannon_contract :132-212)."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"Unsupported triangle multiplication direction: {direction!r}")
    lib = _lib.load()
    grid, (r, c) = ctx.grid, ctx.coords
    n_r, n_c = x.shape[0], x.shape[1]
    n = n_r * grid.rows
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[2] == 128
    assert n_c * grid.cols == n, "tile shape does not match the grid"
    R, Cc, m = grid.rows, grid.cols, grid.m
    outgoing = direction == "outgoing"
    lv = {k: _leaf(params, *k.split(".")) for k in (
        "norm_in.scale", "norm_in.bias", "p_in.kernel", "g_in.kernel", "norm_out.scale", "norm_out.bias",
        "p_out.kernel", "g_out.kernel")}
    mptr = None
    if mask is not None:
        assert mask.is_cuda and mask.dtype == torch.float32 and tuple(mask.shape) == (n, n) and mask.is_contiguous()
        mptr = mask.data_ptr() + 4 * (r * n_r * n + c * n_c)
    if out is None:
        out = torch.empty_like(x)
    else:
        dev.check_out(out, x)
    if residual is not None:
        dev.check_out(residual, x, "residual")

    if outgoing:
        # local tiles as m row blocks of n_c rows: [m][128][n_c][ld], k = the tile's columns
        ld = (n_c + 63) // 64 * 64
        blk = 128 * n_c * ld
        a_all = _bf16_buf("cp_a", Cc, m, 128, n_c, ld)  # slot c' <- a_loc of (r, c')
        b_loc = _bf16_buf("cp_bl", m, 128, n_c, ld)
        b_all = _bf16_buf("cp_b", Cc, 128, n_c, ld)     # slot c' <- block c%m of b_loc of (c//m, c')
        a_loc = a_all[c]
        n_outer, n_inner, xs_o, xs_i, ms_o, ms_i = n_r, n_c, n_c * 128, 128, n, 1
        msgs = trimul_outgoing_msgs(grid)
        n_src, n_k = Cc, n_c
    else:
        # through swapped strides: rows = the tile's columns (n_c), k = the tile's rows (n_r)
        ld = (n_r + 63) // 64 * 64
        blk = 128 * n_c * ld
        a_all = _bf16_buf("cp_a", m, R, 128, n_c, ld)   # slot (s, r'') <- a'_loc of (r'', r*m+s)
        b_all = _bf16_buf("cp_b", R, 128, n_c, ld)      # slot r'' <- b'_loc of (r'', c)
        a_loc = _bf16_buf("cp_al", 128, n_c, ld)
        b_loc = b_all[r]
        n_outer, n_inner, xs_o, xs_i, ms_o, ms_i = n_c, n_r, 128, n_c * 128, 1, n
        msgs = trimul_incoming_msgs(grid)
        n_src, n_k = R, n_r

    # Inside every n_c-row block the rows are grouped again in blocks of 64
    # ([n_c/64][128][64][ld]): same bytes, so the messages do not change, but the
    # projection's channel planes of one tile stay close together in memory.
    rpb = 64 if n_c % 64 == 0 else n_c
    wp, wb = _ws("cp_proj", lib.b200tri_trimul_project_workspace_bytes())
    pa = _lib.TrimulProjectArgs(
        n_outer=n_outer, n_inner=n_inner, eps=float(eps), x=x.data_ptr(), xs_outer=xs_o, xs_inner=xs_i,
        mask=mptr, ms_outer=ms_o, ms_inner=ms_i,
        norm_in_scale=lv["norm_in.scale"].data_ptr(), norm_in_bias=lv["norm_in.bias"].data_ptr(),
        p_in=lv["p_in.kernel"].data_ptr(), g_in=lv["g_in.kernel"].data_ptr(),
        a=a_loc.data_ptr(), b=b_loc.data_ptr(), ld=ld, chan_stride=rpb * ld, block_stride=128 * rpb * ld,
        rows_per_block=rpb,
        workspace=wp, workspace_bytes=wb)
    _call(lib.b200tri_trimul_project, pa)

    def views(msg: Msg, side: str):
        if side == "send":
            src = a_loc if msg.what == "a" else b_loc
            return [src if msg.block is None else src[msg.block]]
        if outgoing:
            return [a_all[msg.slot[0]] if msg.what == "a" else b_all[msg.slot[0]]]
        return [a_all[msg.slot[0], msg.slot[1]] if msg.what == "a" else b_all[msg.slot[0]]]

    # NCCL orders the transfers after the projection (it waits on this stream), and
    # wait() orders the contraction after the transfers; the host does not block.
    _wait(_post(ctx, msgs, views))

    ldt = (n_c + 63) // 64 * 64
    t = _bf16_buf("cp_t", 128, n_r, ldt)
    # t in the same blocked form ([n_r/64][128][64][ldt]) when the rows allow it;
    # otherwise plain channel-major [128][n_r][ldt]
    t_rpb = rpb if rpb == 64 else n_r
    t_chan = t_rpb * ldt
    t_row = 128 * ldt if rpb == 64 else ldt  # elements per output row of one launch's offset
    for s in range(m):
        if outgoing:
            a_ptr, a_src = a_all.data_ptr() + 2 * s * blk, m * blk
        else:
            a_ptr, a_src = a_all[s].data_ptr(), blk
        ca = _lib.TrimulContractArgs(
            n_i=n_c, n_j=n_c, n_k=n_k, n_src=n_src,
            a=a_ptr, a_ld=ld, a_chan_stride=rpb * ld, a_src_stride=a_src,
            b=b_all.data_ptr(), b_ld=ld, b_chan_stride=rpb * ld, b_src_stride=blk,
            acc_in=None, out_f32=None, out_bf16=t.data_ptr() + 2 * s * n_c * t_row, out_ld=ldt,
            out_chan_stride=t_chan,
            a_rows_per_block=rpb, b_rows_per_block=rpb, out_rows_per_block=t_rpb,
            a_block_stride=128 * rpb * ld, b_block_stride=128 * rpb * ld, out_block_stride=128 * t_rpb * ldt)
        _call(lib.b200tri_trimul_contract, ca)
    wp, wb = _ws("cp_fin", lib.b200tri_trimul_finish_workspace_bytes())
    fa = _lib.TrimulFinishArgs(
        n_i=n_r, n_j=n_c, eps=float(eps), t=t.data_ptr(), t_ld=ldt, t_chan_stride=t_chan,
        t_rows_per_block=t_rpb, t_block_stride=128 * t_rpb * ldt,
        x=x.data_ptr(), xs_i=n_c * 128, xs_j=128,
        norm_in_scale=lv["norm_in.scale"].data_ptr(), norm_in_bias=lv["norm_in.bias"].data_ptr(),
        norm_out_scale=lv["norm_out.scale"].data_ptr(), norm_out_bias=lv["norm_out.bias"].data_ptr(),
        p_out=lv["p_out.kernel"].data_ptr(), g_out=lv["g_out.kernel"].data_ptr(),
        residual=None if residual is None else residual.data_ptr(), out=out.data_ptr(),
        os_i=n_c * 128, os_j=128, workspace=wp, workspace_bytes=wb)
    _call(lib.b200tri_trimul_finish, fa)
    return out


def dev_sms() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


# ----------------------------------------------------------------- tri-attn
def triangle_attention_cp(
    ctx: CPContext,
    params: Mapping[str, Any],
    x: torch.Tensor,
    mask: torch.Tensor | None = None,
    starting: bool = True,
    inf: float = 1e9,
    eps: float = 1e-5,
    *,
    residual: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Triangle attention on this rank's tile ``x [n_r, n_c, 128]``; ``mask`` is the whole
    ``[N, N]`` mask (or None). Starting node: this rank's rows attend over the key
    tiles of its grid row; ending node: its columns attend over the key tiles of its
    grid column. Replaces ring_triangle_attention_2d and its callers
    (_cp_attention.py:197-403, boltz2 triangle_attention_cp.py:40-156)."""
    lib = _lib.load()
    grid, (r, c) = ctx.grid, ctx.coords
    n_r, n_c = x.shape[0], x.shape[1]
    n = n_r * grid.rows
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[2] == 128
    assert n_c * grid.cols == n, "tile shape does not match the grid"
    R, Cc, m = grid.rows, grid.cols, grid.m
    lv = {k: _leaf(params, *k.split(".")) for k in (
        "layer_norm.scale", "layer_norm.bias", "linear.kernel", "mha.linear_q.kernel", "mha.linear_k.kernel",
        "mha.linear_v.kernel", "mha.linear_g.kernel", "mha.linear_o.kernel")}
    if mask is not None:
        assert mask.is_cuda and mask.dtype == torch.float32 and tuple(mask.shape) == (n, n) and mask.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    else:
        dev.check_out(out, x)
    if residual is not None:
        dev.check_out(residual, x, "residual")
    if starting:
        n_outer, n_inner, xs_o, xs_i, tiles, own = n_r, n_c, n_c * 128, 128, Cc, c
        msgs = triatt_starting_msgs(grid)
    else:
        n_outer, n_inner, xs_o, xs_i, tiles, own = n_c, n_r, 128, n_c * 128, R, r
        msgs = triatt_ending_msgs(grid)
    n_q = n_c if starting else n_r  # queries of the core calls
    ld = (n_inner + 63) // 64 * 64
    q_loc = _bf16_buf("cp_q", n_outer, n_inner, 128)
    k_all = _bf16_buf("cp_k", tiles, n_outer, n_inner, 128)
    vt_all = _buf("cp_v", torch.float16, tiles, n_outer, 128, ld)
    bias_loc = _bf16_buf("cp_biasl", 4, n_outer, ld)
    bias_all = _bf16_buf("cp_bias", tiles, 4, n_q, ld)
    o_loc = _bf16_buf("cp_o", n_outer, n_q, 128)

    wp, wb = _ws("cp_aproj", lib.b200tri_triatt_project_workspace_bytes())
    pa = _lib.TriattProjectArgs(
        n_outer=n_outer, n_inner=n_inner, heads=4, head_dim=32, eps=float(eps),
        x=x.data_ptr(), xs_outer=xs_o, xs_inner=xs_i,
        norm_scale=lv["layer_norm.scale"].data_ptr(), norm_bias=lv["layer_norm.bias"].data_ptr(),
        w_q=lv["mha.linear_q.kernel"].data_ptr(), w_k=lv["mha.linear_k.kernel"].data_ptr(),
        w_v=lv["mha.linear_v.kernel"].data_ptr(), w_bias=lv["linear.kernel"].data_ptr(),
        q=q_loc.data_ptr(), k=k_all[own].data_ptr(), vt=vt_all[own].data_ptr(), bias=bias_loc.data_ptr(),
        ld=ld, bias_head_stride=n_outer * ld, workspace=wp, workspace_bytes=wb)
    _call(lib.b200tri_triatt_project, pa)

    def views(msg: Msg, side: str):
        if msg.what == "kv":
            if side == "send":
                return [k_all[own], vt_all[own]]
            return [k_all[msg.slot[0]], vt_all[msg.slot[0]]]
        if starting:  # row block of the sender's bias -> the whole bias of one key tile
            if side == "send":
                return [bias_loc[h, msg.block * n_c:(msg.block + 1) * n_c] for h in range(4)]
            return [bias_all[msg.slot[0], h] for h in range(4)]
        if side == "send":  # the sender's whole bias -> one query block of one key tile
            return [bias_loc[h] for h in range(4)]
        rp, s = msg.slot
        return [bias_all[rp, h, s * n_c:(s + 1) * n_c] for h in range(4)]

    # Two batches: the bias chunks (small; even the own key tile's bias may live on
    # another rank) are needed before the first core call, the K/V tiles of the
    # peers only before the second one.
    _wait(_post(ctx, [msg for msg in msgs if msg.what == "bias"], views))
    works = _post(ctx, [msg for msg in msgs if msg.what == "kv"], views)
    if grid.size > 1:
        lib.b200tri_set_sm_limit(dev_sms() - COMM_SMS)

    acc_o = _buf("cp_acc", torch.float32, n_outer, n_q, 128)
    rmax = _buf("cp_rmax", torch.float32, n_outer, 4, n_q)
    rsum = _buf("cp_rsum", torch.float32, n_outer, 4, n_q)
    order = key_order(grid, ctx.rank, starting)
    nb = lib.b200tri_triatt_core_workspace_bytes(n_outer, n_inner)
    wp, wb = _ws("cp_core", nb)
    for idx, t in enumerate(order):
        if idx == 1:
            _wait(works)  # every peer tile has landed; the own tile was computed meanwhile
            lib.b200tri_set_sm_limit(0)
        mptr, ms_i, ms_k = None, 0, 0
        if mask is not None:
            if starting:  # rows I_r, keys K_t
                mptr, ms_i, ms_k = mask.data_ptr() + 4 * (r * n_r * n + t * n_c), n, 1
            else:  # rows J_c, keys I_t of the transposed mask
                mptr, ms_i, ms_k = mask.data_ptr() + 4 * (t * n_r * n + c * n_c), 1, n
        ca = _lib.TriattCoreArgs(
            n_i=n_outer, n_j=n_q, n_k=n_inner, heads=4, head_dim=32,
            q=q_loc.data_ptr(), k=k_all[t].data_ptr(), vt=vt_all[t].data_ptr(), v_ld=ld,
            bias=bias_all[t].data_ptr(), bias_ld=ld, bias_head_stride=n_q * ld,
            mask=mptr, ms_i=ms_i, ms_k=ms_k, inf=float(inf), o=o_loc.data_ptr(),
            row_max=rmax.data_ptr(), row_sum=rsum.data_ptr(), unnormalized=int(idx < len(order) - 1),
            workspace=wp, workspace_bytes=wb, acc_o=acc_o.data_ptr(), resume=int(idx > 0))
        _call(lib.b200tri_triatt_core, ca)
    if len(order) == 1:
        _wait(works)
    lib.b200tri_set_sm_limit(0)

    wp, wb = _ws("cp_afin", lib.b200tri_triatt_finish_workspace_bytes())
    fa = _lib.TriattFinishArgs(
        n_outer=n_outer, n_inner=n_inner, eps=float(eps), o=o_loc.data_ptr(), x=x.data_ptr(),
        xs_outer=xs_o, xs_inner=xs_i,
        norm_scale=lv["layer_norm.scale"].data_ptr(), norm_bias=lv["layer_norm.bias"].data_ptr(),
        w_g=lv["mha.linear_g.kernel"].data_ptr(), w_o=lv["mha.linear_o.kernel"].data_ptr(),
        residual=None if residual is None else residual.data_ptr(), out=out.data_ptr(),
        os_outer=xs_o, os_inner=xs_i, workspace=wp, workspace_bytes=wb)
    _call(lib.b200tri_triatt_finish, fa)
    return out


def triangle_block_cp(ctx: CPContext, params: Mapping[str, Any], z: torch.Tensor, mask: torch.Tensor | None):
    """The pair track of one Pairformer block on this rank's tile, residual adds fused
    (pairformer.py:126-180 under the 2-D layout): the four triangle updates, then the
    pair transition if ``params`` has ``transition_z`` (row-local, so it needs no
    exchange)."""
    work = (torch.empty_like(z), torch.empty_like(z))
    cur = z
    for step, name in enumerate(("tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end")):
        nxt = work[step & 1]
        if name.startswith("tri_mul"):
            triangle_multiplication_cp(ctx, params[name], cur, mask, "outgoing" if name.endswith("out") else "incoming",
                                       residual=cur, out=nxt)
        else:
            triangle_attention_cp(ctx, params[name], cur, mask, starting=name.endswith("start"), residual=cur, out=nxt)
        cur = nxt
    if "transition_z" in params:
        from .transition import transition_forward

        transition_forward(params["transition_z"], cur, residual=cur, out=cur)
    return cur
