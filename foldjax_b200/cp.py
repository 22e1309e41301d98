"""2-D context-parallel triangle ops - host side.

The data plane lives in libb200tri: ``b200tri_comm_*`` (a communicator over NCCL) and
``b200tri_trimul_cp`` / ``b200tri_triatt_cp`` (the two triangle ops on one rank's tile;
tiles cross NVLink on the communicator's own stream, event-fenced and enqueue-only: written
by the copy engines into the peers' CUDA-IPC-mapped workspaces with NCCL carrying 4-byte
tokens, or as grouped ncclSend/ncclRecv - see ``TRANSPORT`` below). This module is the thin Python caller: it keeps the
reference's option surface - ``context_parallel(cp_devices, layout=)``
(src/foldjax/models/_cp.py:259) and the ``cp_devices`` / ``cp_layout`` knobs - creates
the communicator (the 128-byte NCCL id travels over ``torch.distributed``, which is used
for nothing else here), runs the mesh self-test before the first op (the counterpart of
``verify_mesh_exchange``, _cp.py:199-232) and owns the workspaces.

The grid is R x C with C a multiple of R, so the 1x2 and 2x4 grids of one 8-GPU box work
next to the square grids the reference is limited to (_cp.py:182-187). Each rank holds
the tile z[I_r, J_c] of the pair tensor (bf16, contiguous ``[n_r, n_c, 128]``) and the
whole ``[N, N]`` mask (1/256 of the pair tensor; replicating it removes one exchange per
op). ``cp_layout="1d"`` maps to the 1 x P grid: rows whole, columns sharded, the
row-sharded layout of the reference (triangle_attention.py:165-280) up to a transpose.
"""

from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import numpy as np
import torch
import torch.distributed as dist

from . import _device as dev
from . import _lib
from .cp_plan import Grid, grid_for, padded_tokens
from .triangle import _leaf

#: Bytes every rank contributes to the mesh self-test. The reference moves 4 MiB in total
#: (_cp.py:190-196): a token amount proves nothing about an interconnect that drops large
#: transfers.
EXCHANGE_PROBE_BYTES = 4 << 20


#: How tiles travel between GPUs. "push" (default) / "pull": the communicator owns the exchange
#: workspace, the peers' workspaces are mapped through CUDA IPC and the copy engines move the
#: tiles (every sender writes into the receivers' workspaces / every receiver reads out of the
#: owners'; NCCL only carries 4-byte tokens). "nccl": tiles are sent and received by NCCL into a
#: workspace this module allocates.
TRANSPORT = os.environ.get("B200TRI_CP_TRANSPORT", "push").lower()
#: streams the copies of one exchange are spread over (1..4)
COPY_STREAMS = int(os.environ.get("B200TRI_CP_COPY_STREAMS", "1"))
#: SMs the attention launch that runs while key tiles travel leaves to the token kernels
SM_RESERVE = int(os.environ.get("B200TRI_CP_SM_RESERVE", "4"))


@dataclass
class CPContext:
    grid: Grid
    rank: int
    group: Any = None
    comm: int | None = None  # b200tri_comm* (None on a host-only context, e.g. gloo ranks in tests)
    _keep: list = field(default_factory=list)

    @property
    def coords(self) -> tuple[int, int]:
        return self.grid.coords(self.rank)

    def close(self) -> None:
        if self.comm is not None:
            _lib.load().b200tri_comm_destroy(C.c_void_p(self.comm))
            self.comm = None


def exchange_failure(gathered: np.ndarray, expected: np.ndarray, *, devices: int) -> str | None:
    """Describe how a gathered probe differs from what was sent, or None. The judgement is
    separate from the exchange so that it can be tested without a broken interconnect
    (exchange_failure, src/foldjax/models/_cp.py:235-256; same wording)."""
    delta = np.abs(np.asarray(gathered, np.float64) - np.asarray(expected, np.float64)).mean(axis=-1)
    wrong = int((delta > 1e-6).sum())
    if not wrong:
        return None
    first = int(np.argmax(delta > 1e-6))
    return (f"the {devices}-device context-parallel mesh does not exchange data: {wrong} of {len(delta)} rows "
            f"came back wrong, from row {first}, over {EXCHANGE_PROBE_BYTES >> 20} MiB. Every result from this "
            "mesh would be silently incomplete.")


def verify_mesh_exchange(world: int, rank: int, gather: Callable[[np.ndarray], np.ndarray]) -> None:
    """Fail now if the mesh does not actually move data between its ranks. Every rank
    stamps 64 rows with their global row index, ``gather(shard)`` returns all ranks' rows
    as they arrived here, and the host compares them with what must have been sent."""
    rows = 64
    cols = max(EXCHANGE_PROBE_BYTES // (world * rows * 4), 1)
    expected = np.arange(world * rows, dtype=np.float32)[:, None] * np.ones((1, cols), np.float32)
    shard = np.ascontiguousarray(expected[rank * rows:(rank + 1) * rows])
    failure = exchange_failure(gather(shard), expected, devices=world)
    if failure is not None:
        raise RuntimeError(f"{failure} Rank {rank} of {world}.")


def _probe_over_comm(ctx: CPContext) -> Callable[[np.ndarray], np.ndarray]:
    def gather(shard: np.ndarray) -> np.ndarray:
        lib = _lib.load()
        sd = torch.from_numpy(shard).cuda()
        out = torch.full((ctx.grid.size,) + tuple(shard.shape), -1.0, dtype=torch.float32, device=sd.device)
        _lib.check(lib.b200tri_comm_probe(C.c_void_p(ctx.comm), C.c_void_p(sd.data_ptr()), C.c_void_p(out.data_ptr()),
                                          C.c_size_t(shard.nbytes), C.c_void_p(dev.stream_ptr())))
        return out.cpu().numpy().reshape(-1, shard.shape[-1])

    return gather


def context_parallel(cp_devices: int | None = None, layout: str | None = None, group=None,
                     verify: bool = True) -> CPContext:
    """Grid over the ranks of ``group`` (default: the world) and, on CUDA ranks, the
    communicator the context-parallel ops run on. ``layout``: "auto" / "2d" pick the grid
    for the device count (2 -> 1x2, 4 -> 2x2, 8 -> 2x4), "1d" the 1 x P grid, "RxC" an
    explicit one. ``verify`` runs the mesh self-test before the context is returned."""
    if not dist.is_initialized():
        raise RuntimeError("context_parallel needs an initialised torch.distributed process group")
    world = dist.get_world_size(group)
    n = cp_devices or world
    if n != world:
        raise ValueError(f"cp_devices={n} but the process group has {world} ranks")
    if layout in ("auto", "2d"):
        layout = None
    if layout == "1d":
        layout = f"1x{n}"
    grid, rank = grid_for(n, layout), dist.get_rank(group)
    ctx = CPContext(grid, rank, group)
    if not torch.cuda.is_available():
        return ctx  # host-only context: the plan and the option surface, no device ops
    lib = _lib.load()
    ident = torch.zeros(_lib.COMM_ID_BYTES, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_uint8 * _lib.COMM_ID_BYTES)()
        _lib.check(lib.b200tri_comm_unique_id(buf))
        ident = torch.frombuffer(bytearray(buf), dtype=torch.uint8).clone()
    on_device = dist.get_backend(group) == "nccl"
    ident = ident.cuda() if on_device else ident
    dist.broadcast(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    raw = bytes(ident.cpu().numpy().tobytes())
    handle = C.c_void_p()
    _lib.check(lib.b200tri_comm_init(C.byref(handle), raw, world, rank, grid.rows, grid.cols))
    ctx.comm = handle.value
    _lib.check(lib.b200tri_comm_configure(handle, int(TRANSPORT != "pull"), COPY_STREAMS, SM_RESERVE))
    if verify and world > 1:
        verify_mesh_exchange(world, rank, _probe_over_comm(ctx))
    return ctx


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


def _ws(tag: str, nbytes: int) -> tuple[int, int]:
    raw = dev.workspace(nbytes + 1024, tag)
    return dev.aligned_ptr(raw), nbytes




def _exchange_workspace(ctx: CPContext, n: int) -> tuple[int | None, int]:
    """(workspace pointer or None, bytes) for the two context-parallel ops at ``n`` tokens. None
    selects the communicator's own workspace, sized here for both ops (collective: every rank
    reaches this call with the same ``n`` at the same point of its op sequence)."""
    lib = _lib.load()
    need = max(lib.b200tri_trimul_cp_workspace_bytes(C.c_void_p(ctx.comm), n),
               lib.b200tri_triatt_cp_workspace_bytes(C.c_void_p(ctx.comm), n))
    if TRANSPORT == "nccl":
        return _ws("cp_exchange", need)
    if TRANSPORT not in ("push", "pull"):
        raise ValueError(f"B200TRI_CP_TRANSPORT must be 'push', 'pull' or 'nccl', got {TRANSPORT!r}")
    out = C.c_void_p()
    _lib.check(lib.b200tri_comm_workspace(C.c_void_p(ctx.comm), need, C.byref(out)))
    return None, 0


def _tile_checks(ctx: CPContext, x: torch.Tensor, mask, residual, out) -> tuple[int, torch.Tensor]:
    if ctx.comm is None:
        raise RuntimeError("this context has no communicator (created without a CUDA device)")
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
            and x.dim() == 3 and x.shape[2] == 128):
        raise ValueError("x must be this rank's tile: a contiguous CUDA bf16 tensor [n_r, n_c, 128]")
    n = x.shape[0] * ctx.grid.rows
    if x.shape[1] * ctx.grid.cols != n:
        raise ValueError(f"tile shape {tuple(x.shape[:2])} does not match the {ctx.grid.rows}x{ctx.grid.cols} grid")
    if mask is not None and not (isinstance(mask, torch.Tensor) and mask.is_cuda and mask.dtype == torch.float32
                                 and tuple(mask.shape) == (n, n) and mask.is_contiguous()):
        raise ValueError(f"mask must be the whole [{n}, {n}] float32 mask on the device (or None)")
    if out is None:
        out = torch.empty_like(x)
    else:
        dev.check_out(out, x)
    if residual is not None:
        dev.check_out(residual, x, "residual")
    return n, out


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
    n, out = _tile_checks(ctx, x, mask, residual, out)
    lv = {k: _leaf(params, *k.split(".")) for k in (
        "norm_in.scale", "norm_in.bias", "p_in.kernel", "g_in.kernel", "norm_out.scale", "norm_out.bias",
        "p_out.kernel", "g_out.kernel")}
    wp, wb = _exchange_workspace(ctx, n)
    args = _lib.TrimulCpArgs(
        n=n, incoming=int(direction == "incoming"), eps=float(eps), x=x.data_ptr(),
        mask=None if mask is None else mask.data_ptr(),
        norm_in_scale=lv["norm_in.scale"].data_ptr(), norm_in_bias=lv["norm_in.bias"].data_ptr(),
        p_in=lv["p_in.kernel"].data_ptr(), g_in=lv["g_in.kernel"].data_ptr(),
        norm_out_scale=lv["norm_out.scale"].data_ptr(), norm_out_bias=lv["norm_out.bias"].data_ptr(),
        p_out=lv["p_out.kernel"].data_ptr(), g_out=lv["g_out.kernel"].data_ptr(),
        residual=None if residual is None else residual.data_ptr(), out=out.data_ptr(),
        workspace=wp, workspace_bytes=wb)
    _lib.check(lib.b200tri_trimul_cp(C.c_void_p(ctx.comm), C.byref(args), C.c_void_p(dev.stream_ptr())))
    return out


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
    (_cp_attention.py:197-403, boltz2 triangle_attention_cp.py:40-156). Rows without a
    valid key come out as the uniform average over their keys (the dense path's
    convention); the reference's ring returns zeros there (_cp_attention.py:380-385)."""
    lib = _lib.load()
    n, out = _tile_checks(ctx, x, mask, residual, out)
    lv = {k: _leaf(params, *k.split(".")) for k in (
        "layer_norm.scale", "layer_norm.bias", "linear.kernel", "mha.linear_q.kernel", "mha.linear_k.kernel",
        "mha.linear_v.kernel", "mha.linear_g.kernel", "mha.linear_o.kernel")}
    wp, wb = _exchange_workspace(ctx, n)
    args = _lib.TriattCpArgs(
        n=n, starting=int(bool(starting)), heads=4, head_dim=32, inf=float(inf), eps=float(eps), x=x.data_ptr(),
        mask=None if mask is None else mask.data_ptr(),
        norm_scale=lv["layer_norm.scale"].data_ptr(), norm_bias=lv["layer_norm.bias"].data_ptr(),
        w_bias=lv["linear.kernel"].data_ptr(), w_q=lv["mha.linear_q.kernel"].data_ptr(),
        w_k=lv["mha.linear_k.kernel"].data_ptr(), w_v=lv["mha.linear_v.kernel"].data_ptr(),
        w_g=lv["mha.linear_g.kernel"].data_ptr(), w_o=lv["mha.linear_o.kernel"].data_ptr(),
        residual=None if residual is None else residual.data_ptr(), out=out.data_ptr(),
        workspace=wp, workspace_bytes=wb)
    _lib.check(lib.b200tri_triatt_cp(C.c_void_p(ctx.comm), C.byref(args), C.c_void_p(dev.stream_ptr())))
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
