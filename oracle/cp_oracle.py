"""NumPy simulation of the 2-D context-parallel schedules (TEST INFRASTRUCTURE ONLY).

Every "rank" of an R x C grid is simulated in one process: it owns the tiles a
real device would own, receives exactly the messages ``foldjax_b200.cp_plan``
lists for it, and computes its output tile from its panels. The assembled result
must equal the dense operator. This is the host-side proof of the exchange
logic that the reference obtains with forced CPU devices
(tests/models/boltz2/test_context_parallel.py, tests/models/test_cp_ring_attention.py);
3x3 and 2x6 grids are included because a 2x2 grid cannot falsify a swapped index.

Merging of attention partials follows online_softmax_update,
src/foldjax/models/_cp_attention.py:172-194.
"""

from __future__ import annotations

import numpy as np

from foldjax_b200.cp_plan import (
    Grid,
    key_order,
    triatt_ending_msgs,
    triatt_starting_msgs,
    trimul_incoming_msgs,
    trimul_outgoing_msgs,
)


def _rows(grid: Grid, n: int, r: int) -> slice:
    n_r = n // grid.rows
    return slice(r * n_r, (r + 1) * n_r)


def _cols(grid: Grid, n: int, c: int) -> slice:
    n_c = n // grid.cols
    return slice(c * n_c, (c + 1) * n_c)


def _block(arr: np.ndarray, block: int | None, n_c: int, axis: int = 0) -> np.ndarray:
    if block is None:
        return arr
    idx = [slice(None)] * arr.ndim
    idx[axis] = slice(block * n_c, (block + 1) * n_c)
    return arr[tuple(idx)]


def simulate_trimul(grid: Grid, a: np.ndarray, b: np.ndarray, direction: str) -> np.ndarray:
    """a, b: [N, N, D] projections (masked). Returns the contraction [N, N, D]
    assembled from the ranks' output tiles."""
    n = a.shape[0]
    n_r, n_c = grid.tile_shape(n)
    out = np.zeros_like(a, dtype=np.float64)
    # what every rank holds after its local projection
    local = {}
    for rank in grid.ranks():
        r, c = grid.coords(rank)
        ta, tb = a[_rows(grid, n, r), _cols(grid, n, c)], b[_rows(grid, n, r), _cols(grid, n, c)]
        if direction == "outgoing":
            local[rank] = {"a": ta, "b": tb}  # [i in I_r, k in K_c]
        else:
            local[rank] = {"a": np.swapaxes(ta, 0, 1), "b": np.swapaxes(tb, 0, 1)}  # [i in J_c, k in K_r]
    msgs = trimul_outgoing_msgs(grid) if direction == "outgoing" else trimul_incoming_msgs(grid)
    panels = {rank: {} for rank in grid.ranks()}
    for msg in msgs:
        panels[msg.dst][(msg.what,) + msg.slot] = _block(local[msg.src][msg.what], msg.block, n_c)
    for rank in grid.ranks():
        r, c = grid.coords(rank)
        p = panels[rank]
        tile = np.zeros((n_r, n_c, a.shape[2]))
        if direction == "outgoing":
            for cp in range(grid.cols):
                tile += np.einsum("ikd,jkd->ijd", p[("a", cp)], p[("b", cp)])
        else:
            for s in range(grid.m):
                for rp in range(grid.rows):
                    tile[s * n_c:(s + 1) * n_c] += np.einsum("ikd,jkd->ijd", p[("a", s, rp)], p[("b", rp)])
        out[_rows(grid, n, r), _cols(grid, n, c)] = tile
    return out


def _partial(q, k, v, bias, mb):
    """One key tile: q [I,J,H,D], k/v [I,K,H,D], bias [H,J,K], mb [I,K] ->
    unnormalised O [I,J,H,D], row max m and row sum l [I,H,J]."""
    s = np.einsum("ijhd,ikhd->ihjk", q, k) + mb[:, None, None, :] + bias[None]
    m = s.max(-1)
    p = np.exp(s - np.where(np.isfinite(m), m, 0.0)[..., None])
    return np.einsum("ihjk,ikhd->ijhd", p, v), m, p.sum(-1)


def merge(acc, part):
    """Online-softmax merge of (O, m, l) partials."""
    if acc is None:
        return part
    o1, m1, l1 = acc
    o2, m2, l2 = part
    m = np.maximum(m1, m2)
    safe = np.where(np.isfinite(m), m, 0.0)
    s1, s2 = np.exp(m1 - safe), np.exp(m2 - safe)
    o = o1 * np.swapaxes(s1, 1, 2)[..., None] + o2 * np.swapaxes(s2, 1, 2)[..., None]
    return o, m, l1 * s1 + l2 * s2


def simulate_triatt(grid: Grid, q, k, v, bias, mask_bias, starting: bool) -> np.ndarray:
    """Attention-frame operands of the whole problem: q, k, v [N(i), N(j), H, D],
    bias [H, N(j), N(k)], mask_bias [N(i), N(k)]. For the ending node the caller
    passes the operands of the transposed pair tensor; device (r, c) then owns rows
    J_c and queries/keys I_r. Returns o [N, N, H, D] in the attention frame."""
    n = q.shape[0]
    n_r, n_c = grid.tile_shape(n)
    out = np.zeros(q.shape, dtype=np.float64)
    own = {}
    for rank in grid.ranks():
        r, c = grid.coords(rank)
        rows, inner = (_rows(grid, n, r), _cols(grid, n, c)) if starting else (_cols(grid, n, c), _rows(grid, n, r))
        own[rank] = (rows, inner)
    local = {}
    for rank in grid.ranks():
        rows, inner = own[rank]
        # bias of the local tile: queries = the tile's outer index, keys = its inner index
        local[rank] = {"kv": (k[rows, inner], v[rows, inner]), "bias": bias[:, rows, inner], "q": q[rows, inner]}
    msgs = triatt_starting_msgs(grid) if starting else triatt_ending_msgs(grid)
    panels = {rank: {} for rank in grid.ranks()}
    for msg in msgs:
        src = local[msg.src][msg.what]
        if msg.what == "bias":
            src = _block(src, msg.block, n_c, axis=1)
        panels[msg.dst][(msg.what,) + msg.slot] = src
    for rank in grid.ranks():
        r, c = grid.coords(rank)
        rows, inner = own[rank]
        p = panels[rank]
        acc = None
        for t in key_order(grid, rank, starting):
            kt, vt = p[("kv", t)]
            if starting:
                keys = _cols(grid, n, t)
                b = p[("bias", t)]
            else:
                keys = _rows(grid, n, t)
                b = np.concatenate([p[("bias", t, s)] for s in range(grid.m)], axis=1)
            acc = merge(acc, _partial(local[rank]["q"], kt, vt, b, mask_bias[rows, keys]))
        o, m, l = acc
        with np.errstate(invalid="ignore", divide="ignore"):
            out[rows, inner] = o / np.swapaxes(l, 1, 2)[..., None]
    return out
