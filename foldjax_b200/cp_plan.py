"""Tile-exchange plans for the 2-D context-parallel triangle ops (pure Python).

The reference shards the pair tensor over a *square* device grid and moves tiles
with Cannon skews and ring hops (src/foldjax/models/_cp.py:413-461,
src/foldjax/models/boltz2/models/triangle/triangle.py:132-212,
src/foldjax/models/_cp_attention.py:34-89). One 8-GPU box wants 1x2, 2x2 and
2x4 grids, two of which are not square, and NVSwitch gives every pair of GPUs the
same bandwidth, so here every tile is fetched straight from its owner instead of
being passed around a ring: the plan below lists, for one rank, which peer tile
(or row block of a peer tile) lands in which slot of its panels.

Grid: R x C with C = m * R (m = 1 or 2 on one box); rank = r * C + c; device
(r, c) owns z[I_r, J_c] with |I_r| = N / R = m * |J_c|. Row block s of I_r is the
index set J_{r*m + s}.

A message is ``Msg(src, dst, what, block, slot)``: ``what`` names the sender's
local array, ``block`` the row block of it that is sent (None = the whole
tile), ``slot`` the position in the receiver's panel. A message with src == dst
is a local copy. Nothing in this module touches a GPU; the executor is in
``foldjax_b200.cp`` and a NumPy simulation of it in ``oracle/cp_oracle.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator


@dataclass(frozen=True)
class Grid:
    rows: int
    cols: int

    def __post_init__(self):
        if self.rows < 1 or self.cols < 1 or self.cols % self.rows:
            raise ValueError(f"unsupported context-parallel grid {self.rows}x{self.cols}: columns must be a multiple of rows")

    @property
    def size(self) -> int:
        return self.rows * self.cols

    @property
    def m(self) -> int:
        """Column blocks per row block (|I_r| / |J_c|)."""
        return self.cols // self.rows

    def coords(self, rank: int) -> tuple[int, int]:
        return divmod(rank, self.cols)

    def rank(self, r: int, c: int) -> int:
        return r * self.cols + c

    def ranks(self) -> Iterator[int]:
        return iter(range(self.size))

    def tile_shape(self, n: int) -> tuple[int, int]:
        if n % self.cols:
            raise ValueError(f"token count {n} is not divisible by the {self.cols} grid columns; pad it first")
        return n // self.rows, n // self.cols


def padded_tokens(n: int, grid: Grid) -> int:
    """Smallest token count >= n that the grid tiles evenly (a multiple of the
    column count, which the row count divides). The reference pads the same way:
    zero rows/columns in the pair tensor and dropped keys in the mask
    (src/foldjax/models/boltz2/models/triangle/triangle.py:165-172,
    src/foldjax/models/_cp_attention.py:265-279)."""
    return (n + grid.cols - 1) // grid.cols * grid.cols


def grid_for(cp_devices: int, layout: str | None = None) -> Grid:
    """cp_devices -> grid, mirroring the reference's option surface
    (``cp_devices`` / ``cp_layout``, src/foldjax/models/_cp.py:162-187) and
    extending it to the non-square grids of one 8-GPU box. ``layout`` may be an
    explicit "RxC"."""
    if layout and "x" in layout:
        r, c = layout.lower().split("x")
        grid = Grid(int(r), int(c))
        if grid.size != cp_devices:
            raise ValueError(f"cp_layout {layout!r} does not use {cp_devices} devices")
        return grid
    table = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4), 9: (3, 3), 16: (4, 4)}
    if cp_devices not in table:
        raise ValueError(f"no context-parallel grid for {cp_devices} devices (supported: {sorted(table)})")
    return Grid(*table[cp_devices])


@dataclass(frozen=True)
class Msg:
    src: int
    dst: int
    what: str
    block: int | None
    slot: tuple[int, ...]


# ------------------------------------------------------------------ tri-mult
def trimul_outgoing_msgs(grid: Grid) -> list[Msg]:
    """out[I_r, J_c] = sum_{c'} a[I_r, K_c'] . b[J_c, K_c']^T.

    Rank (r, c) projects a_loc[I_r, K_c] (one tile) and b_loc[I_r, K_c] (stored as m
    row blocks). It needs, for every k tile c': a_loc of (r, c') -> slot ("a", c')
    and row block c % m of b_loc of (c // m, c') -> slot ("b", c')."""
    msgs = []
    for dst in grid.ranks():
        r, c = grid.coords(dst)
        for cp in range(grid.cols):
            msgs.append(Msg(grid.rank(r, cp), dst, "a", None, (cp,)))
            msgs.append(Msg(grid.rank(c // grid.m, cp), dst, "b", c % grid.m, (cp,)))
    return msgs


def trimul_incoming_msgs(grid: Grid) -> list[Msg]:
    """out[I_r, J_c] = sum_{r''} a[K_r'', I_r]^T . b[K_r'', J_c].

    Rank (r, c) projects, through swapped strides, a'_loc[J_c, K_r] and b'_loc[J_c, K_r]
    (rows = the tile's columns). Output row block s (rows J_{r*m+s}) needs, for every
    k tile r'': a'_loc of (r'', r*m+s) -> slot ("a", s, r''); every output needs
    b'_loc of (r'', c) -> slot ("b", r'')."""
    msgs = []
    for dst in grid.ranks():
        r, c = grid.coords(dst)
        for rp in range(grid.rows):
            for s in range(grid.m):
                msgs.append(Msg(grid.rank(rp, r * grid.m + s), dst, "a", None, (s, rp)))
            msgs.append(Msg(grid.rank(rp, c), dst, "b", None, (rp,)))
    return msgs


# ----------------------------------------------------------------- tri-attn
def triatt_starting_msgs(grid: Grid) -> list[Msg]:
    """Rows i in I_r, queries j in J_c, keys in all K_c'.

    k_loc / v_loc of (r, c') -> slot ("kv", c'); the bias of (queries J_c, keys K_c')
    is row block c % m of bias_loc of (c // m, c') -> slot ("bias", c')."""
    msgs = []
    for dst in grid.ranks():
        r, c = grid.coords(dst)
        for cp in range(grid.cols):
            msgs.append(Msg(grid.rank(r, cp), dst, "kv", None, (cp,)))
            msgs.append(Msg(grid.rank(c // grid.m, cp), dst, "bias", c % grid.m, (cp,)))
    return msgs


def triatt_ending_msgs(grid: Grid) -> list[Msg]:
    """Transposed frame: rows i' in J_c, queries j' in I_r, keys in all I_r''.

    k'_loc / v'_loc of (r'', c) -> slot ("kv", r''); the bias of (queries J_{r*m+s},
    keys I_r'') is the whole bias'_loc of (r'', r*m+s) -> slot ("bias", r'', s)."""
    msgs = []
    for dst in grid.ranks():
        r, c = grid.coords(dst)
        for rp in range(grid.rows):
            msgs.append(Msg(grid.rank(rp, c), dst, "kv", None, (rp,)))
            for s in range(grid.m):
                msgs.append(Msg(grid.rank(rp, r * grid.m + s), dst, "bias", None, (rp, s)))
    return msgs


def key_order(grid: Grid, rank: int, starting: bool) -> list[int]:
    """Order in which a rank walks the key tiles: its own tile first, then the
    peers' in rotated order, so that at every step each sender serves a different
    receiver (the ring schedule of the reference, realised as direct fetches)."""
    r, c = grid.coords(rank)
    n, own = (grid.cols, c) if starting else (grid.rows, r)
    return [(own + s) % n for s in range(n)]
