"""The context-parallel ops, dry-run on the CPU: every copy and every launch the C layer would
make on every rank of a grid, checked against the layout the kernels rely on.

``b200tri_cp_dry_run`` runs ``b200tri_trimul_cp`` / ``b200tri_triatt_cp`` for one rank with all
CUDA and NCCL calls skipped and returns the copies it would issue (offsets into the ranks'
exchange workspaces) and the launches it would make. Collected over all ranks this is the
whole exchange, so the following can be held without a GPU, on grids a single box cannot even
form (3 x 3, 2 x 6, 4 x 4) as well as on 2 x 4:

* every receive slot of every rank is written exactly once, by the rank the schedule names,
  from the right place in that rank's local arrays (the slot specifications are the ones
  ``foldjax_b200/cp_plan.py`` documents and ``tests/test_cp_plan.py`` proves by simulation);
* the contraction launches of the chunked tri-mult tile the output exactly once, point at the
  slots, and read nothing that arrives in a LATER exchange group than the one that fences them;
* the attention core walks the key tiles in ring order from the right slots, each launch after
  the group that carries its tiles.
"""

from __future__ import annotations

import ctypes as C

import pytest

from foldjax_b200 import _lib
from foldjax_b200.cp_plan import Grid

GRIDS = [(1, 2), (2, 2), (2, 4), (1, 4), (3, 3), (2, 6), (4, 4)]
LOCAL, COPY, PROJECT, CONTRACT, OUTPUT, CORE_TILE = range(6)


def _events(rows, cols, rank, n, op, push):
    lib = _lib.load()
    cap = lib.b200tri_cp_dry_run(rows, cols, rank, n, op, push, None, 0)
    assert cap > 0, lib.b200tri_last_error()
    buf = (_lib.CpEvent * cap)()
    assert lib.b200tri_cp_dry_run(rows, cols, rank, n, op, push, buf, cap) == cap
    return list(buf)


def _layout(rows, cols, rank, n, op):
    out = (C.c_int64 * 16)()
    assert _lib.load().b200tri_cp_layout(rows, cols, rank, n, op, out) == 0
    return list(out)


def _round_up(x, m):
    return (x + m - 1) // m * m


class Slots:
    """Receive regions of one rank: (start, size) -> (source rank, source offset)."""

    def __init__(self):
        self.spec = []

    def add(self, start, size, src, src_off):
        self.spec.append((start, size, src, src_off))

    def check(self, copies, who):
        """copies: (dst_off, bytes, src, src_off, group). Every region covered exactly once, from its source."""
        spans = {i: [] for i in range(len(self.spec))}
        for dst_off, nbytes, src, src_off, _ in copies:
            hit = [i for i, (st, sz, _, _) in enumerate(self.spec) if st <= dst_off and dst_off + nbytes <= st + sz]
            assert len(hit) == 1, f"{who}: copy to [{dst_off}, +{nbytes}) lands in {len(hit)} slots"
            st, sz, want_src, want_off = self.spec[hit[0]]
            assert src == want_src, f"{who}: slot at {st} filled by rank {src}, expected {want_src}"
            assert src_off - want_off == dst_off - st, f"{who}: slot at {st} filled from the wrong place"
            spans[hit[0]].append((dst_off, nbytes))
        for i, (st, sz, _, _) in enumerate(self.spec):
            pos = st
            for off, nbytes in sorted(spans[i]):
                assert off == pos, f"{who}: slot at {st} has a gap or an overlap at {off}"
                pos += nbytes
            assert pos == st + sz, f"{who}: slot at {st} is not filled completely"


def _copies_into(all_events, dst):
    return [(e.dst_off, e.bytes, e.src, e.src_off, e.group) for ev in all_events.values() for e in ev
            if e.kind in (LOCAL, COPY) and e.dst == dst]


@pytest.mark.parametrize("push", [1, 0])
@pytest.mark.parametrize("n_c", [128, 256, 512])
@pytest.mark.parametrize("rows,cols", GRIDS)
def test_trimul_exchange_and_chunked_launches(rows, cols, n_c, push):
    grid = Grid(rows, cols)
    m, n = grid.m, cols * n_c
    n_r = n // rows
    for op, incoming in ((_lib.CP_TRIMUL_OUTGOING, False), (_lib.CP_TRIMUL_INCOMING, True)):
        events = {rank: _events(rows, cols, rank, n, op, push) for rank in grid.ranks()}
        lay = {rank: _layout(rows, cols, rank, n, op) for rank in grid.ranks()}
        for dst in grid.ranks():
            r, c = grid.coords(dst)
            a_all, a_loc, b_all, b_loc, blk, per_slot, t_off, total = lay[dst][:8]
            slots = Slots()
            if not incoming:
                assert per_slot == m
                for cp in range(cols):
                    src = grid.rank(r, cp)
                    slots.add(a_all + m * blk * cp, m * blk, src, lay[src][1])
                    src = grid.rank(c // m, cp)
                    slots.add(b_all + blk * cp, blk, src, lay[src][3] + blk * (c % m))
            else:
                for rp in range(rows):
                    for s in range(m):
                        src = grid.rank(rp, r * m + s)
                        slots.add(a_all + blk * (s * rows + rp), blk, src, lay[src][1])
                    src = grid.rank(rp, c)
                    slots.add(b_all + blk * rp, blk, src, lay[src][3])
            copies = _copies_into(events, dst)
            slots.check(copies, f"{rows}x{cols} rank {dst} op {op}")
            assert max(st + sz for st, sz, _, _ in slots.spec) <= total

            # ---- the launches of this rank
            mine = events[dst]
            n_inner = n_r if incoming else n_c
            ld = _round_up(n_inner, 64)
            if n_c % 64:
                continue
            rb = 128 * 64 * ld * 2                 # one 64-row block of channel-major data
            ldt = _round_up(n_c, 64)
            t_row = 128 * ldt                      # elements between consecutive output rows (64-row blocks)
            n_src = rows if incoming else cols
            covered = set()
            contracts = [e for e in mine if e.kind == CONTRACT]
            outputs = [e for e in mine if e.kind == OUTPUT]
            assert len(contracts) == len(outputs) >= 1
            for e, o in zip(contracts, outputs):
                rel = e.off[2] - t_off
                row0, col0 = rel // (2 * t_row), (rel % (2 * t_row)) // 2
                assert col0 < ldt and row0 % 64 == 0 and col0 % 64 == 0
                assert (o.n_i, o.n_j, o.off[0]) == (e.n_i, e.n_j, e.off[2])      # output stage of the same rectangle
                assert o.off[3] == 2 * (row0 * n_c + col0) * 128                  # ... at the same pairs of the tile
                for rr in range(row0, row0 + e.n_i, 64):
                    for cc in range(col0, col0 + e.n_j, 64):
                        assert (rr, cc) not in covered
                        covered.add((rr, cc))
                # operands: source k of `a` / `b` at a fixed stride from the first one
                s_blk, row_in = divmod(row0, n_c)
                if not incoming:
                    a_first, a_stride = a_all + (row0 // 64) * rb, m * blk
                else:
                    a_first, a_stride = a_all + blk * (s_blk * rows) + (row_in // 64) * rb, blk
                assert (e.off[0], e.off[3]) == (a_first, a_stride)
                assert e.off[1] == b_all + (col0 // 64) * rb
                # nothing the launch reads arrives in a later group than the one that fences it
                reads = [(a_first + k * a_stride, (e.n_i // 64) * rb) for k in range(n_src)]
                reads += [(e.off[1] + k * blk, (e.n_j // 64) * rb) for k in range(n_src)]
                for dst_off, nbytes, _, _, group in copies:
                    for st, sz in reads:
                        if dst_off < st + sz and st < dst_off + nbytes:
                            assert group <= e.group, (rows, cols, dst, op, group, e.group)
            assert covered == {(rr, cc) for rr in range(0, n_r, 64) for cc in range(0, n_c, 64)}


@pytest.mark.parametrize("push", [1, 0])
@pytest.mark.parametrize("n_c", [64, 128])
@pytest.mark.parametrize("rows,cols", GRIDS)
def test_triatt_exchange_and_tile_walk(rows, cols, n_c, push):
    grid = Grid(rows, cols)
    m, n = grid.m, cols * n_c
    n_r = n // rows
    for op, starting in ((_lib.CP_TRIATT_STARTING, True), (_lib.CP_TRIATT_ENDING, False)):
        events = {rank: _events(rows, cols, rank, n, op, push) for rank in grid.ranks()}
        lay = {rank: _layout(rows, cols, rank, n, op) for rank in grid.ranks()}
        n_outer, n_inner = (n_r, n_c) if starting else (n_c, n_r)
        ld = _round_up(n_inner, 64)
        chunk = n_c * ld * 2                       # n_c bias rows of one head
        head_rows = n_outer * ld * 2               # one head of a rank's own bias
        qhead = n_inner * ld * 2                   # one head of a received bias tile
        for dst in grid.ranks():
            r, c = grid.coords(dst)
            q, k_all, vt_all, bias_loc, bias_all, k_tile, vt_tile, bias_tile, tiles, own, total = lay[dst][:11]
            assert tiles == (cols if starting else rows) and own == (c if starting else r)
            assert bias_tile == 4 * qhead
            slots = Slots()
            for t in range(tiles):
                src = grid.rank(r, t) if starting else grid.rank(t, c)
                # (the own tile is written in place by the projection: a local message onto itself)
                slots.add(k_all + k_tile * t, k_tile, src, lay[src][1] + k_tile * t)
                slots.add(vt_all + vt_tile * t, vt_tile, src, lay[src][2] + vt_tile * t)
                for h in range(4):
                    if starting:
                        src = grid.rank(c // m, t)
                        slots.add(bias_all + bias_tile * t + qhead * h, chunk, src, lay[src][3] + head_rows * h + chunk * (c % m))
                    else:
                        for s in range(m):
                            src = grid.rank(t, r * m + s)
                            slots.add(bias_all + bias_tile * t + qhead * h + chunk * s, chunk, src, lay[src][3] + head_rows * h)
            copies = _copies_into(events, dst)
            slots.check(copies, f"{rows}x{cols} rank {dst} op {op}")
            assert max(st + sz for st, sz, _, _ in slots.spec) <= total

            # ---- the key-tile walk: ring order from the own tile, operands in the slots, every
            # launch after the group that carries its tiles (group 0 is the bias group)
            mine = events[dst]
            proj = [e for e in mine if e.kind == PROJECT]
            assert len(proj) == 1 and list(proj[0].off) == [q, k_all + k_tile * own, vt_all + vt_tile * own, bias_loc]
            walk = [e for e in mine if e.kind == CORE_TILE]
            assert [e.n_i for e in walk] == list(range(tiles))
            assert [e.n_j for e in walk] == [(own + i) % tiles for i in range(tiles)]
            launches = [e.group for e in walk]
            assert launches == sorted(launches) and launches[0] == 0 and (tiles == 1 or launches[1] == 1)
            for e in walk:
                t = e.n_j
                assert list(e.off[:3]) == [k_all + k_tile * t, vt_all + vt_tile * t, bias_all + bias_tile * t]
                for dst_off, nbytes, _, _, group in copies:
                    kv = any(st <= dst_off < st + sz for st, sz in ((e.off[0], k_tile), (e.off[1], vt_tile)))
                    if kv and t != own:
                        assert 1 <= group <= e.group, (rows, cols, dst, op, t, group, e.group)
                    elif e.off[2] <= dst_off < e.off[2] + bias_tile:
                        assert group == 0


def test_dry_run_refuses_what_the_ops_refuse():
    lib = _lib.load()
    assert lib.b200tri_cp_dry_run(2, 3, 0, 384, 0, 1, None, 0) == -1   # columns not a multiple of rows
    assert lib.b200tri_cp_dry_run(2, 2, 4, 256, 0, 1, None, 0) == -1   # no such rank
    assert lib.b200tri_cp_dry_run(2, 2, 0, 255, 0, 1, None, 0) == -1   # tokens not divisible by the columns
    assert lib.b200tri_cp_dry_run(2, 2, 0, 256, 7, 1, None, 0) == -1   # no such op
    out = (C.c_int64 * 16)()
    assert lib.b200tri_cp_layout(2, 2, 0, 256, 7, out) == -1
