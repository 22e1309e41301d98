"""Host-side proof of the 2-D context-parallel tile schedules: every rank of an
R x C grid, simulated in NumPy with exactly the messages the plan lists, must
reproduce the dense operators. Grids beyond one box (3x3, 2x6, 4x4) are included
because a 2x2 grid cannot falsify a swapped index (the reference makes the same
point, tests/models/boltz2/test_context_parallel.py:51-54)."""

from __future__ import annotations

import numpy as np
import pytest

from foldjax_b200.cp_plan import Grid, grid_for, key_order, trimul_outgoing_msgs, triatt_starting_msgs
from oracle import cp_oracle as cpo
from oracle import triangle_oracle as orc

GRIDS = [(1, 1), (1, 2), (2, 2), (2, 4), (3, 3), (2, 6), (4, 4)]


def test_grid_for_matches_the_option_surface():
    assert (grid_for(2).rows, grid_for(2).cols) == (1, 2)
    assert (grid_for(4).rows, grid_for(4).cols) == (2, 2)
    assert (grid_for(8).rows, grid_for(8).cols) == (2, 4)
    assert (grid_for(8, "2x4").rows, grid_for(8, "2x4").cols) == (2, 4)
    with pytest.raises(ValueError):
        grid_for(6)
    with pytest.raises(ValueError):
        Grid(4, 2)  # columns must be a multiple of rows
    with pytest.raises(ValueError):
        Grid(2, 4).tile_shape(30)


@pytest.mark.parametrize("rows,cols", GRIDS)
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_trimul_schedule_reproduces_the_contraction(rows, cols, direction):
    grid = Grid(rows, cols)
    n = 2 * rows * cols if rows * cols > 1 else 6
    n = n if n % cols == 0 else cols * rows * 2
    rng = np.random.default_rng(rows * 10 + cols)
    a = rng.standard_normal((n, n, 3))
    b = rng.standard_normal((n, n, 3))
    got = cpo.simulate_trimul(grid, a, b, direction)
    np.testing.assert_allclose(got, orc.triangle_contraction(a, b, direction), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("rows,cols", GRIDS)
@pytest.mark.parametrize("starting", [True, False])
def test_triatt_schedule_reproduces_dense_attention(rows, cols, starting):
    grid = Grid(rows, cols)
    n = 2 * cols * max(1, rows // 1) if cols > 1 else 6
    h, d = 2, 3
    rng = np.random.default_rng(100 + rows * 10 + cols)
    q = rng.normal(size=(n, n, h, d), scale=0.5)
    k = rng.normal(size=(n, n, h, d), scale=0.5)
    v = rng.normal(size=(n, n, h, d))
    bias = rng.normal(size=(h, n, n), scale=4.0)  # large: the running max moves between key tiles
    keep = rng.random((n, n)) > 0.25
    keep[:, 0] = True
    mb = np.where(keep, 0.0, -1e9)
    # dense reference in the oracle's operand order [B, I, H, J, D]
    ref = orc.attention_core(q.transpose(0, 2, 1, 3)[None], k.transpose(0, 2, 1, 3)[None],
                             v.transpose(0, 2, 1, 3)[None], bias[None, None], mb[None, :, None, None, :])
    ref = ref[0].transpose(0, 2, 1, 3)
    got = cpo.simulate_triatt(grid, q, k, v, bias, mb, starting)
    np.testing.assert_allclose(got, ref, rtol=1e-9, atol=1e-9)


def test_every_step_has_distinct_senders_per_receiver_group():
    """The rotated key order makes the C ranks of a grid row fetch from C different
    peers at every step (no sender serves two receivers of the group at once)."""
    grid = Grid(2, 4)
    for step in range(grid.cols):
        for r in range(grid.rows):
            srcs = [key_order(grid, grid.rank(r, c), True)[step] for c in range(grid.cols)]
            assert sorted(srcs) == list(range(grid.cols))


def test_message_lists_are_complete_and_local_copies_are_marked():
    grid = Grid(2, 4)
    msgs = trimul_outgoing_msgs(grid)
    assert len(msgs) == grid.size * grid.cols * 2
    assert sum(m.src == m.dst for m in msgs if m.what == "a") == grid.size
    att = triatt_starting_msgs(grid)
    for dst in grid.ranks():
        slots = sorted(m.slot for m in att if m.dst == dst and m.what == "kv")
        assert slots == [(c,) for c in range(grid.cols)]


@pytest.mark.parametrize("rows,cols,n", [(2, 2, 13), (2, 4, 13), (3, 3, 13), (1, 2, 9)])
def test_padding_to_the_grid_leaves_the_real_block_unchanged(rows, cols, n):
    """Token counts the grid does not divide (the reference's Cannon test runs N = 12
    and 13): zero-padded pairs and dropped padded keys give the unpadded result on
    the real block, for the contraction and for the attention."""
    from foldjax_b200.cp_plan import padded_tokens

    grid = Grid(rows, cols)
    n_pad = padded_tokens(n, grid)
    assert n_pad % cols == 0 and n_pad % rows == 0 and 0 <= n_pad - n < cols
    rng = np.random.default_rng(1000 + rows * 10 + cols)
    a, b = rng.standard_normal((n, n, 3)), rng.standard_normal((n, n, 3))
    ap, bp = np.zeros((n_pad, n_pad, 3)), np.zeros((n_pad, n_pad, 3))
    ap[:n, :n], bp[:n, :n] = a, b
    for direction in ("outgoing", "incoming"):
        got = cpo.simulate_trimul(grid, ap, bp, direction)[:n, :n]
        np.testing.assert_allclose(got, orc.triangle_contraction(a, b, direction), rtol=1e-12, atol=1e-12)
    h, d = 2, 3
    q, k, v = (rng.normal(size=(n, n, h, d), scale=0.5) for _ in range(3))
    bias = rng.normal(size=(h, n, n), scale=4.0)
    keep = rng.random((n, n)) > 0.25
    keep[:, 0] = True
    mb = np.where(keep, 0.0, -1e9)
    ref = orc.attention_core(q.transpose(0, 2, 1, 3)[None], k.transpose(0, 2, 1, 3)[None], v.transpose(0, 2, 1, 3)[None],
                             bias[None, None], mb[None, :, None, None, :])[0].transpose(0, 2, 1, 3)

    def pad(x, axes, fill=0.0):
        shape = list(x.shape)
        for ax in axes:
            shape[ax] = n_pad
        out = np.full(shape, fill)
        out[tuple(slice(0, s) for s in x.shape)] = x
        return out

    qp, kp, vp = pad(q, (0, 1)), pad(k, (0, 1)), pad(v, (0, 1))
    got = cpo.simulate_triatt(grid, qp, kp, vp, pad(bias, (1, 2)), pad(mb, (0, 1), fill=-np.inf), True)[:n, :n]
    np.testing.assert_allclose(got, ref, rtol=1e-9, atol=1e-9)
