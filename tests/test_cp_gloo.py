"""Host side of the context-parallel layer on CPU ranks (gloo, world size 2) and the
exchange schedule the library executes.

* the C++ message lists (``b200tri_cp_plan``, what ``b200tri_trimul_cp`` /
  ``b200tri_triatt_cp`` post) equal the Python plans that the all-ranks NumPy simulation
  proves on grids up to 4x4;
* ``context_parallel`` on two gloo ranks builds the same grid on both, refuses a device
  count that is not the group's, and maps ``cp_layout="1d"`` to the 1 x P grid;
* the mesh self-test: a complete exchange passes; a half-delivered one (the received
  rows of the peer zeroed ON THE HOST, no device involved) raises on the rank that saw
  it, with the reference's wording (tests/models/test_cp_mesh_check.py:36-51).
"""

from __future__ import annotations

import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
ROOT = Path(__file__).resolve().parents[1]


# ------------------------------------------------------------------ schedule parity
@pytest.mark.parametrize("rows,cols", [(1, 1), (1, 2), (2, 2), (2, 4), (3, 3), (1, 4), (2, 6), (4, 4)])
def test_library_schedule_equals_the_python_plan(rows, cols):
    from foldjax_b200 import _lib, cp_plan

    lib = _lib.load()
    grid = cp_plan.Grid(rows, cols)
    plans = {
        _lib.CP_TRIMUL_OUTGOING: cp_plan.trimul_outgoing_msgs(grid),
        _lib.CP_TRIMUL_INCOMING: cp_plan.trimul_incoming_msgs(grid),
        _lib.CP_TRIATT_STARTING: cp_plan.triatt_starting_msgs(grid),
        _lib.CP_TRIATT_ENDING: cp_plan.triatt_ending_msgs(grid),
    }
    what = {"a": 0, "b": 1, "kv": 2, "bias": 3}
    for op, msgs in plans.items():
        count = lib.b200tri_cp_plan(rows, cols, op, None, 0)
        assert count == len(msgs)
        buf = (_lib.CpMsg * count)()
        assert lib.b200tri_cp_plan(rows, cols, op, buf, count) == count
        for got, want in zip(buf, msgs):
            slot = tuple(want.slot) + (0,) * (2 - len(want.slot))
            assert (got.src, got.dst, got.what, got.block, got.slot0, got.slot1) == (
                want.src, want.dst, what[want.what], -1 if want.block is None else want.block, slot[0], slot[1])


@pytest.mark.parametrize("rows,cols", [(1, 2), (2, 2), (2, 4), (3, 3), (1, 4), (2, 6), (4, 4)])
def test_copy_rounds_are_contention_free(rows, cols):
    """The order in which the ops issue their copies: every remote message gets exactly one
    round, local ones none; in a round no rank sends twice or receives twice; and the number of
    rounds equals the busiest rank's message count, the lower bound."""
    from foldjax_b200 import _lib

    lib = _lib.load()
    for op in (_lib.CP_TRIMUL_OUTGOING, _lib.CP_TRIMUL_INCOMING, _lib.CP_TRIATT_STARTING, _lib.CP_TRIATT_ENDING):
        count = lib.b200tri_cp_plan(rows, cols, op, None, 0)
        msgs = (_lib.CpMsg * count)()
        lib.b200tri_cp_plan(rows, cols, op, msgs, count)
        for what in ((-1,) if op in (_lib.CP_TRIMUL_OUTGOING, _lib.CP_TRIMUL_INCOMING) else (2, 3)):
            rounds = (C.c_int32 * count)()
            assert lib.b200tri_cp_rounds(rows, cols, op, what, rounds, count) == count
            seen: dict[int, tuple[set, set]] = {}
            load: dict[tuple[str, int], int] = {}
            for m, r in zip(msgs, rounds):
                wanted = (what < 0 or m.what == what) and m.src != m.dst
                assert (r >= 0) == wanted
                if not wanted:
                    continue
                senders, receivers = seen.setdefault(r, (set(), set()))
                assert m.src not in senders and m.dst not in receivers, (rows, cols, op, r)
                senders.add(m.src)
                receivers.add(m.dst)
                load[("s", m.src)] = load.get(("s", m.src), 0) + 1
                load[("r", m.dst)] = load.get(("r", m.dst), 0) + 1
            if load:
                assert sorted(seen) == list(range(len(seen)))
                assert len(seen) == max(load.values()), (rows, cols, op, len(seen), max(load.values()))


def test_library_refuses_grids_it_cannot_tile():
    from foldjax_b200 import _lib

    lib = _lib.load()
    assert lib.b200tri_cp_plan(2, 3, 0, None, 0) == -1  # columns not a multiple of rows
    assert b"multiple of rows" in lib.b200tri_last_error()
    assert lib.b200tri_cp_plan(2, 2, 9, None, 0) == -1


# ------------------------------------------------------------------ mesh self-test
def _probe(rows=8, cols=4):
    return np.arange(rows, dtype=np.float32)[:, None] * np.ones((rows, cols), np.float32)


def test_exchange_judgement():
    from foldjax_b200 import cp

    sent = _probe()
    assert cp.exchange_failure(sent.copy(), sent, devices=2) is None
    got = sent.copy()
    got[len(got) // 2:] = 0.0
    message = cp.exchange_failure(got, sent, devices=2)
    assert "4 of 8 rows" in message and "from row 4" in message
    got = sent.copy()
    got[3] += 1.0  # one wrong row is enough
    assert cp.exchange_failure(got, sent, devices=4) is not None


def _worker(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from foldjax_b200 import cp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        ctx = cp.context_parallel(world)  # no CUDA here: a host-only context
        ok &= (ctx.grid.rows, ctx.grid.cols) == (1, 2) and ctx.rank == rank and ctx.comm is None
        ok &= cp.context_parallel(world, layout="1d").grid.cols == 2
        try:
            cp.context_parallel(4)
            ok = False
        except ValueError as exc:
            ok &= "process group has 2 ranks" in str(exc)
        try:
            cp.triangle_multiplication_cp(ctx, {}, torch.zeros(1), None, "outgoing")
            ok = False
        except RuntimeError as exc:
            ok &= "no communicator" in str(exc)

        def gather(shard):  # the same all-gather the device probe performs, over gloo
            parts = [torch.zeros(shard.shape) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(shard))
            return torch.cat(parts).numpy()

        cp.verify_mesh_exchange(world, rank, gather)  # a working mesh passes

        def half_delivered(shard):  # what one broken node did: the peer's rows never arrive
            got = gather(shard)
            peer = 1 - rank
            got[peer * 64:(peer + 1) * 64] = 0.0
            return got

        try:
            cp.verify_mesh_exchange(world, rank, half_delivered)
            ok = False  # 63 or 64 of the peer's rows differ from what was sent: must be reported
        except RuntimeError as exc:
            text = str(exc)
            ok &= "does not exchange data" in text and "rows came back wrong" in text and f"Rank {rank} of 2" in text
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_context_and_mesh_check_on_two_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = 29650 + os.getpid() % 200
        procs = [ctx.Process(target=_worker, args=(rank, 2, port, results)) for rank in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0, f"gloo rank exited with {p.exitcode}"
        assert dict(results) == {0: True, 1: True}


def test_context_needs_a_process_group():
    sys.path.insert(0, str(ROOT))
    from foldjax_b200 import cp

    with pytest.raises(RuntimeError, match="process group"):
        cp.context_parallel(2)
