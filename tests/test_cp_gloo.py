"""The exchange executor on CPU: two gloo ranks on a 1x2 grid post exactly the
messages of the plan (point-to-point sends/receives plus local copies) and must
end up with the panels the plan promises."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
ROOT = Path(__file__).resolve().parents[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from foldjax_b200 import cp
    from foldjax_b200.cp_plan import trimul_outgoing_msgs, triatt_starting_msgs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ctx = cp.context_parallel(world)
        grid = ctx.grid
        assert (grid.rows, grid.cols) == (1, 2)
        m, cols = grid.m, grid.cols
        # tile contents encode (owner rank, array, block)
        a_loc = torch.full((m, 4), 100.0 + rank)
        b_loc = torch.stack([torch.full((4,), 200.0 + 10 * rank + s) for s in range(m)])
        a_all = torch.zeros(cols, m, 4)
        b_all = torch.zeros(cols, 4)

        def views(msg, side):
            if side == "send":
                src = a_loc if msg.what == "a" else b_loc
                return [src if msg.block is None else src[msg.block]]
            return [a_all[msg.slot[0]] if msg.what == "a" else b_all[msg.slot[0]]]

        for w in cp._post(ctx, trimul_outgoing_msgs(grid), views):
            w.wait()
        r, c = ctx.coords
        ok = True
        for cp_ in range(cols):
            ok &= bool((a_all[cp_] == 100.0 + grid.rank(r, cp_)).all())
            ok &= bool((b_all[cp_] == 200.0 + 10 * grid.rank(c // m, cp_) + c % m).all())
        # attention messages carry two tensors (k, v) and four bias chunks each
        k_all, v_all = torch.zeros(cols, 3), torch.zeros(cols, 5)
        k_all[c], v_all[c] = 1.0 + rank, 11.0 + rank
        bias_loc = torch.arange(4 * m * 2, dtype=torch.float32).reshape(4, m * 2, 1) + 1000 * rank
        bias_all = torch.zeros(cols, 4, 2, 1)

        def aviews(msg, side):
            if msg.what == "kv":
                return [k_all[c], v_all[c]] if side == "send" else [k_all[msg.slot[0]], v_all[msg.slot[0]]]
            if side == "send":
                return [bias_loc[h, msg.block * 2:(msg.block + 1) * 2] for h in range(4)]
            return [bias_all[msg.slot[0], h] for h in range(4)]

        for w in cp._post(ctx, triatt_starting_msgs(grid), aviews):
            w.wait()
        for cp_ in range(cols):
            src = grid.rank(r, cp_)
            ok &= bool((k_all[cp_] == 1.0 + src).all()) and bool((v_all[cp_] == 11.0 + src).all())
            bsrc = grid.rank(c // m, cp_)
            want = (torch.arange(4 * m * 2, dtype=torch.float32).reshape(4, m * 2, 1) + 1000 * bsrc)[:, (c % m) * 2:(c % m) * 2 + 2]
            ok &= bool((bias_all[cp_] == want).all())
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_exchange_executor_on_two_gloo_ranks():
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


def test_context_needs_a_process_group_and_rejects_1d():
    sys.path.insert(0, str(ROOT))
    from foldjax_b200 import cp

    with pytest.raises(RuntimeError, match="process group"):
        cp.context_parallel(2)
