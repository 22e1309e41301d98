"""Worker for the multi-GPU context-parallel tests (launched by torchrun).

Every rank builds the same seeded full-size problem, keeps its own tile, runs the
context-parallel op through the C ABI (b200tri_trimul_cp / b200tri_triatt_cp), and rank 0
gathers the tiles and compares them with the single-GPU kernels on the full tensor and, at
N <= 256, with the CPU oracle's bf16 emulation of the reference.
Exit code 0 = all comparisons passed.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main() -> int:
    from conftest import assert_parity
    from foldjax_b200 import _device as dev, _lib, cp
    from foldjax_b200.block import triangle_block_forward
    from foldjax_b200.synthetic import block_params, pad_mask, triatt_params, trimul_params
    from foldjax_b200.triangle import triangle_multiplication_forward
    from foldjax_b200.triangle_attention import triangle_attention_forward
    from oracle import triangle_oracle as orc  # the checker, at small N

    n = int(os.environ.get("CP_TEST_TOKENS", "512"))
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = cp.context_parallel(layout=os.environ.get("CP_TEST_LAYOUT") or None)
    grid = ctx.grid
    rng = np.random.default_rng(7)
    pm_np, pa_np = trimul_params(rng, std=0.05), triatt_params(rng, std=0.05)
    pm_np, pa_np = orc.round_params(pm_np, "bfloat16"), orc.round_params(pa_np, "bfloat16")
    pm = dev.params_to_device(pm_np)
    pa = dev.params_to_device(pa_np)
    pb = dev.params_to_device(block_params(np.random.default_rng(8), transition=True))
    gen = torch.Generator(device="cpu").manual_seed(11)
    z_full = torch.randn(n, n, 128, generator=gen).to(torch.bfloat16).cuda()
    mask_full = torch.from_numpy(pad_mask(n, max(1, n // 40))[0]).cuda()
    z_tile = cp.shard_pair(ctx, z_full)
    n_r, n_c = grid.tile_shape(n)
    failures = 0

    def gather(tile):
        tiles = [torch.empty_like(tile) for _ in range(grid.size)] if ctx.rank == 0 else None
        dist.gather(tile, tiles, dst=0)
        if ctx.rank != 0:
            return None
        full = torch.empty(n, n, 128, dtype=tile.dtype, device=tile.device)
        for rk, t in enumerate(tiles):
            r, c = grid.coords(rk)
            full[r * n_r:(r + 1) * n_r, c * n_c:(c + 1) * n_c] = t
        return full

    cases = [("trimul outgoing", lambda: cp.triangle_multiplication_cp(ctx, pm, z_tile, mask_full, "outgoing"),
              lambda: triangle_multiplication_forward(pm, z_full, mask_full[None], "outgoing")),
             ("trimul incoming", lambda: cp.triangle_multiplication_cp(ctx, pm, z_tile, mask_full, "incoming"),
              lambda: triangle_multiplication_forward(pm, z_full, mask_full[None], "incoming")),
             ("triatt starting", lambda: cp.triangle_attention_cp(ctx, pa, z_tile, mask_full, starting=True),
              lambda: triangle_attention_forward(pa, z_full, mask_full[None], starting=True)),
             ("triatt ending", lambda: cp.triangle_attention_cp(ctx, pa, z_tile, mask_full, starting=False),
              lambda: triangle_attention_forward(pa, z_full, mask_full[None], starting=False)),
             # the whole pair track of a block, residual adds and the (row-local) pair transition included
             ("block with transition", lambda: cp.triangle_block_cp(ctx, pb, z_tile, mask_full),
              lambda: triangle_block_forward(pb, z_full[None], mask_full[None])[0])]
    for name, run_cp, run_single in cases:
        tile = run_cp()
        _lib.device_status()
        full = gather(tile)
        if ctx.rank == 0:
            ref = run_single()
            _lib.device_status()
            valid = mask_full.bool().any(dim=1)  # rows/cols with a valid key
            ok_rows = valid[:, None, None].expand_as(ref) if "ending" not in name else valid[None, :, None].expand_as(ref)
            if name.startswith("block"):  # fully padded rows and columns pass through both attention nodes
                ok_rows = (valid[:, None, None] & valid[None, :, None]).expand_as(ref)
            elif "triatt" not in name:
                ok_rows = torch.ones_like(ref, dtype=torch.bool)
            try:
                info = assert_parity(ref.float().cpu().numpy(), full.float().cpu().numpy(),
                                     where=ok_rows.cpu().numpy(), label=f"{grid.rows}x{grid.cols} {name} N={n}",
                                     mean_tol=1e-3)
                print(info, flush=True)
                if n <= 256 and not name.startswith("block"):
                    # the CPU oracle's bf16 emulation of the reference, at the benchmark's tolerance
                    x_np = z_full.float().cpu().numpy()[None]
                    m_np = mask_full.cpu().numpy()[None]
                    if name.startswith("trimul"):
                        emu = orc.triangle_multiplication(pm_np, x_np, m_np, name.split()[1], dtype="bfloat16")[0]
                    else:
                        emu = orc.triangle_attention(pa_np, x_np, m_np, starting=name.endswith("starting"),
                                                     dtype="bfloat16")[0]
                    print(assert_parity(emu, full.float().cpu().numpy(), where=ok_rows.cpu().numpy(),
                                        label=f"{grid.rows}x{grid.cols} {name} N={n} vs oracle"), flush=True)
            except AssertionError as exc:
                failures += 1
                print("FAILED", exc, flush=True)
    # a second call must give the same tile (buffers are reused, transfers re-posted)
    a = cp.triangle_attention_cp(ctx, pa, z_tile, mask_full, starting=True)
    b = cp.triangle_attention_cp(ctx, pa, z_tile, mask_full, starting=True)
    if not torch.equal(a, b):
        failures += 1
        print("FAILED: repeated call differs", flush=True)
    flag = torch.tensor([failures], device="cuda")
    dist.all_reduce(flag)
    pulls = bool(_lib.load().b200tri_comm_pulls(ctx.comm))
    ctx.close()
    dist.destroy_process_group()
    if ctx.rank == 0:
        print(f"transport: {cp.TRANSPORT if pulls else 'nccl'}", flush=True)
        print("CP_WORKER_OK" if flag.item() == 0 else "CP_WORKER_FAILED", flush=True)
    return int(flag.item() != 0)


if __name__ == "__main__":
    sys.exit(main())
