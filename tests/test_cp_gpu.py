"""Multi-GPU context-parallel parity: needs at least 2 GPUs on the box; each case
runs tests/cp_worker.py under torchrun (one process per GPU, NCCL) and checks that
the gathered tiles equal the single-GPU kernels on the full tensor."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = Path(__file__).resolve().parents[1]


def _run(world: int, tokens: int, transport: str = "push", layout: str = "") -> str:
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, CP_TEST_TOKENS=str(tokens), NCCL_NVLS_ENABLE="0", B200TRI_CP_TRANSPORT=transport,
               CP_TEST_LAYOUT=layout)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(ROOT / "tests" / "cp_worker.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900)
    assert done.returncode == 0 and "CP_WORKER_OK" in done.stdout, done.stdout[-3000:] + done.stderr[-3000:]
    return done.stdout


@pytest.mark.parametrize("world,tokens", [(2, 512), (2, 200), (2, 256), (4, 512), (4, 256), (4, 1024), (4, 1536),
                                          (8, 1024), (8, 256), (8, 3072)])
def test_context_parallel_matches_single_gpu(world, tokens):
    """Tiles written into the peers' mapped workspaces by the senders (the default transport)."""
    out = _run(world, tokens)
    assert "transport: push" in out, out[-2000:]
    print(out)


@pytest.mark.parametrize("world,tokens", [(4, 512), (4, 1024)])
def test_context_parallel_on_a_one_row_grid(world, tokens):
    """1 x 4: four key tiles per row, so the peers' tiles arrive and are computed in groups."""
    out = _run(world, tokens, layout="1x4")
    assert "transport: push" in out, out[-2000:]
    print(out)


@pytest.mark.parametrize("world,tokens", [(2, 256), (4, 512), (8, 1024)])
def test_context_parallel_pulling_tiles(world, tokens):
    """The same ops with every receiver reading its tiles out of the owners' mapped workspaces."""
    out = _run(world, tokens, transport="pull")
    assert "transport: pull" in out, out[-2000:]
    print(out)


@pytest.mark.parametrize("world,tokens", [(2, 256), (4, 512), (8, 1024)])
def test_context_parallel_over_nccl_send_recv(world, tokens):
    """The same ops with the tiles sent and received by NCCL into a caller-provided workspace."""
    out = _run(world, tokens, transport="nccl")
    assert "transport: nccl" in out, out[-2000:]
    print(out)
