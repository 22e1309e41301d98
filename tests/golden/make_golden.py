"""Generate the golden vectors that pin the oracle.

Run in a container that has the reference checkout (eightmm/FoldJAX) at
``$FOLDJAX_REFERENCE`` (default: a ``reference`` directory beside this repository) and PyTorch:

    python tests/golden/make_golden.py

The reference's XLA path cannot run here (no JAX). Its own test-suite, however,
carries complete PyTorch restatements of both triangle ops, which it asserts
equal to its jnp path within 2e-4 / 3e-4:

* tests/models/boltz2/test_triangle_checkpoint_parity.py
    ``_torch_triangle_multiplication_forward`` (lines 155-192)
* tests/models/boltz2/test_triangle_attention_checkpoint_parity.py
    ``_torch_triangle_attention_forward`` / ``_torch_mha`` (lines 94-147)

and a PyTorch module for the pair transition, asserted equal to 1e-5:

* tests/models/boltz2/test_transition_forward.py ``TorchTransition`` (lines 11-33)
* tests/models/boltz2/test_attention_checkpoint_parity.py
    ``_torch_attention_pair_bias_forward`` (lines 109-148, asserted to 2e-4)

This script imports those test modules from the checkout *unmodified* (JAX
and the FoldJAX package, which the modules import at the top but the helpers do
not touch, are replaced by empty stand-ins), runs the helpers on seeded random
inputs and weights, and stores inputs, weights and outputs in ``*.npz`` next to
this file. The weights those tests normally read come from a checkpoint that is
not available, so seeded N(0, 0.1) weights in the same torch ``[out, in]``
layout stand in; the formulas under test are the reference's own.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

REF = Path(os.environ.get("FOLDJAX_REFERENCE", Path(__file__).resolve().parents[3] / "reference"))
OUT = Path(__file__).resolve().parent


def _stub(name: str, **attrs) -> None:
    mod = types.ModuleType(name)
    mod.__dict__.update(attrs)
    mod.__path__ = []  # behave like a package
    sys.modules[name] = mod


def _load_reference_test(rel: str):
    for name in (
        "jax", "jax.numpy", "foldjax", "foldjax.models", "foldjax.models.boltz2",
        "foldjax.models.boltz2.bridge", "foldjax.models.boltz2.models", "foldjax.models.boltz2.models.triangle",
        "tests", "tests.models", "tests.models.boltz2",
    ):
        _stub(name)
    sys.modules["jax"].numpy = sys.modules["jax.numpy"]
    _stub("foldjax.models.boltz2.bridge.torch_mapping", map_triangle_multiplication_state_dict=None,
          map_triangle_attention_state_dict=None, map_transition_state_dict=None)
    sys.modules["foldjax.models.boltz2.bridge.torch_mapping"].map_attention_pair_bias_state_dict = None
    _stub("foldjax.models.boltz2.models.primitives")
    _stub("foldjax.models.boltz2.models.primitives.attention", attention_pair_bias_forward=None)
    _stub("foldjax.models.boltz2.models.primitives.transition", transition_forward=None)
    _stub("foldjax.models.boltz2.models.triangle.triangle", triangle_multiplication_forward=None)
    _stub("foldjax.models.boltz2.models.triangle.triangle_attention", triangle_attention_forward=None)
    _stub("tests.models.boltz2.torch_checkpoint", load_torch_checkpoint_state_dict=None)
    path = REF / rel
    spec = importlib.util.spec_from_file_location("_ref_" + path.stem, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _w(gen: torch.Generator, *shape, std: float = 0.1) -> torch.Tensor:
    return torch.randn(*shape, generator=gen, dtype=torch.float32) * std


def _mask(gen: torch.Generator, n: int, keep: float, pad: int) -> torch.Tensor:
    m = (torch.rand(1, n, n, generator=gen) < keep).float()
    idx = torch.arange(n)
    m[0, idx, idx] = 1.0  # every row keeps at least one key
    if pad:
        m[0, n - pad:, :] = 0.0
        m[0, :, n - pad:] = 0.0
    return m


def make_trimul(mod, seed: int, n: int, c: int, keep: float, pad: int) -> dict:
    gen = torch.Generator().manual_seed(seed)
    prefix = "layer"
    state = {
        f"{prefix}.norm_in.weight": 1.0 + _w(gen, c),
        f"{prefix}.norm_in.bias": _w(gen, c),
        f"{prefix}.p_in.weight": _w(gen, 2 * c, c),
        f"{prefix}.g_in.weight": _w(gen, 2 * c, c),
        f"{prefix}.norm_out.weight": 1.0 + _w(gen, c),
        f"{prefix}.norm_out.bias": _w(gen, c),
        f"{prefix}.p_out.weight": _w(gen, c, c),
        f"{prefix}.g_out.weight": _w(gen, c, c),
    }
    x = torch.randn(1, n, n, c, generator=gen, dtype=torch.float32)
    mask = _mask(gen, n, keep, pad)
    out = {"x": x.numpy(), "mask": mask.numpy()}
    for key, val in state.items():
        out["w." + key[len(prefix) + 1:]] = val.numpy()
    for direction in ("outgoing", "incoming"):
        y = mod._torch_triangle_multiplication_forward(state, prefix, x, mask, direction)
        out["out." + direction] = y.detach().numpy()
    return out


def make_triatt(mod, seed: int, n: int, c: int, heads: int, hidden: int, keep: float, pad: int) -> dict:
    gen = torch.Generator().manual_seed(seed)
    prefix = "layer"
    hd = heads * hidden
    state = {
        f"{prefix}.layer_norm.weight": 1.0 + _w(gen, c),
        f"{prefix}.layer_norm.bias": _w(gen, c),
        f"{prefix}.linear.weight": _w(gen, heads, c, std=0.5),
        f"{prefix}.mha.linear_q.weight": _w(gen, hd, c, std=0.3),
        f"{prefix}.mha.linear_k.weight": _w(gen, hd, c, std=0.3),
        f"{prefix}.mha.linear_v.weight": _w(gen, hd, c),
        f"{prefix}.mha.linear_g.weight": _w(gen, hd, c),
        f"{prefix}.mha.linear_o.weight": _w(gen, c, hd),
    }
    x = torch.randn(1, n, n, c, generator=gen, dtype=torch.float32)
    mask = _mask(gen, n, keep, pad)
    out = {"x": x.numpy(), "mask": mask.numpy(), "heads": np.int64(heads), "hidden": np.int64(hidden)}
    for key, val in state.items():
        out["w." + key[len(prefix) + 1:]] = val.numpy()
    for name, starting in (("starting", True), ("ending", False)):
        y = mod._torch_triangle_attention_forward(state, prefix, x, mask, starting=starting)
        out["out." + name] = y.detach().numpy()
    return out


def make_transition(mod, seed: int, rows: tuple[int, ...], dim: int, hidden: int) -> dict:
    torch.manual_seed(seed)
    module = mod.TorchTransition(dim=dim, hidden_dim=hidden).eval()
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        module.norm.weight.copy_(1.0 + _w(gen, dim))
        module.norm.bias.copy_(_w(gen, dim))
        x = torch.randn(*rows, dim, generator=gen, dtype=torch.float32)
        out = {"x": x.numpy(), "out": module(x).numpy(), "out.chunked": module(x, chunk_size=max(1, hidden // 3)).numpy()}
    for key, val in module.state_dict().items():  # torch [out, in] layout
        out["w." + key] = val.detach().numpy()
    return out


def make_attention_pair_bias(mod, seed: int, n: int, c_s: int, c_z: int, heads: int) -> dict:
    gen = torch.Generator().manual_seed(seed)
    prefix = mod.PREFIX
    state = {
        f"{prefix}.proj_q.weight": _w(gen, c_s, c_s), f"{prefix}.proj_q.bias": _w(gen, c_s),
        f"{prefix}.proj_k.weight": _w(gen, c_s, c_s), f"{prefix}.proj_v.weight": _w(gen, c_s, c_s),
        f"{prefix}.proj_g.weight": _w(gen, c_s, c_s), f"{prefix}.proj_o.weight": _w(gen, c_s, c_s),
        f"{prefix}.proj_z.0.weight": 1.0 + _w(gen, c_z), f"{prefix}.proj_z.0.bias": _w(gen, c_z),
        f"{prefix}.proj_z.1.weight": _w(gen, heads, c_z, std=0.5),
    }
    s = torch.randn(1, n, c_s, generator=gen)
    k_in = torch.randn(1, n, c_s, generator=gen)
    z = torch.randn(1, n, n, c_z, generator=gen)
    mask = (torch.rand(1, n, generator=gen) < 0.8).float()
    mask[0, 0] = 1.0
    out = {"s": s.numpy(), "k_in": k_in.numpy(), "z": z.numpy(), "mask": mask.numpy()}
    for key, val in state.items():
        out["w." + key[len(prefix) + 1:]] = val.numpy()
    out["out"] = mod._torch_attention_pair_bias_forward(state, s, z, mask, k_in).detach().numpy()
    return out


def main() -> None:
    torch.manual_seed(0)
    tm = _load_reference_test("tests/models/boltz2/test_triangle_checkpoint_parity.py")
    ta = _load_reference_test("tests/models/boltz2/test_triangle_attention_checkpoint_parity.py")
    # Small generic shapes (any channel count) and one case at the kernels' width.
    np.savez_compressed(OUT / "trimul_n7_c8.npz", **make_trimul(tm, 11, n=7, c=8, keep=0.8, pad=0))
    np.savez_compressed(OUT / "trimul_n12_c128.npz", **make_trimul(tm, 12, n=12, c=128, keep=0.85, pad=2))
    np.savez_compressed(OUT / "triatt_n7_c8.npz", **make_triatt(ta, 13, n=7, c=8, heads=2, hidden=4, keep=0.8, pad=0))
    np.savez_compressed(OUT / "triatt_n12_c128.npz",
                        **make_triatt(ta, 14, n=12, c=128, heads=4, hidden=32, keep=0.85, pad=2))
    tr = _load_reference_test("tests/models/boltz2/test_transition_forward.py")
    np.savez_compressed(OUT / "transition_d5_h11.npz", **make_transition(tr, 15, rows=(2, 3), dim=5, hidden=11))
    np.savez_compressed(OUT / "transition_d128_h512.npz", **make_transition(tr, 16, rows=(3, 8), dim=128, hidden=512))
    ap = _load_reference_test("tests/models/boltz2/test_attention_checkpoint_parity.py")
    np.savez_compressed(OUT / "attention_pair_bias_n7.npz", **make_attention_pair_bias(ap, 17, n=7, c_s=12, c_z=8, heads=3))
    np.savez_compressed(OUT / "attention_pair_bias_n12_c96.npz",  # head dim 24 and c_z 128 as in the trunk
                        **make_attention_pair_bias(ap, 18, n=12, c_s=96, c_z=128, heads=4))
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
