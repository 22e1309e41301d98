"""Seeded synthetic inputs of the benchmark's shapes (no dataset is available):
pair tensor z ~ N(0,1), linear kernels ~ N(0, 0.02^2) in the reference's
[in, out] layout, layer-norm scale 1 / bias 0, pad mask on the trailing tokens."""

from __future__ import annotations

import numpy as np


def trimul_params(rng: np.random.Generator, c_z: int = 128, c_hidden: int = 128, std: float = 0.02) -> dict:
    w = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    ln = lambda c: {"scale": np.ones(c, np.float32), "bias": np.zeros(c, np.float32)}
    return {
        "norm_in": ln(c_z), "p_in": {"kernel": w(c_z, 2 * c_hidden)}, "g_in": {"kernel": w(c_z, 2 * c_hidden)},
        "norm_out": ln(c_hidden), "p_out": {"kernel": w(c_hidden, c_z)}, "g_out": {"kernel": w(c_z, c_z)},
    }


def triatt_params(rng: np.random.Generator, c_z: int = 128, heads: int = 4, head_dim: int = 32,
                  std: float = 0.02) -> dict:
    w = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    hd = heads * head_dim
    return {
        "layer_norm": {"scale": np.ones(c_z, np.float32), "bias": np.zeros(c_z, np.float32)},
        "linear": {"kernel": w(c_z, heads)},
        "mha": {name: {"kernel": w(c_z if name != "linear_o" else hd, hd if name != "linear_o" else c_z)}
                for name in ("linear_q", "linear_k", "linear_v", "linear_g", "linear_o")},
    }


def transition_params(rng: np.random.Generator, c_z: int = 128, expansion: int = 4, std: float = 0.02) -> dict:
    w = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    hidden = expansion * c_z
    return {
        "norm": {"scale": np.ones(c_z, np.float32), "bias": np.zeros(c_z, np.float32)},
        "fc1": {"kernel": w(c_z, hidden)}, "fc2": {"kernel": w(c_z, hidden)}, "fc3": {"kernel": w(hidden, c_z)},
    }


def block_params(rng: np.random.Generator, transition: bool = False) -> dict:
    """The four triangle sub-modules of a block; with ``transition`` also ``transition_z``."""
    params = {
        "tri_mul_out": trimul_params(rng), "tri_mul_in": trimul_params(rng),
        "tri_att_start": triatt_params(rng), "tri_att_end": triatt_params(rng),
    }
    if transition:
        params["transition_z"] = transition_params(rng)
    return params


def attention_pair_bias_params(rng: np.random.Generator, c_s: int = 384, c_z: int = 128, heads: int = 16,
                               std: float = 0.02) -> dict:
    w = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    return {
        "proj_q": {"kernel": w(c_s, c_s), "bias": w(c_s)}, "proj_k": {"kernel": w(c_s, c_s)},
        "proj_v": {"kernel": w(c_s, c_s)}, "proj_g": {"kernel": w(c_s, c_s)},
        "proj_z_norm": {"scale": np.ones(c_z, np.float32), "bias": np.zeros(c_z, np.float32)},
        "proj_z": {"kernel": w(c_z, heads)}, "proj_o": {"kernel": w(c_s, c_s)},
    }


def pairformer_params(rng: np.random.Generator, c_s: int = 384, heads_s: int = 16) -> dict:
    """Every sub-module of one Pairformer block, by the reference's names
    (trunk_blocks/pairformer.py:126-206)."""
    params = block_params(rng, transition=True)
    params["pre_norm_s"] = {"scale": np.ones(c_s, np.float32), "bias": np.zeros(c_s, np.float32)}
    params["attention"] = attention_pair_bias_params(rng, c_s=c_s, heads=heads_s)
    params["transition_s"] = transition_params(rng, c_z=c_s)
    return params


def pad_mask(n: int, n_pad: int) -> np.ndarray:
    """[1, n, n] float32 pair mask m m^T with the last n_pad tokens dropped."""
    m = np.ones(n, dtype=np.float32)
    if n_pad:
        m[n - n_pad:] = 0.0
    return (m[:, None] * m[None, :])[None]
