"""Parameter-container adapters: Protenix / OpenFold3 / OpenDDE -> the Boltz-style
mapping the operators of this package take.

The reference keeps two parameter conventions for the same ops:

* Boltz-2: nested dicts, kernels stored ``[in, out]``, fused projections
  (``p_in``/``g_in`` of width 2c hold a then b), no biases
  (src/foldjax/models/boltz2/bridge/torch_mapping.py:513-600);
* Protenix, OpenFold3 (and OpenDDE, which reuses Protenix's): ``NamedTuple``s of
  ``LinearParams(weight [out, in], bias | None)`` and
  ``LayerNormParams(weight, bias)``, with SEPARATE ``linear_a_p / a_g / b_p / b_g``
  (src/foldjax/models/protenix/models/primitives/primitives.py:11-30,
  src/foldjax/models/protenix/models/triangle/triangle.py:77-98,
  src/foldjax/models/openfold3/models/triangle.py:40-54,
  src/foldjax/models/openfold3/models/triangle_attention.py:83-92).

The arithmetic is the same: Protenix's ``mask * sigmoid(g) * p`` and Boltz's
``sigmoid(g) * p * mask`` agree for 0/1 masks, ``a`` is the first half of the
fused projection in both (Boltz triangle.py:102), and the attention differs only
in names. These functions only transpose, concatenate and rename - they work on
NumPy arrays and torch tensors alike and never touch a GPU.

Linear biases: every triangle projection is bias-free upstream (OpenFold3 says so
in its docstrings; Protenix uses LinearNoBias), so a non-None bias is refused
rather than silently dropped.
"""

from __future__ import annotations

from typing import Any

import numpy as np


def _get(node: Any, name: str) -> Any:
    if isinstance(node, dict):
        return node[name]
    return getattr(node, name)


def _t(w: Any) -> Any:
    """[out, in] -> [in, out] for NumPy arrays and torch tensors."""
    if isinstance(w, np.ndarray):
        return np.ascontiguousarray(w.T)
    if hasattr(w, "t") and hasattr(w, "contiguous"):
        return w.t().contiguous()
    return np.ascontiguousarray(np.asarray(w).T)


def _cat(a: Any, b: Any) -> Any:
    if isinstance(a, np.ndarray):
        return np.concatenate([a, b], axis=-1)
    import torch

    return torch.cat([a, b], dim=-1)


def _kernel(linear: Any, what: str) -> Any:
    if _get(linear, "bias") is not None:
        raise ValueError(f"{what}: linear biases are not supported by the b200 backend (the projection is bias-free upstream)")
    return _t(_get(linear, "weight"))


def _norm(ln: Any, what: str) -> dict:
    weight, bias = _get(ln, "weight"), _get(ln, "bias")
    if weight is None or bias is None:
        raise ValueError(f"{what}: the b200 backend needs both the layer-norm scale and offset")
    return {"scale": weight, "bias": bias}


def triangle_multiplication_params(params: Any) -> dict:
    """Protenix / OpenFold3 ``TriangleMultiplicationParams`` -> the mapping
    ``triangle_multiplication_forward`` takes."""
    a_p, b_p = _kernel(_get(params, "linear_a_p"), "linear_a_p"), _kernel(_get(params, "linear_b_p"), "linear_b_p")
    a_g, b_g = _kernel(_get(params, "linear_a_g"), "linear_a_g"), _kernel(_get(params, "linear_b_g"), "linear_b_g")
    return {
        "norm_in": _norm(_get(params, "layer_norm_in"), "layer_norm_in"),
        "p_in": {"kernel": _cat(a_p, b_p)},
        "g_in": {"kernel": _cat(a_g, b_g)},
        "norm_out": _norm(_get(params, "layer_norm_out"), "layer_norm_out"),
        "p_out": {"kernel": _kernel(_get(params, "linear_z"), "linear_z")},
        "g_out": {"kernel": _kernel(_get(params, "linear_g"), "linear_g")},
    }


def triangle_attention_params(params: Any) -> dict:
    """Protenix (``linear`` + ``attention``) or OpenFold3 (``linear_z`` + ``mha``)
    ``TriangleAttentionParams`` -> the mapping ``triangle_attention_forward`` takes."""
    has = (lambda n: n in params) if isinstance(params, dict) else (lambda n: hasattr(params, n))
    bias_proj = _get(params, "linear" if has("linear") else "linear_z")
    mha = _get(params, "attention" if has("attention") else "mha")
    gate = _get(mha, "linear_g")
    if gate is None:
        raise ValueError("triangle attention without an output gate is not supported by the b200 backend")
    return {
        "layer_norm": _norm(_get(params, "layer_norm"), "layer_norm"),
        "linear": {"kernel": _kernel(bias_proj, "pair-bias projection")},
        "mha": {name: {"kernel": _kernel(_get(mha, name), name)}
                for name in ("linear_q", "linear_k", "linear_v", "linear_g", "linear_o")},
    }


def transition_params(norm: Any, fc1: Any, fc2: Any, fc3: Any) -> dict:
    """Torch-layout transition weights (``norm``, and ``[out, in]`` ``fc1``/``fc2``/``fc3``
    linears) -> the mapping ``transition_forward`` takes."""
    return {
        "norm": _norm(norm, "norm"),
        "fc1": {"kernel": _kernel(fc1, "fc1")},
        "fc2": {"kernel": _kernel(fc2, "fc2")},
        "fc3": {"kernel": _kernel(fc3, "fc3")},
    }


def esmfold2_triangle_multiplication_params(params: Any, prefix: str) -> dict:
    """ESMFold2's flat checkpoint mapping -> the mapping ``triangle_multiplication_forward``
    takes. ESMFold2 packs the four input projections into ONE linear, ``proj_bundle`` of
    width 4c with torch ``[out, in]`` weights: rows [0, 2c) are the signal (left | right, our
    a | b) and rows [2c, 4c) the gate logits (src/foldjax/models/esmfold2/models/trunk.py:52-62);
    ``proj_emit`` / ``proj_gate`` are our ``p_out`` / ``g_out``, ``norm_start`` / ``norm_mix``
    our ``norm_in`` / ``norm_out`` (:84-91). ``prefix`` names the
    ``TriangleMultiplicativeUpdate``; the ``_engine`` level is added here as the reference does
    (:45). Biases are optional in that checkpoint format; these projections carry none, and one
    that does is refused rather than dropped."""
    engine = f"{prefix}._engine" if prefix else "_engine"

    def weight(name: str) -> Any:
        if params.get(f"{engine}.{name}.bias") is not None:
            raise ValueError(f"{engine}.{name}: linear biases are not supported by the b200 backend")
        return params[f"{engine}.{name}.weight"]

    bundle = weight("proj_bundle")  # [4c, c_z]
    width = bundle.shape[0] // 2
    return {
        "norm_in": {"scale": params[f"{engine}.norm_start.weight"], "bias": params[f"{engine}.norm_start.bias"]},
        "p_in": {"kernel": _t(bundle[:width])},
        "g_in": {"kernel": _t(bundle[width:])},
        "norm_out": {"scale": params[f"{engine}.norm_mix.weight"], "bias": params[f"{engine}.norm_mix.bias"]},
        "p_out": {"kernel": _t(weight("proj_emit"))},
        "g_out": {"kernel": _t(weight("proj_gate"))},
    }


def stack_layers(layers: list) -> Any:
    """Per-layer parameter mappings -> ONE mapping whose leaves carry a leading layer axis,
    the form the reference's scan carries (stack_leaves / prestack_layer_lists,
    src/foldjax/models/_stacking.py:46-120) and ``pairformer_forward(..., num_blocks=L)`` takes.
    A leaf that is None must be None in every layer."""
    first = layers[0]
    if isinstance(first, dict):
        return {k: stack_layers([layer[k] for layer in layers]) for k in first}
    if first is None:
        if any(leaf is not None for leaf in layers):
            raise ValueError("cannot stack mixed None/non-None layer leaves")
        return None
    if isinstance(first, np.ndarray) or np.isscalar(first):
        return np.stack([np.asarray(leaf) for leaf in layers])
    import torch

    return torch.stack(list(layers))
