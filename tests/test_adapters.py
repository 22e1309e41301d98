"""Parameter adapters (Protenix / OpenFold3 containers -> this package's mapping),
checked the way the reference checks its Protenix ops: against the explicit formula
(tests/models/protenix/test_triangle.py:22-166, 289-330), on that file's shapes and
seeds (3x3x4 with c_hidden 5, 2 heads x 3; default_rng(7..10)), at its tolerance 1e-5.
The formula below is written with Protenix's own operation order (mask first, separate
a/b projections, torch [out, in] weights); the oracle evaluates the adapted parameters.
"""

from __future__ import annotations

from typing import NamedTuple

import numpy as np
import pytest

from foldjax_b200 import adapters
from oracle import triangle_oracle as orc


class LinearParams(NamedTuple):
    weight: np.ndarray
    bias: np.ndarray | None = None


class LayerNormParams(NamedTuple):
    weight: np.ndarray
    bias: np.ndarray


class TriMul(NamedTuple):
    layer_norm_in: LayerNormParams
    layer_norm_out: LayerNormParams
    linear_a_p: LinearParams
    linear_a_g: LinearParams
    linear_b_p: LinearParams
    linear_b_g: LinearParams
    linear_z: LinearParams
    linear_g: LinearParams


class Attention(NamedTuple):
    linear_q: LinearParams
    linear_k: LinearParams
    linear_v: LinearParams
    linear_o: LinearParams
    linear_g: LinearParams | None


class TriAttProtenix(NamedTuple):
    layer_norm: LayerNormParams
    linear: LinearParams
    attention: Attention


class TriAttOpenFold3(NamedTuple):
    layer_norm: LayerNormParams
    linear_z: LinearParams
    mha: Attention


def _ln(x, p, eps=1e-5):
    mean = x.mean(-1, keepdims=True)
    var = np.square(x - mean).mean(-1, keepdims=True)
    return (x - mean) / np.sqrt(var + eps) * p.weight + p.bias


def _lin(x, p):
    return x @ p.weight.T


def _sig(x):
    return 1.0 / (1.0 + np.exp(-x))


def _trimul_state(rng, c_z, c_hidden) -> TriMul:
    n = lambda *s: rng.normal(size=s)
    return TriMul(LayerNormParams(n(c_z), n(c_z)), LayerNormParams(n(c_hidden), n(c_hidden)),
                  LinearParams(n(c_hidden, c_z)), LinearParams(n(c_hidden, c_z)), LinearParams(n(c_hidden, c_z)),
                  LinearParams(n(c_hidden, c_z)), LinearParams(n(c_z, c_hidden)), LinearParams(n(c_z, c_z)))


@pytest.mark.parametrize("seed,direction", [(7, "outgoing"), (8, "incoming")])
def test_protenix_triangle_multiplication_formula(seed, direction):
    rng = np.random.default_rng(seed)
    z = rng.normal(size=(1, 3, 3, 4))
    mask = rng.integers(0, 2, size=(1, 3, 3)).astype(np.float64)
    p = _trimul_state(rng, 4, 5)
    zn = _ln(z, p.layer_norm_in)
    a = mask[..., None] * _sig(_lin(zn, p.linear_a_g)) * _lin(zn, p.linear_a_p)
    b = mask[..., None] * _sig(_lin(zn, p.linear_b_g)) * _lin(zn, p.linear_b_p)
    spec = "...ikd,...jkd->...ijd" if direction == "outgoing" else "...kid,...kjd->...ijd"
    expected = _lin(_ln(np.einsum(spec, a, b), p.layer_norm_out), p.linear_z) * _sig(_lin(zn, p.linear_g))
    got = orc.triangle_multiplication(adapters.triangle_multiplication_params(p), z, mask, direction, dtype="float64")
    np.testing.assert_allclose(got, expected, rtol=1e-5, atol=1e-5)


def _triatt_reference(x, mask, ln, bias_proj, att, heads, inf=1e9):
    x = _ln(x, ln)

    def project(lin):
        y = _lin(x, lin)
        return np.swapaxes(y.reshape(y.shape[:-1] + (heads, -1)), -2, -3)

    q, k, v = project(att.linear_q), project(att.linear_k), project(att.linear_v)
    q = q / np.sqrt(q.shape[-1])
    logits = np.einsum("...hid,...hjd->...hij", q, k)
    mask_bias = (inf * (mask - 1.0))[..., :, None, None, :]
    tri_bias = np.expand_dims(np.moveaxis(_lin(x, bias_proj), -1, -3), -4)
    logits = logits + mask_bias + tri_bias
    probs = np.exp(logits - logits.max(-1, keepdims=True))
    probs = probs / probs.sum(-1, keepdims=True)
    out = np.swapaxes(np.einsum("...hij,...hjd->...hid", probs, v), -2, -3)
    gate = _sig(_lin(x, att.linear_g))
    out = (out * gate.reshape(gate.shape[:-1] + (heads, -1))).reshape(out.shape[:-2] + (-1,))
    return _lin(out, att.linear_o)


def _triatt_state(rng, c_in, heads, head_dim):
    n = lambda *s: rng.normal(size=s)
    hd = heads * head_dim
    ln = LayerNormParams(n(c_in), n(c_in))
    bias_proj = LinearParams(n(heads, c_in))
    q, k, v, o, g = n(hd, c_in), n(hd, c_in), n(hd, c_in), n(c_in, hd), n(hd, c_in)
    return ln, bias_proj, Attention(LinearParams(q), LinearParams(k), LinearParams(v), LinearParams(o), LinearParams(g))


@pytest.mark.parametrize("container", ["protenix", "openfold3"])
@pytest.mark.parametrize("seed,starting", [(9, True), (10, False)])
def test_triangle_attention_formula(container, seed, starting):
    rng = np.random.default_rng(seed)
    x = rng.normal(size=(1, 3, 3, 4))
    mask = rng.integers(0, 2, size=(1, 3, 3)).astype(np.float64)
    mask[0, np.arange(3), np.arange(3)] = 1.0  # fp64 does not absorb the scores of an all-masked row
    ln, bias_proj, att = _triatt_state(rng, 4, 2, 3)
    params = TriAttProtenix(ln, bias_proj, att) if container == "protenix" else TriAttOpenFold3(ln, bias_proj, att)
    if starting:
        expected = _triatt_reference(x, mask, ln, bias_proj, att, 2)
    else:  # the ending node is the starting node of the transposed pair tensor
        expected = np.swapaxes(_triatt_reference(np.swapaxes(x, -2, -3), np.swapaxes(mask, -1, -2), ln, bias_proj, att, 2),
                               -2, -3)
    got = orc.triangle_attention(adapters.triangle_attention_params(params), x, mask, starting=starting, dtype="float64")
    np.testing.assert_allclose(got, expected, rtol=1e-5, atol=1e-5)


def test_biases_and_missing_gate_are_refused():
    rng = np.random.default_rng(12)
    p = _trimul_state(rng, 4, 5)
    bad = p._replace(linear_z=LinearParams(p.linear_z.weight, np.zeros(4)))
    with pytest.raises(ValueError, match="linear biases are not supported"):
        adapters.triangle_multiplication_params(bad)
    ln, bias_proj, att = _triatt_state(rng, 4, 2, 3)
    with pytest.raises(ValueError, match="without an output gate"):
        adapters.triangle_attention_params(TriAttProtenix(ln, bias_proj, att._replace(linear_g=None)))


def test_adapters_accept_torch_tensors_and_dicts():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(13)
    p = _trimul_state(rng, 4, 5)
    as_np = adapters.triangle_multiplication_params(p)
    as_dict = {name: ({"weight": torch.from_numpy(leaf.weight), "bias": None if leaf.bias is None else torch.from_numpy(leaf.bias)})
               for name, leaf in p._asdict().items()}
    as_torch = adapters.triangle_multiplication_params(as_dict)
    for key in ("p_in", "g_in", "p_out", "g_out"):
        np.testing.assert_array_equal(as_torch[key]["kernel"].numpy(), as_np[key]["kernel"])
    assert as_np["p_in"]["kernel"].shape == (4, 10)  # [in, 2c]: a then b


def test_transition_adapter_matches_torch_layout_formula():
    rng = np.random.default_rng(14)
    x = rng.normal(size=(2, 3, 5))
    norm = LayerNormParams(rng.normal(size=5), rng.normal(size=5))
    fc1, fc2, fc3 = (LinearParams(rng.normal(size=s)) for s in ((11, 5), (11, 5), (5, 11)))
    xn = _ln(x, norm)
    a = _lin(xn, fc1)
    expected = _lin(a * _sig(a) * _lin(xn, fc2), fc3)
    got = orc.transition(adapters.transition_params(norm, fc1, fc2, fc3), x, dtype="float64")
    np.testing.assert_allclose(got, expected, rtol=1e-9, atol=1e-9)


def test_esmfold2_packed_bundle_maps_to_the_fused_projections():
    """ESMFold2's formula (trunk.py:45-91: one `proj_bundle` linear, signal * sigmoid(gate),
    left | right halves) restated here on its own flat parameter names, against the oracle run
    on the adapted mapping."""
    from foldjax_b200 import adapters
    from oracle import triangle_oracle as orc

    rng = np.random.default_rng(41)
    n, c_z, c = 9, 128, 128
    prefix = "trunk.blocks.0.tri_out"
    e = prefix + "._engine"
    flat = {
        f"{e}.norm_start.weight": 1 + 0.1 * rng.standard_normal(c_z), f"{e}.norm_start.bias": 0.1 * rng.standard_normal(c_z),
        f"{e}.proj_bundle.weight": 0.1 * rng.standard_normal((4 * c, c_z)),
        f"{e}.norm_mix.weight": 1 + 0.1 * rng.standard_normal(c), f"{e}.norm_mix.bias": 0.1 * rng.standard_normal(c),
        f"{e}.proj_emit.weight": 0.1 * rng.standard_normal((c_z, c)),
        f"{e}.proj_gate.weight": 0.1 * rng.standard_normal((c_z, c_z)),
    }
    x = rng.standard_normal((1, n, n, c_z))
    mask = (rng.random((1, n, n)) > 0.2).astype(np.float64)

    def ln(v, w, b):
        mu = v.mean(-1, keepdims=True)
        var = ((v - mu) ** 2).mean(-1, keepdims=True)
        return (v - mu) / np.sqrt(var + 1e-5) * w + b

    sig = lambda v: 1 / (1 + np.exp(-v))
    for outgoing in (True, False):
        normed = ln(x, flat[f"{e}.norm_start.weight"], flat[f"{e}.norm_start.bias"])
        bundled = normed @ flat[f"{e}.proj_bundle.weight"].T
        width = bundled.shape[-1] // 2
        routed = bundled[..., :width] * sig(bundled[..., width:]) * mask[..., None]
        left, right = routed[..., : width // 2], routed[..., width // 2:]
        contracted = np.einsum("bikd,bjkd->bijd" if outgoing else "bkid,bkjd->bijd", left, right)
        mixed = ln(contracted, flat[f"{e}.norm_mix.weight"], flat[f"{e}.norm_mix.bias"]) @ flat[f"{e}.proj_emit.weight"].T
        want = mixed * sig(normed @ flat[f"{e}.proj_gate.weight"].T)
        mapped = adapters.esmfold2_triangle_multiplication_params(flat, prefix)
        got = orc.triangle_multiplication(mapped, x, mask, "outgoing" if outgoing else "incoming", dtype="float64")
        np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-11)
    flat[f"{e}.proj_gate.bias"] = np.zeros(c_z)
    with pytest.raises(ValueError, match="biases are not supported"):
        adapters.esmfold2_triangle_multiplication_params(flat, prefix)


def test_stack_layers_builds_the_scan_form():
    from foldjax_b200 import adapters

    layers = [{"a": {"w": np.full((2, 3), i, np.float32)}, "n": 4, "none": None} for i in range(3)]
    stacked = adapters.stack_layers(layers)
    assert stacked["a"]["w"].shape == (3, 2, 3) and stacked["a"]["w"][2, 0, 0] == 2
    assert stacked["n"].tolist() == [4, 4, 4] and stacked["none"] is None
    layers[1]["none"] = 1
    with pytest.raises(ValueError, match="mixed None"):
        adapters.stack_layers(layers)
