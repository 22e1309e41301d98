"""The selector glue: one spelling reaches every table, unknown values are errors,
nothing falls back silently.

Two targets. (1) FoldJAX's real option layer - ``foldjax.execution`` and
``foldjax.backends.{boltz2,protenix,openfold3}`` import without JAX - when a FoldJAX
checkout sits beside this repository (``../reference/src``) or ``FOLDJAX_SRC`` points
at one; the test is skipped otherwise. (2) A stand-in with the same structure
(``execution.KNOBS`` plus ``<Model>Backend.execution_options``), so the logic is
covered on a machine without the checkout.
"""

from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path

import pytest

from foldjax_b200 import backend


def _fake_backend(native_name: str, suffix: str = ""):
    class FakeBackend:
        execution_options = {
            "dtype": ("compute_dtype", {"float32": "float32"}),
            "triangle_kernel": (native_name, {"auto": "cueq" + suffix, "cueq": "cueq" + suffix, "xla": "xla" + suffix}),
        }

    return FakeBackend


def _fake_foldjax():
    pkg = types.SimpleNamespace(__name__="fake_foldjax")
    pkg.execution = types.SimpleNamespace(KNOBS={"triangle_kernel": ("auto", "cueq", "xla"), "dtype": ("bf16", "fp32")})

    class OpenDDEBackend:  # exposes no triangle knob on purpose, like the reference
        execution_options = {}

    pkg.backends = types.SimpleNamespace(
        boltz2=types.SimpleNamespace(Boltz2Backend=_fake_backend("triangle_backend")),
        protenix=types.SimpleNamespace(ProtenixBackend=_fake_backend("trunk_triangle_attention_backend", "_jit")),
        openfold3=types.SimpleNamespace(OpenFold3Backend=_fake_backend("triangle_kernel")),
        opendde=types.SimpleNamespace(OpenDDEBackend=OpenDDEBackend),
    )
    return pkg


def test_register_adds_the_value_everywhere_and_is_idempotent():
    pkg = _fake_foldjax()
    report = backend.register(pkg)
    assert pkg.execution.KNOBS["triangle_kernel"] == ("auto", "cueq", "xla", "b200")
    name, values = pkg.backends.protenix.ProtenixBackend.execution_options["triangle_kernel"]
    assert name == "trunk_triangle_attention_backend" and values["b200"] == "b200_jit" and values["xla"] == "xla_jit"
    assert pkg.backends.boltz2.Boltz2Backend.execution_options["triangle_kernel"][1]["b200"] == "b200"
    assert pkg.backends.openfold3.OpenFold3Backend.execution_options["triangle_kernel"][1]["b200"] == "b200"
    assert len(report) == 4
    assert backend.register(pkg) == report
    assert pkg.execution.KNOBS["triangle_kernel"].count("b200") == 1
    assert pkg.execution.KNOBS["dtype"] == ("bf16", "fp32")  # other knobs untouched
    assert "triangle_kernel" not in pkg.backends.opendde.OpenDDEBackend.execution_options


def test_register_refuses_a_package_without_selector_tables():
    with pytest.raises(RuntimeError, match="KNOBS"):
        backend.register(types.SimpleNamespace(__name__="empty"))
    pkg = _fake_foldjax()
    pkg.backends = types.SimpleNamespace()
    with pytest.raises(RuntimeError, match="no model backend"):
        backend.register(pkg)


def _foldjax_src() -> Path | None:
    candidates = [os.environ.get("FOLDJAX_SRC"), Path(__file__).resolve().parents[2] / "reference" / "src"]
    for c in candidates:
        if c and (Path(c) / "foldjax" / "execution.py").exists():
            return Path(c)
    return None


@pytest.fixture
def real_foldjax():
    src = _foldjax_src()
    if src is None:
        pytest.skip("no FoldJAX checkout beside this repository")
    sys.path.insert(0, str(src))
    try:
        yield importlib.import_module("foldjax")
    finally:
        sys.path.remove(str(src))
        for name in [m for m in sys.modules if m == "foldjax" or m.startswith("foldjax.")]:
            del sys.modules[name]


def test_register_on_the_real_option_layer(real_foldjax):
    """normalize -> translate carries triangle_kernel=b200 to each model's native option,
    old spellings still work, and an unknown value still raises (the policy of the
    reference's tests/test_execution_vocabulary.py:140-155)."""
    execution = importlib.import_module("foldjax.execution")
    report = backend.register(real_foldjax)
    assert "b200" in execution.KNOBS["triangle_kernel"]
    assert len(report) == 4, report
    expected = {
        "boltz2": ("Boltz2Backend", "triangle_backend", "b200"),
        "protenix": ("ProtenixBackend", "trunk_triangle_attention_backend", "b200_jit"),
        "openfold3": ("OpenFold3Backend", "triangle_kernel", "b200"),
    }
    for model, (cls_name, native_name, native_value) in expected.items():
        cls = getattr(importlib.import_module(f"foldjax.backends.{model}"), cls_name)
        table = cls.execution_options
        opts = execution.normalize({"triangle_kernel": "b200"}, native=set())
        out = execution.translate(opts, table, model=model)
        assert out == {native_name: native_value}, (model, out)
        # values that were there before still translate as before
        assert execution.translate({"triangle_kernel": "xla"}, table, model=model)[native_name].startswith("xla")
        with pytest.raises(ValueError, match="triangle_kernel must be one of"):
            execution.translate({"triangle_kernel": "pallas"}, table, model=model)
    # the old spelling of the knob reaches the same place
    with pytest.warns(execution.Alias):
        opts = execution.normalize({"trunk_triangle_attention_backend": "b200"}, native=set())
    assert opts == {"triangle_kernel": "b200"}
    # OpenDDE exposes no triangle knob and must keep refusing it
    opendde = importlib.import_module("foldjax.backends.opendde")
    with pytest.raises(ValueError, match="does not support triangle_kernel"):
        execution.translate({"triangle_kernel": "b200"}, opendde.OpenDDEBackend.execution_options, model="opendde")


def test_unknown_value_is_an_error_and_auto_never_invents_a_backend():
    with pytest.raises(ValueError, match="unknown triangle_kernel"):
        backend.resolve("pallas")
    assert backend.resolve("xla") == "xla"
    assert backend.resolve("B200") == "b200"
    assert backend.resolve("auto") in ("b200", "xla")  # "xla" on a machine without a GPU


def test_env_selection_uses_the_reference_variable_names():
    env = {}
    assert backend.select_by_env("boltz2_tri_mult", environ=env) == "BOLTZ_JAX_TRIANGLE_MULTIPLICATION_BACKEND"
    assert env == {"BOLTZ_JAX_TRIANGLE_MULTIPLICATION_BACKEND": "b200"}
    with pytest.raises(KeyError):
        backend.select_by_env("esmfold2", environ=env)


def test_operator_names_match_the_reference():
    ops = backend.operators()
    assert set(ops) == {"triangle_multiplication_forward", "triangle_attention_forward", "attention_core",
                        "transition_forward", "attention_pair_bias_forward"}
