"""The selector glue against a stand-in FoldJAX package (FoldJAX itself needs JAX,
which is not installed): one spelling reaches every table, unknown values are
errors, nothing falls back silently."""

from __future__ import annotations

import types

import pytest

from foldjax_b200 import backend


def _fake_foldjax():
    pkg = types.SimpleNamespace()
    pkg.execution = types.SimpleNamespace(KNOBS={"triangle_kernel": ("auto", "cueq", "xla"), "dtype": ("bf16", "fp32")})
    pkg.backends = types.SimpleNamespace(
        boltz2=types.SimpleNamespace(TRIANGLE_KERNEL_VALUES={"cueq": "cueq", "xla": "xla"}),
        protenix=types.SimpleNamespace(TRIANGLE_KERNEL_VALUES={"cueq": "cueq_jit", "xla": "xla_jit"}),
        openfold3=types.SimpleNamespace(TRIANGLE_KERNEL_VALUES={"cueq": "cueq", "xla": "xla"}),
        opendde=types.SimpleNamespace(),  # exposes no table on purpose, like the reference
    )
    return pkg


def test_register_adds_the_value_everywhere_and_is_idempotent():
    pkg = _fake_foldjax()
    report = backend.register(pkg)
    assert pkg.execution.KNOBS["triangle_kernel"] == ("auto", "cueq", "xla", "b200")
    assert pkg.backends.protenix.TRIANGLE_KERNEL_VALUES["b200"] == "b200_jit"
    assert pkg.backends.boltz2.TRIANGLE_KERNEL_VALUES["b200"] == "b200"
    assert len(report) == 4
    backend.register(pkg)
    assert pkg.execution.KNOBS["triangle_kernel"].count("b200") == 1
    assert pkg.execution.KNOBS["dtype"] == ("bf16", "fp32")  # other knobs untouched


def test_register_refuses_a_package_without_selector_tables():
    with pytest.raises(RuntimeError, match="no triangle-kernel selector"):
        backend.register(types.SimpleNamespace())


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
