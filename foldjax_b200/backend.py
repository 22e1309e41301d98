"""Selector glue: makes "b200" a value of FoldJAX's triangle-kernel option surface.

FoldJAX has no single registry object for triangle kernels; the "registry" is a
set of tables and dispatch sites (src/foldjax/execution.py:40-50 KNOBS,
src/foldjax/backends/boltz2.py:162-165, protenix.py:181-184, openfold3.py:168-170,
and the dispatch in boltz2 triangle_attention.py:384-418 / triangle.py:67-76).
``register(foldjax)`` adds the new value to the tables it finds on an importable
FoldJAX package and returns what it changed; the dispatch-site edits a maintainer
makes are listed in INTEGRATION.md. FoldJAX (and JAX) are not installed next to
this repository, so this module is exercised against a stand-in package in the
tests. Policy kept from the reference: an unknown value is an error and nothing
falls back silently (tests/test_execution_vocabulary.py:140-155).
"""

from __future__ import annotations

import os
from types import ModuleType
from typing import Any, Callable

BACKEND = "b200"

# env vars the reference's ports read at trace time (per model)
ENV_VARS = {
    "boltz2_tri_mult": "BOLTZ_JAX_TRIANGLE_MULTIPLICATION_BACKEND",
    "protenix_tri_attn": "PROTENIX_TRIANGLE_BACKEND",
    "protenix_tri_mult": "PROTENIX_TRIANGLE_MULTIPLICATION_BACKEND",
    "openfold3_tri_attn": "OPENFOLD3_TRIANGLE_BACKEND",
}


def resolve(value: str | None, allowed: tuple[str, ...] = ("auto", "cueq", "xla", BACKEND)) -> str:
    """Normalise a ``triangle_kernel`` option the way execution.normalize does:
    unknown values raise, ``auto`` resolves to the fastest kernel that really runs
    here (this backend, when its library loads and a GPU is present)."""
    v = (value or "auto").lower()
    if v not in allowed:
        raise ValueError(f"unknown triangle_kernel {value!r}; expected one of {allowed}")
    if v != "auto":
        return v
    try:
        import torch

        from . import _lib

        _lib.load()
        return BACKEND if torch.cuda.is_available() else "xla"
    except Exception:
        return "xla"


def register(foldjax: ModuleType | Any) -> dict[str, Any]:
    """Add "b200" to every selector table found on ``foldjax``. Returns a report
    {site: new value}; raises if no site was found (a silent no-op would hide a
    layout change upstream)."""
    changed: dict[str, Any] = {}
    execution = getattr(foldjax, "execution", None)
    knobs = getattr(execution, "KNOBS", None)
    if isinstance(knobs, dict) and "triangle_kernel" in knobs:
        values = tuple(knobs["triangle_kernel"])
        if BACKEND not in values:
            knobs["triangle_kernel"] = values + (BACKEND,)
        changed["execution.KNOBS['triangle_kernel']"] = knobs["triangle_kernel"]
    backends = getattr(foldjax, "backends", None)
    for model, suffix in (("boltz2", ""), ("protenix", "_jit"), ("openfold3", "")):
        mod = getattr(backends, model, None)
        table = getattr(mod, "TRIANGLE_KERNEL_VALUES", None)
        if isinstance(table, dict):
            table.setdefault(BACKEND, BACKEND + suffix)
            changed[f"backends.{model}.TRIANGLE_KERNEL_VALUES"] = dict(table)
    if not changed:
        raise RuntimeError("no triangle-kernel selector table found on the given foldjax package")
    return changed


def select_by_env(model_op: str, value: str = BACKEND, environ=os.environ) -> str:
    """Set the env var one of the reference's ports reads for its triangle backend
    (explicit env wins over option tables there, tests/test_triangle_backend_reach.py)."""
    if model_op not in ENV_VARS:
        raise KeyError(f"unknown model/op {model_op!r}; known: {sorted(ENV_VARS)}")
    environ[ENV_VARS[model_op]] = value
    return ENV_VARS[model_op]


def operators() -> dict[str, Callable]:
    """The operator entry points this backend provides, by the reference's names."""
    from .attention import attention_pair_bias_forward
    from .transition import transition_forward
    from .triangle import triangle_multiplication_forward
    from .triangle_attention import attention_core, triangle_attention_forward

    return {
        "triangle_multiplication_forward": triangle_multiplication_forward,
        "triangle_attention_forward": triangle_attention_forward,
        "attention_core": attention_core,
        "transition_forward": transition_forward,
        "attention_pair_bias_forward": attention_pair_bias_forward,
    }
