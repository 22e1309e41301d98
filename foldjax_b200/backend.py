"""Selector glue: makes "b200" a value of FoldJAX's triangle-kernel option surface.

FoldJAX has no single registry object for triangle kernels; the "registry" is a
set of tables and dispatch sites:

* ``foldjax.execution.KNOBS["triangle_kernel"]`` (src/foldjax/execution.py:40-45),
  the neutral vocabulary ``normalize``/``translate`` check values against;
* one ``execution_options["triangle_kernel"] = (native option name, {neutral value:
  native value})`` entry per model backend class: ``Boltz2Backend``
  (src/foldjax/backends/boltz2.py:160-165), ``ProtenixBackend`` (protenix.py:179-184,
  native values carry a ``_jit`` suffix) and ``OpenFold3Backend``
  (openfold3.py:168-170); OpenDDE exposes no such knob on purpose;
* the dispatch inside the ports (boltz2 triangle_attention.py:384-418 /
  triangle.py:67-76 and their Protenix / OpenFold3 counterparts), which a
  maintainer extends with the stubs shown in this repository's integration notes.

``register(foldjax)`` adds the new value to the first two kinds of table on an
imported FoldJAX package and returns what it changed. The option layer of FoldJAX
imports without JAX, so the tests run this against the real modules when a FoldJAX
checkout sits beside this repository (and against a stand-in with the same
structure otherwise). Policy kept from the reference: an unknown value is an error
and nothing falls back silently (tests/test_execution_vocabulary.py:140-155).
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


# model backend module -> the native spelling of the value in that port
NATIVE_VALUES = {"boltz2": BACKEND, "protenix": BACKEND + "_jit", "openfold3": BACKEND}


def _backend_classes(module: ModuleType | Any):
    """Classes of a ``foldjax.backends.<model>`` module that carry a triangle-kernel entry."""
    for name, obj in sorted(vars(module).items()):
        if not isinstance(obj, type):
            continue
        table = obj.__dict__.get("execution_options")
        if isinstance(table, dict) and "triangle_kernel" in table:
            yield name, obj, table


def register(foldjax: ModuleType | Any) -> dict[str, Any]:
    """Add "b200" to every triangle-kernel selector table found on ``foldjax``.

    ``foldjax.execution`` and ``foldjax.backends.<model>`` are imported on demand (none
    of them needs JAX). Returns a report {site: new value}. Raises if the neutral
    vocabulary or every model table is missing: a silent no-op would hide a layout
    change upstream. Calling it twice changes nothing the second time."""
    import importlib

    changed: dict[str, Any] = {}
    pkg = getattr(foldjax, "__name__", "foldjax")

    def sub(name: str):
        parts = name.split(".")
        obj: Any = foldjax
        for part in parts:
            nxt = getattr(obj, part, None)
            if nxt is None:
                try:
                    nxt = importlib.import_module(f"{getattr(obj, '__name__', pkg)}.{part}")
                except Exception:
                    return None
            obj = nxt
        return obj

    execution = sub("execution")
    knobs = getattr(execution, "KNOBS", None)
    if not (isinstance(knobs, dict) and "triangle_kernel" in knobs):
        raise RuntimeError("foldjax.execution.KNOBS['triangle_kernel'] not found: the option layer changed upstream")
    values = tuple(knobs["triangle_kernel"])
    if BACKEND not in values:
        knobs["triangle_kernel"] = values + (BACKEND,)
    changed["execution.KNOBS['triangle_kernel']"] = knobs["triangle_kernel"]

    models = 0
    for model, native in NATIVE_VALUES.items():
        mod = sub(f"backends.{model}")
        if mod is None:
            continue
        for cls_name, _cls, table in _backend_classes(mod):
            native_name, mapping = table["triangle_kernel"]
            if mapping.get(BACKEND) != native:
                mapping = dict(mapping)
                mapping[BACKEND] = native
                table["triangle_kernel"] = (native_name, mapping)
            changed[f"backends.{model}.{cls_name}.execution_options['triangle_kernel']"] = table["triangle_kernel"]
            models += 1
    if models == 0:
        raise RuntimeError("no model backend with a triangle_kernel entry found on the given foldjax package")
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
