"""The C-ABI library loads without a GPU and exports every symbol the header declares."""

from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols() -> set[str]:
    text = (ROOT / "include" / "b200tri.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(b200tri_[a-z0-9_]+)\s*\(", text))


def test_library_exports_every_declared_symbol():
    from foldjax_b200 import _lib

    lib = _lib.load()
    declared = _declared_symbols()
    assert declared, "no declarations found in include/b200tri.h"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.b200tri_version() >= 100


def test_argument_validation_needs_no_gpu():
    from foldjax_b200 import _lib

    lib = _lib.load()
    assert lib.b200tri_trimul_workspace_bytes(0) == 0
    assert lib.b200tri_trimul_workspace_bytes(256) > 3 * 128 * 256 * 256 * 2
    assert lib.b200tri_trimul_forward(None, None) == _lib.ERR_INVALID
    assert b"null args" in lib.b200tri_last_error()
    args = _lib.TrimulContractArgs(n_i=0)
    assert lib.b200tri_trimul_contract(C.byref(args), None) == _lib.ERR_INVALID


def test_struct_sizes_match_the_header():
    """ctypes mirrors must have the C layout: compile a probe with gcc and compare."""
    import shutil
    import subprocess
    import tempfile

    from foldjax_b200 import _lib

    gcc = shutil.which("gcc")
    if gcc is None:
        import pytest

        pytest.skip("gcc not available")
    names = dict(_lib.STRUCTS)
    header = (ROOT / "include" / "b200tri.h").read_text()
    assert set(re.findall(r"}\s*(b200tri_[a-z_]+_(?:args|msg|event));", header)) == set(names)
    assert set(re.findall(r"}\s*(b200tri_[a-z_]+_params);", header)) == set(_lib.PARAM_STRUCTS)
    names.update(_lib.PARAM_STRUCTS)
    src = '#include <stdio.h>\n#include "b200tri.h"\nint main(void){\n'
    for cname in names:
        src += f'  printf("{cname} %zu\\n", sizeof({cname}));\n'
    src += "  return 0; }\n"
    with tempfile.TemporaryDirectory() as tmp:
        c_file = Path(tmp) / "probe.c"
        c_file.write_text(src)
        exe = Path(tmp) / "probe"
        subprocess.run([gcc, "-I", str(ROOT / "include"), str(c_file), "-o", str(exe)], check=True)
        out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    sizes = dict(line.split() for line in out.strip().splitlines())
    for cname, struct in names.items():
        assert int(sizes[cname]) == C.sizeof(struct), cname
