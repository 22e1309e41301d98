"""Build recipe for libb200tri.so (nvcc, sm_100a only, in-tree).

``python -m foldjax_b200.build`` compiles every ``csrc/*.cu`` into one shared
library next to this file. nvcc cross-compiles, so this works on a machine
without a GPU. The library links the CUDA runtime statically and reaches the
driver only through ``cudaGetDriverEntryPoint``, so it can be loaded (and its
exported symbols checked) where no driver is installed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libb200tri.so"
OBJ = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libb200tri.so cannot be built")
    return exe


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "b200tri.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if sources changed; return its path."""
    stamp = OBJ / "stamp"
    digest = _digest()
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(CSRC.glob("*.cu"))

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objects)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(digest)
    return LIB


FFI_SRC = HERE.parent / "ffi" / "b200tri_ffi.cc"
FFI_LIB = HERE / "libb200tri_ffi.so"


def ffi_include_dir() -> Path | None:
    """Directory holding xla/ffi/api/ffi.h (it ships inside jaxlib), or None."""
    candidates = []
    if os.environ.get("XLA_FFI_INCLUDE_DIR"):
        candidates.append(Path(os.environ["XLA_FFI_INCLUDE_DIR"]))
    try:
        import jax.ffi  # noqa: PLC0415

        candidates.append(Path(jax.ffi.include_dir()))
    except Exception:
        pass
    for c in candidates:
        if (c / "xla" / "ffi" / "api" / "ffi.h").exists():
            return c
    return None


def build_ffi(verbose: bool = False) -> Path | None:
    """Compile the XLA FFI handlers (ffi/b200tri_ffi.cc) against libb200tri.so when the XLA
    FFI headers are available; returns None (and builds nothing) when they are not."""
    inc = ffi_include_dir()
    if inc is None:
        if verbose:
            sys.stderr.write("xla/ffi/api/ffi.h not found (no jaxlib here): libb200tri_ffi.so not built\n")
        return None
    build()
    cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-I", str(inc),
           "-I", str(HERE.parent / "include"), str(FFI_SRC), "-o", str(FFI_LIB),
           f"-L{HERE}", "-l:libb200tri.so", "-Xlinker", "-rpath=$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the FFI handlers failed:\n{res.stdout}\n{res.stderr}")
    return FFI_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_ffi(verbose=True) or "FFI handlers skipped")
