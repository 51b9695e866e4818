"""Build and load the in-tree sm_100a kernel library.

The library is compiled from ``csrc/*.cu`` (kernels, no torch headers) and ``csrc/bindings.cpp``
(torch op registrations) into ``_build/ws_b200_C.so`` next to this file.  ``build()`` cross-compiles
without a GPU; ``load()`` loads the shared object and registers ``torch.ops.ws_b200.*``.  A stamp
file with a hash of the sources decides whether a rebuild is needed, so a machine that received
a prebuilt ``.so`` never invokes the compiler.

On a machine with a CUDA device a missing library is an error (`require()`): the CUDA ops never
fall back silently to PyTorch there.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import threading
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
CSRC = _HERE / "csrc"
BUILD_DIR = _HERE / "_build"
LIB_NAME = "ws_b200_C"
LIB_PATH = BUILD_DIR / f"{LIB_NAME}.so"
STAMP = BUILD_DIR / "sources.sha256"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]

_lock = threading.Lock()
_loaded = False
_cdll = None


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _source_hash() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.cuh"))
                       + list(CSRC.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_built() -> bool:
    return LIB_PATH.exists() and STAMP.exists() and STAMP.read_text().strip() == _source_hash()


def build(verbose: bool = False) -> Path:
    """Compile the library for sm_100a (works without a GPU)."""
    if is_built():
        return LIB_PATH
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=LIB_NAME,
        sources=[str(p) for p in sources()],
        extra_cflags=["-O2", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(CSRC)],
        build_directory=str(BUILD_DIR),
        is_python_module=False,
        verbose=verbose,
    )
    STAMP.write_text(_source_hash())
    return LIB_PATH


def load() -> bool:
    """Load the library if it exists (building it when the toolchain is present)."""
    global _loaded, _cdll
    with _lock:
        if _loaded:
            return True
        if not is_built():
            try:
                build()
            except Exception:
                if torch.cuda.is_available():
                    raise
                return False
        torch.ops.load_library(str(LIB_PATH))
        _cdll = ctypes.CDLL(str(LIB_PATH))
        _loaded = True
        return True


def require() -> None:
    if not load():
        raise RuntimeError("warpstate_ai_b200: the sm_100a kernel library is not built "
                           "(run `python -c 'import __graft_entry__ as g; g.build()'`)")


def available() -> bool:
    """True when CUDA kernels can run: a CUDA device is present and the library is loaded."""
    if not torch.cuda.is_available():
        return False
    require()
    return True


def cdll():
    require()
    return _cdll


def launch_count() -> int:
    if not _loaded:
        return 0
    fn = _cdll.ws_launch_count
    fn.restype = ctypes.c_longlong
    return int(fn())
