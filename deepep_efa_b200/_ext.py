"""Builds and loads the native extension ``_dx`` (C++ host runtime + sm_100a CUDA kernels) in-tree.

The shared object is written next to the sources (``deepep_efa_b200/_build/_dx.so``) so that it
travels with the source tree to machines that have no compiler cache. A content hash of all sources
and flags is stored beside it; when the hash matches, the existing ``.so`` is imported directly and no
compiler runs.

The reference builds its extension with ``setup.py`` (``setup.py:16-137``: 14 sources, ``-lfabric
-lgdrapi``); this build needs neither libfabric nor GDRCopy.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path
from typing import Optional

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_BUILD = _PKG / "_build"
_NAME = "_dx"
_LOCK = threading.Lock()
_MODULE = None

CUDA_SOURCES = [
    "kernels/layout.cu",
    "kernels/normal.cu",
    "kernels/fp8_cast.cu",
    "kernels/ll.cu",
    "kernels/grouped_gemm.cu",
    "kernels/permute.cu",
    "kernels/noalloc.cu",
    "kernels/hier.cu",
    "kernels/train_ops.cu",
    "kernels/sf_atoms.cu",
    "kernels/fused.cu",
]
CPP_SOURCES = [
    "host/bindings.cpp",
    "host/gemm_bindings.cpp",
    "host/hier_bindings.cpp",
    "host/fused_bindings.cpp",
]

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-Wno-unused-variable", "-Wno-sign-compare"]


def _sources():
    cu = [str(_CSRC / s) for s in CUDA_SOURCES if (_CSRC / s).exists()]
    cpp = [str(_CSRC / s) for s in CPP_SOURCES]
    return cpp + cu


def _content_hash() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in _CSRC.rglob("*") if p.suffix in (".cu", ".cuh", ".h", ".hpp", ".cpp"))
    for p in files:
        h.update(str(p.relative_to(_CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(CUDA_FLAGS + CXX_FLAGS).encode())
    import torch

    h.update(torch.__version__.encode())
    return h.hexdigest()


def _import_so(path: Path):
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(_NAME, str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def so_path() -> Path:
    return _BUILD / f"{_NAME}.so"


def build(verbose: bool = False, force: bool = False):
    """Compile the extension for sm_100a if the in-tree build is missing or stale, then import it."""
    global _MODULE
    with _LOCK:
        if _MODULE is not None and not force:
            return _MODULE
        _BUILD.mkdir(exist_ok=True)
        want = _content_hash()
        stamp = _BUILD / f"{_NAME}.hash"
        so = so_path()
        if not force and so.exists() and stamp.exists() and stamp.read_text().strip() == want:
            _MODULE = _import_so(so)
            return _MODULE
        if os.environ.get("DEEPEP_B200_NO_BUILD") == "1":
            raise ImportError(f"{so} is missing or stale and DEEPEP_B200_NO_BUILD=1 forbids compiling")
        from torch.utils import cpp_extension

        os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 8)))
        mod = cpp_extension.load(
            name=_NAME,
            sources=_sources(),
            extra_cflags=CXX_FLAGS,
            extra_cuda_cflags=CUDA_FLAGS,
            extra_include_paths=[str(_CSRC)],
            build_directory=str(_BUILD),
            verbose=verbose,
            with_cuda=True,
        )
        stamp.write_text(want)
        _MODULE = mod
        return _MODULE


def load():
    """Return the native module, building it on first use."""
    return build()


def is_built() -> bool:
    stamp = _BUILD / f"{_NAME}.hash"
    return so_path().exists() and stamp.exists() and stamp.read_text().strip() == _content_hash()
