"""Build / load the in-tree sm_100a extension ``terra_b200_C``.

The shared object is built next to the sources (``terra_b200/_build``) so that it travels with a
snapshot of the tree; ``load()`` imports that file directly and never falls back to another
implementation: on a machine with a GPU a missing extension is an error.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
# TERRA_DEBUG_BOUNDS=1: the bounds-checked build of the kernels (indices that come from tables or from cross-rank
# arithmetic are checked before the access and a violation is reported through the status word, see csrc/common.cuh).
# It is a separate shared object in its own directory, so the two builds never mix.
DEBUG_BOUNDS = os.environ.get("TERRA_DEBUG_BOUNDS", "0") == "1"
# TERRA_GELU_EXACT=1: GELU and its derivative through erff / expf instead of the tanh-based fit (csrc/common.cuh); also a
# build of its own.
GELU_EXACT = os.environ.get("TERRA_GELU_EXACT", "0") == "1"
# TERRA_B200_BUILD_DIR: use (and build into) another directory, e.g. to keep two builds of the kernels side by side
BUILD_DIR = os.environ.get("TERRA_B200_BUILD_DIR") or os.path.join(
    _HERE, "_build" + ("_debug" if DEBUG_BOUNDS else "") + ("_erf" if GELU_EXACT else ""))
EXT_NAME = "terra_b200_C"

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]

if DEBUG_BOUNDS:
    CUDA_FLAGS.append("-DTERRA_DEBUG_BOUNDS")
if GELU_EXACT:
    CUDA_FLAGS.append("-DTERRA_GELU_EXACT_ERF")

_lock = threading.Lock()
_module = None


def sources():
    out = []
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cpp")):
            out.append(os.path.join(CSRC, name))
    return out


def _so_path():
    return os.path.join(BUILD_DIR, EXT_NAME + ".so")


def build(verbose: bool = False):
    """Compile every CUDA/C++ source for sm_100a (cross-compiles without a GPU) and return the module."""
    global _module
    import torch  # noqa: F401  (initialises the dispatcher before the extension is imported)
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    # torch's own arch list is bypassed: the -gencode flags above are the only targets.
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    with _lock:
        mod = cpp_extension.load(
            name=EXT_NAME,
            sources=sources(),
            extra_cflags=["-O3", "-std=c++17"] + (["-DTERRA_DEBUG_BOUNDS"] if DEBUG_BOUNDS else []),
            extra_cuda_cflags=CUDA_FLAGS,
            extra_include_paths=[CSRC],
            build_directory=BUILD_DIR,
            with_cuda=True,
            verbose=verbose,
        )
        _module = mod
    return mod


def load():
    """Import the already built shared object; build it first only if it is absent."""
    global _module
    if _module is not None:
        return _module
    with _lock:
        if _module is not None:
            return _module
        path = _so_path()
        if os.path.exists(path):
            import torch  # noqa: F401

            loader = importlib.machinery.ExtensionFileLoader(EXT_NAME, path)
            spec = importlib.util.spec_from_loader(EXT_NAME, loader)
            mod = importlib.util.module_from_spec(spec)
            loader.exec_module(mod)
            sys.modules[EXT_NAME] = mod
            _module = mod
            return mod
    return build()


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False
