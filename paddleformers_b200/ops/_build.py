"""In-tree build and loading of the sm_100a CUDA extension.

The extension is compiled with ``-gencode arch=compute_100a,code=sm_100a`` into
``paddleformers_b200/_ext/pfb200_C.so`` (next to the sources, so the binary travels with the tree) and is loaded
with ``torch.ops.load_library``; its operators appear as ``torch.ops.pfb200.*``.
"""
from __future__ import annotations

import os
import threading

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
EXT_DIR = os.path.join(_PKG_DIR, "_ext")
EXT_NAME = "pfb200_C"
SOURCES = ["bindings.cu", "gemm_sm100.cu", "attention_sm100.cu", "ops_elementwise.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
]

_lock = threading.Lock()
_loaded = False


def ext_path() -> str:
    return os.path.join(EXT_DIR, EXT_NAME + ".so")


def extra_sources() -> list:
    """Optional translation units that are built when present (kept in separate files so that a subset of the
    tree still builds)."""
    out = []
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith(".cu") and name not in SOURCES:
            out.append(name)
    return out


def build_extension(verbose: bool = False) -> str:
    """Compile the extension for sm_100a (works without a GPU: nvcc cross-compiles) and return the .so path."""
    from torch.utils import cpp_extension

    os.makedirs(EXT_DIR, exist_ok=True)
    # An empty arch list makes cpp_extension skip its own -gencode flags; ours are in NVCC_FLAGS.
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    srcs = [os.path.join(CSRC_DIR, s) for s in SOURCES + extra_sources()]
    cpp_extension.load(
        name=EXT_NAME,
        sources=srcs,
        extra_cflags=["-O2", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[CSRC_DIR],
        build_directory=EXT_DIR,
        is_python_module=False,
        verbose=verbose,
    )
    global _loaded
    _loaded = True
    return ext_path()


HOST_SRC_DIR = os.path.join(_PKG_DIR, "csrc_host")
HOST_LIB = os.path.join(EXT_DIR, "pfb_host.so")


def build_host_library() -> str:
    """Compile the host-only C++ helpers (dataset index builders, block-scaled checkpoint converters) into ``_ext/pfb_host.so`` with g++."""
    import subprocess

    os.makedirs(EXT_DIR, exist_ok=True)
    srcs = sorted(os.path.join(HOST_SRC_DIR, f) for f in os.listdir(HOST_SRC_DIR) if f.endswith(".cpp"))
    newest = max(os.path.getmtime(f) for f in srcs)
    if not os.path.exists(HOST_LIB) or os.path.getmtime(HOST_LIB) < newest:
        subprocess.run(["g++", "-O3", "-std=c++17", "-pthread", "-shared", "-fPIC", "-o", HOST_LIB] + srcs, check=True)
    return HOST_LIB


def load_host_library():
    """ctypes handle of the host helpers, or None when the library has not been built."""
    import ctypes

    if not os.path.exists(HOST_LIB):
        return None
    return ctypes.CDLL(HOST_LIB)


def load_extension(required: bool = False) -> bool:
    """Load the prebuilt extension if it exists. Returns True when ``torch.ops.pfb200`` is usable."""
    global _loaded
    with _lock:
        if _loaded:
            return True
        path = ext_path()
        if not os.path.exists(path):
            if required:
                raise RuntimeError(
                    f"CUDA extension {path} is missing; run `python -c 'import __graft_entry__ as g; g.build()'` "
                    "or `python -m paddleformers_b200.ops._build` first"
                )
            return False
        import torch

        torch.ops.load_library(path)
        _loaded = True
        return True


def is_loaded() -> bool:
    return _loaded


if __name__ == "__main__":
    print(build_host_library())
    print(build_extension(verbose=True))
