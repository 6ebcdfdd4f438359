"""Loader (and in-tree builder) of ``libprism_b200.so``, the C-ABI library with the sm_100a kernels.

The library is compiled ahead of time with ``nvcc`` next to this file; there is no JIT cache,
no per-shape recompilation and no fallback: if the library is missing or cannot be loaded the
import of any compute entry point raises.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.environ.get("PRISM_B200_LIB", os.path.join(_HERE, "libprism_b200.so"))
SOURCES = ["prism_abi.cu", "prism_fwd.cu", "prism_fwd_small.cu", "prism_bwd_db.cu", "prism_bwd_dadr.cu",
           "prism_bwd_dadr_f16.cu", "prism_bwd_dadr_bf16.cu", "prism_fwd_noalloc.cu", "prism_cayley.cu", "prism_peer_reduce.cu"]
HEADERS = ["prism_common.cuh", "prism_host.cuh", "prism_kernels.cuh", "prism_bwd_dadr_kernel.cuh"]
PUBLIC_HEADER = os.path.join(os.path.dirname(_HERE), "include", "prism_b200.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

# every symbol include/prism_b200.h declares
EXPORTS = [
    "prism_fwd", "prism_fwd_dropout", "prism_fwd_noalloc", "prism_bwd_dadr", "prism_bwd_db", "prism_dbias", "prism_fold_weight", "prism_cayley", "prism_cayley_bwd", "prism_peer_reduce", "prism_workspace_bytes",
    "prism_status",
    "prism_last_error_string", "prism_abi_version", "prism_launch_count",
]

ABI_VERSION = 4

_lock = threading.Lock()
_lib = None


def _existing_sources():
    return [os.path.join(_CSRC, s) for s in SOURCES if os.path.exists(os.path.join(_CSRC, s))]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = _existing_sources() + [os.path.join(_CSRC, h) for h in HEADERS] + [PUBLIC_HEADER]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library for sm_100a with nvcc (cross-compiles without a GPU): one object per source
    file, compiled side by side, then one link."""
    if not force and not needs_build():
        return LIB_PATH
    import concurrent.futures
    import tempfile
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose else [])
    objdir = tempfile.mkdtemp(prefix="prism_b200_build_")
    sources = _existing_sources()

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        cmd = [nvcc] + flags + ["-c", "-o", obj, src]
        res = subprocess.run(cmd, cwd=_CSRC, capture_output=True, text=True)
        return obj, cmd, res

    log = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(sources), os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, sources))
    for obj, cmd, res in results:
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        log.append(res.stderr)
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", LIB_PATH] + \
           [obj for obj, _, _ in results]
    res = subprocess.run(link, cwd=_CSRC, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
    for obj, _, _ in results:
        os.remove(obj)
    os.rmdir(objdir)
    if verbose:
        print("\n".join(log))
    return LIB_PATH


class PrismError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"prism_b200 error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (no CPU or torch fallback exists)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                    "or cute_mma_b200._lib.build(); there is no fallback path")
            L = ctypes.CDLL(LIB_PATH)
            vp, ll, i, sz = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_size_t
            ip = ctypes.POINTER(ctypes.c_int)
            L.prism_fwd.restype = i
            L.prism_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, ll, ll, ll, ll, ip, vp, sz, vp]
            L.prism_fwd_dropout.restype = i
            L.prism_fwd_dropout.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, ll, ll, ll, ll, vp, ctypes.c_float,
                                            ip, vp, sz, vp]
            L.prism_fwd_noalloc.restype = i
            L.prism_fwd_noalloc.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, ll, ll, ll, ll, ip, vp, vp]
            if hasattr(L, "prism_bwd_dadr"):
                L.prism_bwd_dadr.restype = i
                L.prism_bwd_dadr.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, ctypes.c_float,
                                             ll, ll, ll, ll, ll, ll, vp, ctypes.c_float, ip, vp, sz, vp]
            if hasattr(L, "prism_bwd_db"):
                L.prism_bwd_db.restype = i
                L.prism_bwd_db.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, ctypes.c_float,
                                           ll, ll, ll, ll, vp, ctypes.c_float, ip, vp, sz, vp]
            L.prism_dbias.restype = i
            L.prism_dbias.argtypes = [vp, vp, i, i, i, i, ll, vp, sz, vp]
            L.prism_fold_weight.restype = i
            L.prism_fold_weight.argtypes = [vp, vp, vp, i, i, i, i, i, ll, ll, ll, vp]
            L.prism_cayley.restype = i
            L.prism_cayley.argtypes = [vp, vp, i, i, i, i, ll, ll, vp]
            L.prism_cayley_bwd.restype = i
            L.prism_cayley_bwd.argtypes = [vp, vp, vp, i, i, i, i, ll, ll, ll, vp]
            L.prism_peer_reduce.restype = i
            L.prism_peer_reduce.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), i, i, ll, i, ctypes.c_float, i, vp]
            L.prism_workspace_bytes.restype = sz
            L.prism_workspace_bytes.argtypes = [i, i, i, i, i, i, i, ip]
            L.prism_status.restype = i
            L.prism_status.argtypes = [vp, vp]
            L.prism_last_error_string.restype = ctypes.c_char_p
            L.prism_last_error_string.argtypes = []
            L.prism_abi_version.restype = i
            if L.prism_abi_version() != ABI_VERSION:
                raise RuntimeError(f"{LIB_PATH} has ABI version {L.prism_abi_version()}, this package needs "
                                   f"{ABI_VERSION}: rebuild it (cute_mma_b200._lib.build(force=True))")
            L.prism_launch_count.restype = ll
            _lib = L
        return _lib


def check(code: int) -> None:
    if code != 0:
        raise PrismError(code, lib().prism_last_error_string().decode("utf-8", "replace"))
