"""The C-ABI library: it builds for sm_100a, loads, exports every symbol that
include/prism_b200.h declares, and rejects bad arguments before touching a GPU."""
import ctypes
import os
import re

import pytest

from cute_mma_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "prism_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(prism_[a-z_0-9]+)\s*\(", text)))


def test_header_and_loader_agree():
    assert _declared_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(built_lib):
    for name in _declared_symbols():
        assert hasattr(built_lib, name), name
    assert built_lib.prism_abi_version() == _lib.ABI_VERSION == 4


def _call_fwd(L, M, N, K, gs, rs, dtype=1, gate=0, ptr=0x1000, ws=0x1000, ws_bytes=1 << 20):
    p = ctypes.c_void_p(ptr)
    return L.prism_fwd(p, p, p, None, None, p, M, N, K, gs, rs, dtype, gate, K, K, K, N, None,
                       ctypes.c_void_p(ws), ws_bytes, None)


@pytest.mark.parametrize("args,code", [
    (dict(M=16, N=64, K=64, gs=32, rs=12), 1),     # reconn_sz not a multiple of 8
    (dict(M=16, N=64, K=64, gs=20, rs=8), 1),      # group_size not a multiple of 8
    (dict(M=16, N=60, K=64, gs=32, rs=8), 1),      # N not divisible by group_size
    (dict(M=16, N=64, K=60, gs=32, rs=8), 1),      # K not divisible by reconn_sz
    (dict(M=16, N=64, K=64, gs=32, rs=8, dtype=7), 1),
    (dict(M=16, N=64, K=64, gs=32, rs=8, gate=3), 1),
    (dict(M=16, N=96, K=96, gs=24, rs=24), 2),     # unsupported reconn_sz
    (dict(M=16, N=48, K=64, gs=24, rs=8), 2),      # unsupported group_size
    (dict(M=16, N=64, K=64, gs=32, rs=8, ptr=0x1004), 1),  # misaligned pointer
    (dict(M=16, N=64, K=64, gs=32, rs=8, ws_bytes=16), 3),  # workspace too small
])
def test_bad_arguments_are_rejected_without_a_gpu(built_lib, args, code):
    assert _call_fwd(built_lib, **args) == code
    assert len(built_lib.prism_last_error_string()) > 0


def test_gradient_dtype_codes_are_checked(built_lib):
    p = ctypes.c_void_p(0x1000)
    rc = built_lib.prism_bwd_db(p, p, p, None, p, 16, 64, 64, 32, 8, 1, 1, 0, ctypes.c_float(1.0), 64, 64, 64, 64, None, ctypes.c_float(0.0), None,
                                p, 1 << 20, None)
    assert rc == 1 and b"db_dtype" in built_lib.prism_last_error_string()   # fp16 gradient of bf16 inputs
    rc = built_lib.prism_dbias(p, p, 16, 60, 1, -1, 64, p, 1 << 20, None)
    assert rc == 1                                                          # N not a multiple of 8


def test_workspace_sizes(built_lib):
    L = built_lib
    hdr = 256
    # rs = 16: forward needs only the status header
    assert L.prism_workspace_bytes(0, 1024, 1024, 256, 256, 16, 1, None) == hdr
    # rs = 8: plus the 16-wide copy of R
    assert L.prism_workspace_bytes(0, 1024, 1024, 256, 256, 8, 1, None) == hdr + 4 * 16 * 256 * 2
    cfg = (ctypes.c_int * 8)(256, 3, 0, 0, 0, 0, 0, 0)
    assert L.prism_workspace_bytes(2, 1024, 1024, 256, 256, 16, 1, cfg) == hdr + 3 * 1024 * 256 * 4
    # dA+dR: the kernel's (halved) copy of R, then 6 partial buffers for 3 CTA pairs per feature column
    cfg = (ctypes.c_int * 8)(3, 0, 0, 0, 0, 0, 0, 0)
    assert L.prism_workspace_bytes(1, 1024, 1024, 256, 256, 16, 1, cfg) == hdr + 4 * 16 * 256 * 2 + 2 * 3 * 4 * 16 * 256 * 4
    # benchmark shape (148 SMs assumed without a GPU): 32 feature columns x 2 runs = 64 main CTA pairs,
    # 10 extra pairs that each help up to 7 main pairs -> 20 CTAs x 7 slabs of [G*E x 128] fp32
    G, E, K = 56, 16, 4096
    want = hdr + G * E * K * 2 + 2 * 2 * G * E * K * 4 + 2 * 10 * 7 * G * E * 128 * 4
    assert L.prism_workspace_bytes(1, 16384, 14336, K, 256, 16, 1, None) == want
    # bias gradient: one fp32 row of N partial sums per row range (64 ranges at most)
    assert L.prism_workspace_bytes(3, 8192, 2304, 0, 0, 0, 1, None) == hdr + 64 * 2304 * 4
    assert L.prism_workspace_bytes(3, 100, 256, 0, 0, 0, 1, None) == hdr + 2 * 256 * 4
    cfg = (ctypes.c_int * 8)(2, -1, 0, 0, 0, 0, 0, 0)   # no extra pairs
    assert L.prism_workspace_bytes(1, 16384, 14336, K, 256, 16, 1, cfg) == hdr + G * E * K * 2 + 2 * 2 * G * E * K * 4
