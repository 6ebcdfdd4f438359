"""prism_fwd_noalloc: the forward for callers that have no way to allocate a device workspace
(code running inside an allocator callback, a server whose device memory is fully pre-assigned,
a plug-in that is only lent input/output buffers).  Its scratch is a fixed array inside the
library, so what has to be shown is that, called through the C ABI, it returns exactly what the
regular prism_fwd returns with a caller workspace -- also on a second call right after the first,
when the shared array still holds the first call's data -- and that it refuses shapes whose
scratch need is larger than the array.  This file is collected last on purpose."""
import ctypes

import pytest
import torch

from cute_mma_b200 import _lib
from oracle import prism_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
DEV = "cuda"
SCRATCH_BYTES = 8 * 1024 * 1024 + 256


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call_pair(L, M, K, N, gs, rs, dt, act, seed):
    A, B, R, _ = [t.to(dt).to(DEV).contiguous() for t in O.make_inputs(M, K, N, gs, rs, seed=seed, b_std=K ** -0.5)]
    code = 1 if dt == torch.bfloat16 else 0
    gate = 1 if act else 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # regular entry point with a caller-provided workspace
    need = L.prism_workspace_bytes(0, M, N, K, gs, rs, code, None)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    C_ref = torch.empty(M, N, dtype=dt, device=DEV)
    _lib.check(L.prism_fwd(_p(A), _p(B), _p(R), None, None, _p(C_ref), M, N, K, gs, rs, code, gate,
                           K, K, K, N, None, _p(ws), need, stream))
    # the variant that brings its own scratch
    C = torch.full((M, N), float("nan"), dtype=dt, device=DEV)
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    _lib.check(L.prism_fwd_noalloc(_p(A), _p(B), _p(R), None, _p(C), M, N, K, gs, rs, code, gate,
                                   K, K, K, N, None, _p(status), stream))
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(C, C_ref)
    ref = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, act)
    assert O.rel_err(C.float(), ref) < TOL


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    L = _lib.lib()
    # reconn_sz = 8: the scratch holds the widened copy of R, different for the two calls
    _call_pair(L, 1024, 256, 1024, 256, 8, torch.float16, "silu_gate", seed=0)
    _call_pair(L, 384, 512, 512, 128, 8, torch.bfloat16, None, seed=1)
    # reconn_sz = 16: only the status header of the scratch is used
    _call_pair(L, 300, 256, 512, 256, 16, torch.bfloat16, "silu_gate", seed=2)


def test_noalloc_refuses_shapes_beyond_its_scratch():
    L = _lib.lib()
    M, K, N, gs, rs = 128, 8192, 16384, 128, 8      # needs 128 * 16 * 8192 * 2 bytes = 32 MiB
    assert L.prism_workspace_bytes(0, M, N, K, gs, rs, 1, None) > SCRATCH_BYTES
    p = ctypes.c_void_p(0x1000)
    rc = L.prism_fwd_noalloc(p, p, p, None, p, M, N, K, gs, rs, 1, 1, K, K, K, N, None, None, None)
    assert rc == 3
    assert b"scratch" in L.prism_last_error_string()
