"""GPU tests of the boundary features around the three kernels: non-finite propagation, fp32
gradient outputs, the bias-gradient kernel, the ``cute_prism`` import name and its custom ops, the
per-stream workspaces, and the bounded-wait error path."""
import ctypes
import os
import subprocess
import threading

import pytest
import torch

import cute_mma_b200 as cp
from cute_mma_b200 import _functional as F
from cute_mma_b200 import _lib
from oracle import prism_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
DEV = "cuda"
HERE = os.path.dirname(os.path.abspath(__file__))


def _inputs(M, K, N, gs, rs, dt, seed=0):
    ts = O.make_inputs(M, K, N, gs, rs, seed=seed, b_std=K ** -0.5)
    return [t.to(dt).to(DEV).contiguous() for t in ts]


@pytest.mark.parametrize("act", [None, "silu_gate"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_nan_and_inf_rows_propagate(dt, act):
    """A NaN row and an Inf row in A (forward) and in dC (backward) come back non-finite exactly
    where the oracle's are, and finite everywhere else: a diverged step must not look healthy."""
    M, K, N, gs, rs = 256, 256, 512, 256, 16
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, 31)
    A[5, :] = float("nan")
    A[77, 3] = float("inf")
    # NaN bit patterns whose upper mantissa bits are all ones (a plain add-and-truncate rounding
    # would turn these into zeros)
    A.view(torch.int16)[130, 9] = 0x7FFF
    C, _ = cp.forward(A, B, R, gs, rs, activation=act)
    rC = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, act)
    bad_rows = ~torch.isfinite(rC).all(dim=1)
    assert bad_rows[5] and bad_rows[77] and bad_rows[130]
    assert (~torch.isfinite(C)).any(dim=1)[bad_rows].all(), "a non-finite input row came back finite"
    assert torch.isfinite(C[~bad_rows]).all()
    assert O.rel_err(C[~bad_rows].float(), rC[~bad_rows]) < TOL
    # backward with clean A and poisoned dC rows
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, 32)
    dC[9, :] = float("nan")
    dC[200, 17] = float("inf")
    dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation=act)
    assert not torch.isfinite(dA[9]).any() and not torch.isfinite(dA[200]).all()
    ok_rows = torch.ones(M, dtype=torch.bool, device=DEV)
    ok_rows[9] = ok_rows[200] = False
    assert torch.isfinite(dA[ok_rows]).all()
    assert not torch.isfinite(dR).all(), "dR sums over the poisoned rows"
    if act is not None:
        assert not torch.isfinite(dB).all()
    cp.check_device_status()


def test_fp32_gradient_outputs_are_the_unrounded_sums():
    M, K, N, gs, rs = 1024, 512, 1024, 256, 8
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.bfloat16, 41)
    dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
    dA2, dR32, dB32, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate",
                                     dR_dtype=torch.float32, dB_dtype=torch.float32)
    assert dR32.dtype == torch.float32 and dB32.dtype == torch.float32 and torch.equal(dA, dA2)
    # rounding the fp32 outputs gives the 16-bit outputs bit for bit
    assert torch.equal(dR32.to(torch.bfloat16), dR) and torch.equal(dB32.to(torch.bfloat16), dB)
    rA, rR, rB = O.prism_backward(dC.float(), A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    e16, e32 = O.rel_err(dR.float(), rR), O.rel_err(dR32, rR)
    assert e32 <= e16 + 1e-6 and e32 < TOL and O.rel_err(dB32, rB) < TOL
    # split dB accumulation (second-level reduce) and the plain mode take the same path
    dB32s = F._backward_db(dC, A, R, gs, rs, 1, tile_cfg=[128, 4], out_dtype=torch.float32)
    assert O.rel_err(dB32s, rB) < TOL
    _, dRp, _, _ = cp.backward(dC, A, B, R, gs, rs, dR_dtype=torch.float32)
    assert dRp.dtype == torch.float32
    with pytest.raises(ValueError):
        cp.backward(dC, A, B, R, gs, rs, dR_dtype=torch.float64)
    cp.check_device_status()


@pytest.mark.parametrize("shape", [(1, 256), (300, 264), (4096, 2304), (8192, 14336)])
def test_bias_grad_kernel(shape):
    M, N = shape
    g = torch.Generator(device=DEV).manual_seed(M + N)
    dC = torch.randn(M, N, device=DEV, generator=g).to(torch.bfloat16)
    ref = dC.double().sum(0)
    out32 = cp.bias_grad(dC, torch.float32)
    out16 = cp.bias_grad(dC)
    assert out32.dtype == torch.float32 and out16.dtype == torch.bfloat16
    assert (out32.double() - ref).abs().max() <= 1e-5 * max(1.0, ref.abs().max().item()) * max(1, M) ** 0.5
    assert torch.equal(out32.to(torch.bfloat16), out16)
    assert torch.equal(cp.bias_grad(dC, torch.float32), out32)   # fixed summation order
    cp.check_device_status()


def test_cute_prism_import_name_and_ops():
    """A script written against the reference runs unedited: same package name, same op names."""
    import cute_prism
    M, K, N, gs, rs = 512, 256, 512, 256, 8
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.float16, 43)
    C, seeds = cute_prism.forward(A, B, R, group_size=gs, reconn_sz=rs, backend="cute", activation="silu_gate")
    assert seeds == []
    C2 = torch.ops.cute_prism.forward(A, B, R, gs, rs, "cute", "silu_gate", False, False)
    assert torch.equal(C, C2)
    dA, dR, dB = torch.ops.cute_prism.backward(dC, A, B, R, gs, rs, "cublas", "", False, False)
    assert dB.abs().max() == 0          # plain mode: frozen-B contract
    rA, rR, _ = O.prism_backward(dC.float(), A.float(), B.float(), R.float(), gs, rs, None)
    assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL
    # autograd through the reference-named op
    Ar, Br, Rr = [t.clone().requires_grad_(True) for t in (A, B, R)]
    torch.ops.cute_prism.forward(Ar, Br, Rr, gs, rs, "cute", "silu_gate", False, False).backward(dC)
    gA, gR, gB, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
    assert torch.equal(Ar.grad, gA) and torch.equal(Rr.grad, gR) and torch.equal(Br.grad, gB)
    layer = cute_prism.PrismLinear(K, N, group_size=gs, reconn_sz=rs, backend="cute", autotuning=True)
    assert float(layer.reconn_diag_sq_sum()) == pytest.approx((N // gs) * K, rel=1e-5)   # R = identity blocks
    with pytest.raises(ValueError):
        cute_prism.PrismLinear(64, 72, group_size=24, reconn_sz=8)   # 16-wide tensor-core tiles
    cp.check_device_status()


def test_workspaces_are_per_stream_and_all_are_polled():
    """Calls on two streams use different scratch buffers (they may overlap on the GPU); a backward
    run by an autograd thread uses the forward's stream, and check_device_status reads every header."""
    M, K, N, gs, rs = 512, 256, 512, 256, 8
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.float16, 47)
    ref, _ = cp.forward(A, B, R, gs, rs, activation="silu_gate")
    rA, rR, rB, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(2)]
    outs = [None, None]
    for rep in range(10):
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                outs[i] = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[0], rA) and torch.equal(o[1], rR) and torch.equal(o[2], rB)
    keys = [k for k in F._workspace._bufs if k[0] == A.device]
    assert len({k[1] for k in keys}) >= 3          # default stream + the two side streams
    # a backward issued from another host thread on the same stream shares that stream's buffer
    n_before = len(F._workspace._bufs)
    t = threading.Thread(target=lambda: cp.backward(dC, A, B, R, gs, rs, activation="silu_gate"))
    t.start(); t.join()
    assert len(F._workspace._bufs) == n_before
    # a sticky error word in ANY buffer of the device is reported and cleared
    side = F._workspace._bufs[(A.device, streams[1].cuda_stream)]
    side[:4].copy_(torch.tensor([5, 0, 0, 0], dtype=torch.uint8))
    with pytest.raises(_lib.PrismError) as ei:
        cp.check_device_status()
    assert ei.value.code == 5
    cp.check_device_status()
    C, _ = cp.forward(A, B, R, gs, rs, activation="silu_gate")
    assert torch.equal(C, ref)


def _build_wait_probe():
    src = os.path.join(HERE, "csrc", "wait_probe.cu")
    out = os.path.join(HERE, "csrc", "libwait_probe.so")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.run([os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O2",
                        "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-o", out, src], check=True)
    return ctypes.CDLL(out)


def test_bounded_wait_runs_out_and_is_reported():
    """The device-side failure path, without any fault: a wait on a barrier that nothing arrives on
    gives up after its (shortened) limit, the kernel records PRISM_ERR_DEVICE_WAIT in the workspace
    header and returns; prism_status reports code 5 and clears it; the same workspace then serves
    a normal forward."""
    probe = _build_wait_probe()
    probe.wait_probe_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    L = _lib.lib()
    M, K, N, gs, rs = 256, 256, 256, 256, 16
    A, B, R, _ = _inputs(M, K, N, gs, rs, torch.bfloat16, 53)
    need = L.prism_workspace_bytes(0, M, N, K, gs, rs, 1, None)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.prism_status(ctypes.c_void_p(ws.data_ptr()), stream) == 0
    assert probe.wait_probe_launch(ctypes.c_void_p(ws.data_ptr()), stream) == 0
    rc = L.prism_status(ctypes.c_void_p(ws.data_ptr()), stream)
    assert rc == 5, L.prism_last_error_string()
    assert b"wait ran out" in L.prism_last_error_string()
    assert L.prism_status(ctypes.c_void_p(ws.data_ptr()), stream) == 0     # cleared
    assert int(ws[:4].view(torch.int32).item()) == 0
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(L.prism_fwd(p(A), p(B), p(R), None, None, p(C), M, N, K, gs, rs, 1, 1, K, K, K, N, None,
                           p(ws), ws.numel(), stream))
    assert L.prism_status(p(ws), stream) == 0
    assert O.rel_err(C.float(), O.prism_forward(A.float(), B.float(), R.float(), gs, rs, "silu_gate")) < TOL


@pytest.mark.parametrize("shape", [
    (1, 256, 256, 256, 16), (7, 200, 384, 128, 8), (16, 512, 512, 256, 16), (17, 320, 256, 128, 32),
    (100, 576, 512, 256, 64), (128, 1024, 1024, 256, 16), (64, 256, 1024, 512, 16), (128, 4096, 1792, 256, 16),
], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("act", [None, "silu_gate"])
def test_few_token_streaming_forward(shape, act):
    """The streaming kernel that serves M <= 128 (B tiles as the M dimension of the MMA, K shared by
    several CTAs, partial sums added in a fixed order): against the oracle, against the general
    kernel, with a bias, and bit-identical over repeats."""
    M, K, N, gs, rs = shape
    dt = torch.bfloat16 if (M + rs) % 3 else torch.float16
    A, B, R, _ = _inputs(M, K, N, gs, rs, dt, seed=M + K)
    bias = (torch.randn(N, device=DEV) * 0.5).to(dt)
    ref = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, act, bias=bias.float())
    C, _ = cp.forward(A, B, R, gs, rs, activation=act, bias=bias, tile_cfg=[0, 0, 0, 2])   # streaming kernel, forced
    Cg, _ = cp.forward(A, B, R, gs, rs, activation=act, bias=bias, tile_cfg=[0, 0, 0, 1])  # general kernel
    Cd, _ = cp.forward(A, B, R, gs, rs, activation=act, bias=bias)                         # default choice
    cp.check_device_status()
    assert torch.isfinite(C).all()
    assert O.rel_err(C.float(), ref) < TOL and O.rel_err(Cg.float(), ref) < TOL
    assert torch.equal(Cd, C if M <= 48 else Cg), "up to 48 tokens the streaming kernel is the default"
    for _ in range(5):
        C2, _ = cp.forward(A, B, R, gs, rs, activation=act, bias=bias, tile_cfg=[0, 0, 0, 2])
        assert torch.equal(C2, C)
    cp.check_device_status()


def test_few_token_kernel_is_refused_where_it_does_not_apply():
    A, B, R, _ = _inputs(200, 256, 256, 256, 16, torch.bfloat16)
    with pytest.raises(_lib.PrismError):
        cp.forward(A, B, R, 256, 16, tile_cfg=[0, 0, 0, 2])           # more than 128 tokens
    A, B, R, _ = _inputs(16, 256, 192, 64, 16, torch.bfloat16)
    C, _ = cp.forward(A, B, R, 64, 16)                                # group size 64: general kernel
    assert O.rel_err(C.float(), O.prism_forward(A.float(), B.float(), R.float(), 64, 16, None)) < TOL


@pytest.mark.parametrize("shape", [(64, 256, 512, 256, 8), (200, 512, 768, 128, 16), (33, 256, 256, 64, 32), (128, 128, 128, 32, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_rw_mode_weight_folding(shape):
    """mode='rw' (the reference's inference form): the folded weight gives the plain-mode forward."""
    M, K, N, gs, rs = shape
    dt = torch.bfloat16 if rs != 8 else torch.float16
    A, B, R, _ = _inputs(M, K, N, gs, rs, dt, seed=61)
    Bp = cp.fold_weight(B, R, gs, rs)
    G, nb = N // gs, K // rs
    Rb = R.float().reshape(G, rs, nb, rs).permute(0, 2, 1, 3)                       # (G, nb, i, j)
    ref_Bp = torch.einsum("gnbi,gbij->gnbj", B.float().reshape(G, gs, nb, rs), Rb).reshape(N, K)
    assert O.rel_err(Bp.float(), ref_Bp) < 1e-2
    C_rw, seeds = cp.forward(A, B, R, gs, rs, mode="rw")
    C_ar, _ = cp.forward(A, B, R, gs, rs, mode="ar")
    ref = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, None)
    assert seeds == [] and O.rel_err(C_rw.float(), ref) < TOL and O.rel_err(C_ar.float(), ref) < TOL
    cp.check_device_status()


@pytest.mark.parametrize("rs", [8, 16])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_cayley_kernel_matches_linalg_solve(rs, dt):
    """The batched Cayley kernel against the reference's construction (torch.linalg.solve per block,
    src/cute_prism/_module.py:534-577), values and gradient; R is orthogonal."""
    G, K = 5, 12 * rs
    nb = K // rs
    torch.manual_seed(rs)
    M = (torch.randn(G * rs, K, device=DEV) * 0.3).to(dt).requires_grad_(True)
    R = torch.ops.prism_b200.cayley(M, rs)
    Mb = M.detach().float().reshape(G, rs, nb, rs).permute(0, 2, 1, 3).requires_grad_(True)
    S = Mb - Mb.transpose(-1, -2)
    eye = torch.eye(rs, device=DEV).expand_as(S)
    Rb = torch.linalg.solve(eye - S, eye + S)
    R_ref = Rb.permute(0, 2, 1, 3).reshape(G * rs, K)
    tol = 1e-4 if dt == torch.float32 else 1e-2
    assert O.rel_err(R.float(), R_ref) < tol
    Rk = R.detach().float().reshape(G, rs, nb, rs).permute(0, 2, 1, 3)
    if dt == torch.float32:
        assert (Rk @ Rk.transpose(-1, -2) - torch.eye(rs, device=DEV)).abs().max() < 1e-4
    W = torch.randn_like(R_ref)
    (R.float() * W).sum().backward()
    (R_ref * W).sum().backward()
    dM_ref = Mb.grad.permute(0, 2, 1, 3).reshape(G * rs, K)
    assert O.rel_err(M.grad.float(), dM_ref) < (1e-4 if dt == torch.float32 else 2e-2)


def test_library_calls_can_be_captured_in_a_cuda_graph():
    """Forward, backward, bias gradient and the Cayley construction replayed from a CUDA graph give
    the eager results (every call is stream-ordered, no host synchronisation, no allocation)."""
    M, K, N, gs, rs = 512, 256, 512, 256, 8
    layer = cp.PrismLinear(K, N, group_size=gs, reconn_sz=rs).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        layer.reconn.normal_(std=0.1)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)

    def fb():
        layer.zero_grad(set_to_none=False)
        if x.grad is not None:
            x.grad.zero_()
        y = layer(x)
        y.backward(dy)
        return y

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            y_eager = fb().detach().clone()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    gx, gr, gb = x.grad.clone(), layer.reconn.grad.clone(), layer.bias.grad.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y_static = fb()
    x.grad.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_static, y_eager) and torch.equal(x.grad, gx)
    assert torch.equal(layer.reconn.grad, gr) and torch.equal(layer.bias.grad, gb)
    cp.check_device_status()


@pytest.mark.parametrize("shape", [(1024, 256, 1024, 256, 8), (300, 208, 256, 128, 16), (2048, 512, 512, 256, 16),
                                   (16, 256, 512, 256, 16), (512, 512, 256, 64, 32)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("act", ["silu_gate", "sigmoid_gate"])
def test_internal_bias_forward_and_backward(shape, act):
    """S = A . blockdiag(R_g)^T + internal_bias[g] before the gate; d_internal_bias = sum over tokens of dS
    (reference: src/cute_prism/_pytorch_backend.py:154-156, 271-272), bit-stable like dR."""
    M, K, N, gs, rs = shape
    dt = torch.bfloat16 if rs != 8 else torch.float16
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, seed=71)
    ib = (torch.randn(N // gs, K, device=DEV) * 0.5).to(dt)
    C, _ = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib)
    dA, dR, dB, d_ib = cp.backward(dC, A, B, R, gs, rs, activation=act, internal_bias=ib)
    cp.check_device_status()
    Af, Bf, Rf, ibf = A.float(), B.float(), R.float(), ib.float()
    rC = O.prism_forward(Af, Bf, Rf, gs, rs, act, internal_bias=ibf)
    rA, rR, rB, r_ib = O.prism_backward(dC.float(), Af, Bf, Rf, gs, rs, act, internal_bias=ibf)
    for name, val, ref in (("C", C, rC), ("dA", dA, rA), ("dR", dR, rR), ("dB", dB, rB), ("d_ib", d_ib, r_ib)):
        assert torch.isfinite(val).all(), name
        assert O.rel_err(val.float(), ref) < TOL, (name, O.rel_err(val.float(), ref))
    # the bias really takes part: without it the forward differs
    C0, _ = cp.forward(A, B, R, gs, rs, activation=act)
    assert O.rel_err(C0.float(), rC) > 5e-2
    for _ in range(3):
        dA2, dR2, dB2, d_ib2 = cp.backward(dC, A, B, R, gs, rs, activation=act, internal_bias=ib)
        assert torch.equal(d_ib2, d_ib) and torch.equal(dR2, dR) and torch.equal(dA2, dA)
    with pytest.raises(ValueError):
        cp.forward(A, B, R, gs, rs, internal_bias=ib)   # plain mode


def test_prism_linear_with_internal_bias_trains():
    torch.manual_seed(3)
    layer = cp.PrismLinear(256, 512, group_size=256, reconn_sz=16, activation="silu_gate", internal_bias=True)
    layer = layer.to(DEV).to(torch.bfloat16)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    A = x.detach().reshape(-1, 256)
    s = layer._bwd_scale
    rA, rR, rB, r_ib = O.prism_backward(dy.reshape(-1, 512).float() * s, A.float(), layer.weight.detach().float(),
                                        layer.reconn.detach().float(), 256, 16, "silu_gate",
                                        internal_bias=layer._internal_bias.detach().float())
    assert O.rel_err(layer._internal_bias.grad.float(), r_ib) < TOL
    assert O.rel_err(x.grad.reshape(-1, 256).float(), rA) < TOL and O.rel_err(layer.weight.grad.float(), rB) < TOL
    cp.check_device_status()


@pytest.mark.parametrize("shape", [(1024, 256, 1024, 256, 8), (300, 208, 256, 128, 16), (24, 512, 512, 256, 16),
                                   (2048, 512, 768, 256, 16)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("act", ["silu_gate", "sigmoid_gate"])
def test_hash_dropout_forward_and_backward(shape, act):
    """Training-mode dropout of the gated activation: the kernels' mask is the reference kernels' hash mask
    (regenerated in both backward kernels from the per-group seeds); checked against the oracle with the
    same seeds, together with an internal bias."""
    M, K, N, gs, rs = shape
    dt = torch.bfloat16 if rs != 8 else torch.float16
    p = 0.25
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, seed=83)
    ib = (torch.randn(N // gs, K, device=DEV) * 0.5).to(dt)
    C, seeds = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib, dropout_p=p, training=True)
    assert len(seeds) == 1 and seeds[0].dtype == torch.int64 and seeds[0].shape == (N // gs,)
    dA, dR, dB, d_ib = cp.backward(dC, A, B, R, gs, rs, activation=act, internal_bias=ib, dropout_seeds=seeds,
                                   dropout_p=p)
    cp.check_device_status()
    Af, Bf, Rf, ibf = A.float(), B.float(), R.float(), ib.float()
    sl = seeds[0].tolist()
    rC = O.prism_forward(Af, Bf, Rf, gs, rs, act, internal_bias=ibf, dropout_seeds=sl, dropout_p=p)
    rA, rR, rB, r_ib = O.prism_backward(dC.float(), Af, Bf, Rf, gs, rs, act, internal_bias=ibf, dropout_seeds=sl,
                                        dropout_p=p)
    for name, val, ref in (("C", C, rC), ("dA", dA, rA), ("dR", dR, rR), ("dB", dB, rB), ("d_ib", d_ib, r_ib)):
        assert torch.isfinite(val).all(), name
        assert O.rel_err(val.float(), ref) < TOL, (name, O.rel_err(val.float(), ref))
    # same seeds, same result; eval mode (training=False) is the plain gated forward
    C2, _ = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib, dropout_p=p, training=True,
                       dropout_seeds=seeds[0])
    assert torch.equal(C2, C)
    Ce, se = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib, dropout_p=p, training=False)
    assert se == [] and O.rel_err(Ce.float(), O.prism_forward(Af, Bf, Rf, gs, rs, act, internal_bias=ibf)) < TOL
    assert O.rel_err(Ce.float(), rC) > 5e-2      # the mask really changed the result


def test_prism_linear_dropout_train_and_eval():
    torch.manual_seed(5)
    layer = cp.PrismLinear(256, 512, group_size=256, reconn_sz=16, activation="silu_gate", dropout=0.5)
    layer = layer.to(DEV).to(torch.bfloat16)
    x = torch.randn(256, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    layer.eval()
    y_eval = layer(x)
    layer.train()
    y1, y2 = layer(x), layer(x)
    assert not torch.equal(y1, y2) and not torch.equal(y1, y_eval)       # fresh seeds per call
    y1.float().pow(2).mean().backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(layer.reconn.grad).all()
    # expectation over masks is the eval output: the mean over many draws approaches it
    acc = torch.zeros_like(y_eval, dtype=torch.float32)
    with torch.no_grad():
        for _ in range(64):
            acc += layer(x).float()
    assert O.rel_err(acc / 64, y_eval.float()) < 0.35
    cp.check_device_status()


@pytest.mark.parametrize("shape", [(512, 256, 512, 256), (300, 192, 384, 128), (16, 512, 1024, 256), (2048, 1024, 768, 256)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("act", [None, "silu_gate", "sigmoid_gate"])
def test_input_shuffle_forward_and_backward(shape, act):
    """Every group sees its own butterfly permutation of the input features (reference:
    src/cute_prism/_module.py:236-270, _pytorch_backend.py:31-76): served by the 64-wide rotation of the same
    kernels on folded parameters, checked against the oracle's per-group gather, with an internal bias."""
    from cute_mma_b200 import _shuffle as S
    M, K, N, gs = shape
    rs = 16
    dt = torch.bfloat16 if M % 32 == 0 else torch.float16
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, seed=91)
    masks, _ = S.build_shuffle_masks(K, N, gs, rs)
    masks = masks.to(DEV)
    ib = (torch.randn(N // gs, K, device=DEV) * 0.5).to(dt) if act else None
    C, seeds = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib, shuffle_masks=masks)
    dA, dR, dB, d_ib = cp.backward(dC, A, B, R, gs, rs, activation=act, internal_bias=ib, shuffle_masks=masks)
    cp.check_device_status()
    assert seeds == [] and dR.shape == R.shape and dR.dtype == dt
    Af, Bf, Rf = A.float(), B.float(), R.float()
    ibf = None if ib is None else ib.float()
    rC = O.prism_forward(Af, Bf, Rf, gs, rs, act, internal_bias=ibf, shuffle_masks=masks)
    ref = O.prism_backward(dC.float(), Af, Bf, Rf, gs, rs, act, internal_bias=ibf, shuffle_masks=masks)
    pairs = [("C", C, rC), ("dA", dA, ref[0]), ("dR", dR, ref[1])]
    if act:
        pairs += [("dB", dB, ref[2]), ("d_ib", d_ib, ref[3])]
    else:
        assert dB is None and d_ib is None
    for name, val, r in pairs:
        assert torch.isfinite(val).all(), name
        assert O.rel_err(val.float(), r) < TOL, (name, O.rel_err(val.float(), r))
    # without the masks the result is another one (groups 1.. are permuted)
    C0, _ = cp.forward(A, B, R, gs, rs, activation=act, internal_bias=ib)
    assert O.rel_err(C0.float(), rC) > 5e-2
    with pytest.raises(ValueError):
        cp.forward(A, B, R, gs, rs, activation="silu_gate", shuffle_masks=masks, dropout_p=0.1, training=True)


def test_prism_linear_input_shuffle_trains():
    """PrismLinear(input_shuffle=True): forward and all parameter gradients through autograd (the fold is made
    of differentiable index operations) against the oracle with the module's own masks."""
    torch.manual_seed(3)
    K, N, gs, rs, M = 256, 512, 128, 16, 192
    layer = cp.PrismLinear(K, N, group_size=gs, reconn_sz=rs, activation="silu_gate", input_shuffle=True,
                           internal_bias=True).to(DEV, torch.bfloat16)
    with torch.no_grad():
        layer._internal_bias.normal_(0, 0.3)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    cp.check_device_status()
    R = layer._build_R().detach().float()
    W, ib, bias = layer.weight.detach().float(), layer._internal_bias.detach().float(), layer.bias.detach().float()
    masks = layer._shuffle_masks
    rC = O.prism_forward(x.detach().float(), W, R, gs, rs, "silu_gate", bias=bias, internal_bias=ib, shuffle_masks=masks)
    scale = float(layer._bwd_scale)
    rA, rR, rB, r_ib = O.prism_backward(dy.float() * scale, x.detach().float(), W, R, gs, rs, "silu_gate",
                                        internal_bias=ib, shuffle_masks=masks)
    assert O.rel_err(y.float(), rC) < TOL
    assert O.rel_err(x.grad.float(), rA) < TOL
    assert O.rel_err(layer.weight.grad.float(), rB) < TOL
    assert O.rel_err(layer._internal_bias.grad.float(), r_ib) < TOL
    assert layer.reconn.grad is not None and torch.isfinite(layer.reconn.grad).all() and layer.reconn.grad.abs().sum() > 0
