"""Parity of the sm_100a kernels (called through the C ABI) with the oracle.

Metric and bar: the reference's own ``max|x - ref| / (max|ref| + 1e-6)`` (tests/test_correctness.py:24-31)
must stay below TOL = 2e-2 for fp16 and bf16 outputs with fp32 accumulation; the oracle is evaluated
in fp32 on the same 16-bit-rounded inputs."""
import glob
import os

import numpy as np
import pytest
import torch

import cute_mma_b200 as cp
from cute_mma_b200 import _functional as F
from oracle import prism_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEV = "cuda"


def _inputs(M, K, N, gs, rs, dt, seed=0, b_std=None, dc_std=1.0, r_kind="orthogonal"):
    b_std = K ** -0.5 if b_std is None else b_std
    ts = O.make_inputs(M, K, N, gs, rs, seed=seed, b_std=b_std, dc_std=dc_std, r_kind=r_kind)
    return [t.to(dt).to(DEV).contiguous() for t in ts]


def _check_all(M, K, N, gs, rs, dt, act, seed=0, **kw):
    A, B, R, dC = _inputs(M, K, N, gs, rs, dt, seed, **kw)
    C, seeds = cp.forward(A, B, R, gs, rs, activation=act)
    dA, dR, dB, dib = cp.backward(dC, A, B, R, gs, rs, activation=act)
    cp.check_device_status()
    assert seeds == [] and dib is None
    Af, Bf, Rf, dCf = A.float(), B.float(), R.float(), dC.float()
    rC = O.prism_forward(Af, Bf, Rf, gs, rs, act)
    rA, rR, rB = O.prism_backward(dCf, Af, Bf, Rf, gs, rs, act)
    for name, val, ref in (("C", C, rC), ("dA", dA, rA), ("dR", dR, rR)):
        assert val.dtype == dt and val.shape == ref.shape
        assert torch.isfinite(val).all(), name
        assert O.rel_err(val.float(), ref) < TOL, name
    if act is None:
        assert dB is None
    else:
        assert torch.isfinite(dB).all() and O.rel_err(dB.float(), rB) < TOL


@pytest.mark.parametrize("act", [None, "silu_gate", "sigmoid_gate"])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_config1_all_modes(dt, act, seed):
    """M=1024, K=256, N=1024, gs=256, rs=8 (benchmark configurations 0/1)."""
    _check_all(1024, 256, 1024, 256, 8, dt, act, seed)


@pytest.mark.parametrize("shape", [
    (1, 256, 256, 256, 16),      # a single token
    (100, 64, 256, 256, 16),     # ragged M, one K chunk
    (300, 200, 96, 32, 8),       # ragged M and K, small groups
    (257, 136, 192, 64, 8),      # K = 8 * odd
    (640, 320, 192, 96, 16),     # group size that is not a power of two
    (512, 512, 512, 128, 32),    # 32-wide rotation blocks
    (512, 512, 256, 64, 64),     # 64-wide rotation blocks
    (256, 256, 512, 512, 16),    # group wider than one tile
    (2048, 1024, 1024, 256, 8),  # several tiles per CTA
], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("act", [None, "silu_gate", "sigmoid_gate"])
def test_shapes(shape, act):
    M, K, N, gs, rs = shape
    _check_all(M, K, N, gs, rs, torch.bfloat16 if rs != 8 else torch.float16, act, seed=4)


def test_gaussian_R_and_unit_variance_inputs():
    """The reference's GPU tests draw A, B, R, dC ~ N(0,1) (tests/test_correctness.py:139-145)."""
    _check_all(512, 256, 512, 256, 8, torch.float16, None, seed=7, b_std=1.0, r_kind="gaussian")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "small_*.npz"))), ids=os.path.basename)
def test_golden_vectors(path):
    """Kernels on the golden inputs (rounded to bf16) against the reference's own outputs."""
    z = np.load(path)
    M, K, N, gs, rs = [int(v) for v in z["meta"]]
    if gs % 16 != 0:
        pytest.skip("group size below the tensor-core tile")
    A, B, R, dC = [torch.from_numpy(z[k]).to(torch.bfloat16).to(DEV).contiguous() for k in ("A", "B", "R", "dC")]
    for act, tag in ((None, "plain"), ("silu_gate", "gated"), ("sigmoid_gate", "sgate")):
        C, _ = cp.forward(A, B, R, gs, rs, activation=act)
        dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation=act)
        ref = {k: torch.from_numpy(z[f"{k}_{tag}"]).to(DEV) for k in ("C", "dA", "dR")}
        assert O.rel_err(C.float(), ref["C"]) < TOL
        assert O.rel_err(dA.float(), ref["dA"]) < TOL
        assert O.rel_err(dR.float(), ref["dR"]) < TOL
        if act is not None:
            assert O.rel_err(dB.float(), torch.from_numpy(z[f"dB_{tag}"]).to(DEV)) < TOL
    cp.check_device_status()


def test_structural_known_answers():
    M, K, N, gs, rs = 256, 128, 256, 128, 16
    A, B, _, _ = _inputs(M, K, N, gs, rs, torch.float16, 3)
    eye = torch.eye(rs, device=DEV, dtype=torch.float16).repeat(N // gs, K // rs)
    C, _ = cp.forward(A, B, eye, gs, rs)
    assert O.rel_err(C.float(), A.float() @ B.float().T) < 2e-3   # identity rotation = dense linear layer
    Cz, _ = cp.forward(A, B, torch.zeros_like(eye), gs, rs, activation="silu_gate")
    assert Cz.abs().max().item() == 0.0                          # gate of zero is zero


def test_empty_batch():
    A, B, R, dC = _inputs(0, 64, 64, 32, 8, torch.float16)
    C, _ = cp.forward(A, B, R, 32, 8, activation="silu_gate")
    assert C.shape == (0, 64)
    dA, dR, dB, _ = cp.backward(dC, A, B, R, 32, 8, activation="silu_gate")
    assert dA.shape == (0, 64) and dR.abs().max() == 0 and dB.abs().max() == 0


def test_fused_bias_and_dc_scale():
    M, K, N, gs, rs = 384, 256, 512, 256, 16
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.bfloat16, 5)
    bias = (torch.randn(N, device=DEV) * 0.5).to(torch.bfloat16)
    C, _ = cp.forward(A, B, R, gs, rs, activation="silu_gate", bias=bias)
    ref = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, "silu_gate", bias=bias.float())
    assert O.rel_err(C.float(), ref) < TOL
    s = 1 / 1.437
    dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate", dc_scale=s)
    rA, rR, rB = O.prism_backward(dC.float() * s, A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL and O.rel_err(dB.float(), rB) < TOL


@pytest.mark.parametrize("act", [None, "silu_gate"])
def test_bit_stable_run_to_run(act):
    """Forward and every gradient are bit-identical across repeated calls, at a size where a CTA
    accumulates dR over many token tiles (the reference is only deterministic for <= 8 tiles,
    tests/test_cute_determinism.py:43-50 and cute_prism_backward_dadr.cu:675-682)."""
    M, K, N, gs, rs = 8192, 512, 1024, 256, 8
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.float16, 9)
    first = None
    for _ in range(5):
        C, _ = cp.forward(A, B, R, gs, rs, activation=act)
        dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation=act)
        cur = [C, dA, dR] + ([dB] if dB is not None else [])
        if first is None:
            first = cur
        else:
            for a, b in zip(first, cur):
                assert torch.equal(a, b)
    cp.check_device_status()


def test_full_size_properties_config2():
    """Benchmark configuration 2 (K=4096, N=14336, gs=256, rs=16, bf16, silu_gate) at M=2048:
    size-independent properties plus an oracle check evaluated on the GPU in fp32."""
    M, K, N, gs, rs, act = 2048, 4096, 14336, 256, 16, "silu_gate"
    dt = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    A = torch.randn(M, K, device=DEV, generator=g).to(dt)
    B = (torch.randn(N, K, device=DEV, generator=g) * K ** -0.5).to(dt)
    R = O.orthogonal_R(N // gs, K, rs, torch.Generator().manual_seed(0)).to(dt).to(DEV)
    dC = torch.randn(M, N, device=DEV, generator=g).to(dt)
    C, _ = cp.forward(A, B, R, gs, rs, activation=act)
    dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation=act)
    # (1) rows are independent: a slice of the batch gives bit-identical rows
    C2, _ = cp.forward(A[640:1000].contiguous(), B, R, gs, rs, activation=act)
    assert torch.equal(C2, C[640:1000])
    # (2) the backward is linear in dC: scaling dC by 2 scales every gradient by exactly 2
    dA2, dR2, dB2, _ = cp.backward((dC * 2).contiguous(), A, B, R, gs, rs, activation=act)
    assert torch.equal(dA2, dA * 2) and torch.equal(dR2, dR * 2) and torch.equal(dB2, dB * 2)
    # (3) parameter gradients add over token shards (what data parallelism relies on)
    h = M // 2
    _, dRa, dBa, _ = cp.backward(dC[:h].contiguous(), A[:h].contiguous(), B, R, gs, rs, activation=act)
    _, dRb, dBb, _ = cp.backward(dC[h:].contiguous(), A[h:].contiguous(), B, R, gs, rs, activation=act)
    assert O.rel_err(dRa.float() + dRb.float(), dR.float()) < TOL
    assert O.rel_err(dBa.float() + dBb.float(), dB.float()) < TOL
    # (4) oracle on the same inputs, fp32 on the GPU
    Af, Bf, Rf, dCf = A.float(), B.float(), R.float(), dC.float()
    assert O.rel_err(C.float(), O.prism_forward(Af, Bf, Rf, gs, rs, act)) < TOL
    rA, rR, rB = O.prism_backward(dCf, Af, Bf, Rf, gs, rs, act)
    assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL and O.rel_err(dB.float(), rB) < TOL
    cp.check_device_status()


def test_small_m_decode_shapes_config2():
    """Configuration 2, forward only, M in {1, 16, 128}."""
    K, N, gs, rs, act = 4096, 14336, 256, 16, "silu_gate"
    dt = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(1)
    B = (torch.randn(N, K, device=DEV, generator=g) * K ** -0.5).to(dt)
    R = O.orthogonal_R(N // gs, K, rs, torch.Generator().manual_seed(1)).to(dt).to(DEV)
    for M in (1, 16, 128):
        A = torch.randn(M, K, device=DEV, generator=g).to(dt)
        C, _ = cp.forward(A, B, R, gs, rs, activation=act)
        assert O.rel_err(C.float(), O.prism_forward(A.float(), B.float(), R.float(), gs, rs, act)) < TOL


def test_config3_slice_fp16():
    """Configuration 3 shapes (K=1024, N=16384, gs=256, rs=8, fp16, silu_gate, dC std 0.1) on the
    per-GPU token slice of an 8-way split (M=8192)."""
    M, K, N, gs, rs, act = 8192, 1024, 16384, 256, 8, "silu_gate"
    dt = torch.float16
    g = torch.Generator(device=DEV).manual_seed(2)
    A = torch.randn(M, K, device=DEV, generator=g).to(dt)
    B = (torch.randn(N, K, device=DEV, generator=g) * K ** -0.5).to(dt)
    R = O.orthogonal_R(N // gs, K, rs, torch.Generator().manual_seed(2)).to(dt).to(DEV)
    dC = (torch.randn(M, N, device=DEV, generator=g) * 0.1).to(dt)
    C, _ = cp.forward(A, B, R, gs, rs, activation=act)
    dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation=act)
    Af, Bf, Rf, dCf = A.float(), B.float(), R.float(), dC.float()
    assert O.rel_err(C.float(), O.prism_forward(Af, Bf, Rf, gs, rs, act)) < TOL
    rA, rR, rB = O.prism_backward(dCf, Af, Bf, Rf, gs, rs, act)
    assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL and O.rel_err(dB.float(), rB) < TOL
    cp.check_device_status()


def test_repeat_stress_gated_backward():
    """The reference's race detector (KNOWN_ISSUES.md:43-56): many repeats of the gated backward
    must all agree with the first result (here: bit-exactly)."""
    M, K, N, gs, rs = 1024, 512, 512, 256, 8
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.float16, 13)
    dA0, dR0, dB0, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
    for _ in range(100):
        dA, dR, dB, _ = cp.backward(dC, A, B, R, gs, rs, activation="silu_gate")
        assert torch.equal(dA, dA0) and torch.equal(dR, dR0) and torch.equal(dB, dB0)
    cp.check_device_status()


def test_tile_configurations_agree():
    M, K, N, gs, rs = 1024, 512, 1024, 256, 16
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.bfloat16, 17)
    ref = O.prism_forward(A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    for cfg in ([256, 16, 0, 0], [128, 4, 0, 0], [64, 2, 0, 0], [32, 1, 4, 0]):
        C, _ = cp.forward(A, B, R, gs, rs, activation="silu_gate", tile_cfg=cfg)
        assert O.rel_err(C.float(), ref) < TOL, cfg
    rA, rR, rB = O.prism_backward(dC.float(), A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    # {main CTA pairs per feature column, token tiles left to extra pairs (-1: none), extra pairs}
    for cfg in ([1, -1], [2, -1], [8, -1], [1, 1, 3], [1, 2, 1], [2, 1, 0], [1, 3, 4]):
        dA, dR = F._backward_dadr(dC, A, B, R, gs, rs, 1, tile_cfg=cfg)
        assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL, cfg
    for cfg in ([256, 1], [128, 2], [64, 8]):
        dB = F._backward_db(dC, A, R, gs, rs, 1, tile_cfg=cfg)
        assert O.rel_err(dB.float(), rB) < TOL, cfg
    cp.check_device_status()


def test_db_last_wave_split_and_dadr_extra_pairs():
    """Launch plans that only large problems pick by themselves, forced at a small size: the dB kernel
    gives the n-tile rows of a mostly empty last wave to a second launch with a split token range
    (80 tiles of 64 outputs on 74 SM pairs here), the dA+dR kernel lets extra CTA pairs take over the
    main pairs' last tiles.  Results must match the oracle and repeat bit-exactly."""
    M, K, N, gs, rs = 512, 512, 2560, 128, 16
    A, B, R, dC = _inputs(M, K, N, gs, rs, torch.bfloat16, 23)
    rA, rR, rB = O.prism_backward(dC.float(), A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    outs = []
    for cfg in ([64, 0], [64, -1], [64, 0]):
        dB = F._backward_db(dC, A, R, gs, rs, 1, tile_cfg=cfg)
        assert O.rel_err(dB.float(), rB) < TOL, cfg
        outs.append(dB)
    assert torch.equal(outs[0], outs[2])
    M2 = 2048
    A, B, R, dC = _inputs(M2, K, N, gs, rs, torch.bfloat16, 29)
    rA, rR, rB = O.prism_backward(dC.float(), A.float(), B.float(), R.float(), gs, rs, "silu_gate")
    outs = []
    for cfg in ([1, 3, 2], [2, 1, 3], [1, 3, 2]):
        dA, dR = F._backward_dadr(dC, A, B, R, gs, rs, 1, tile_cfg=cfg)
        assert O.rel_err(dA.float(), rA) < TOL and O.rel_err(dR.float(), rR) < TOL, cfg
        outs.append((dA, dR))
    assert torch.equal(outs[0][0], outs[2][0]) and torch.equal(outs[0][1], outs[2][1])
    cp.check_device_status()
