"""The oracle (oracle/prism_oracle.py) against the reference's own outputs (golden vectors made
by tests/golden/make_golden.py from the reference package), against torch autograd in float64
(the reference's own self-check, tests/test_pytorch_backend.py:184-239) and against the
structural known answers the reference relies on."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import prism_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "small_*.npz"))), ids=os.path.basename)
def test_oracle_matches_reference_small(path):
    z = np.load(path)
    M, K, N, gs, rs = [int(v) for v in z["meta"]]
    A, B, R, dC = _t(z["A"]), _t(z["B"]), _t(z["R"]), _t(z["dC"])
    tol = 1e-12 if A.dtype == torch.float64 else 2e-5
    for act, tag in ((None, "plain"), ("silu_gate", "gated"), ("sigmoid_gate", "sgate")):
        C = O.prism_forward(A, B, R, gs, rs, act)
        dA, dR, dB = O.prism_backward(dC, A, B, R, gs, rs, act)
        assert O.rel_err(C, _t(z[f"C_{tag}"])) < tol
        assert O.rel_err(dA, _t(z[f"dA_{tag}"])) < tol
        assert O.rel_err(dR, _t(z[f"dR_{tag}"])) < tol
        if act is None:
            assert dB is None and f"dB_{tag}" not in z.files
        else:
            assert O.rel_err(dB, _t(z[f"dB_{tag}"])) < tol


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "small_*.npz"))), ids=os.path.basename)
def test_oracle_matches_reference_internal_bias(path):
    z = np.load(path)
    M, K, N, gs, rs = [int(v) for v in z["meta"]]
    A, B, R, dC, ib = _t(z["A"]), _t(z["B"]), _t(z["R"]), _t(z["dC"]), _t(z["ib"])
    tol = 1e-12 if A.dtype == torch.float64 else 2e-5
    C = O.prism_forward(A, B, R, gs, rs, "silu_gate", internal_bias=ib)
    dA, dR, dB, d_ib = O.prism_backward(dC, A, B, R, gs, rs, "silu_gate", internal_bias=ib)
    for val, key in ((C, "C_ib"), (dA, "dA_ib"), (dR, "dR_ib"), (dB, "dB_ib"), (d_ib, "dib_ib")):
        assert O.rel_err(val, _t(z[key])) < tol, key


def test_oracle_matches_reference_input_shuffle():
    """Input shuffle: the reference's masks and its outputs (tests/golden/shuffle_a.npz); the masks are
    also what the package's own mask builder produces."""
    from cute_mma_b200 import _shuffle as S
    z = np.load(os.path.join(GOLD, "shuffle_a.npz"))
    M, K, N, gs, rs = [int(v) for v in z["meta"]]
    A, B, R, dC, ib, masks = (_t(z[k]) for k in ("A", "B", "R", "dC", "ib", "masks"))
    mine, deltas = S.build_shuffle_masks(K, N, gs, rs, 64)
    assert torch.equal(mine, masks) and deltas == [int(v) for v in z["deltas"]]
    assert int(masks[0].abs().sum()) == 0 and int(masks[1:].abs().sum()) > 0
    for act, tag in ((None, "plain"), ("silu_gate", "gated"), ("sigmoid_gate", "sgate")):
        ibx = ib if act else None
        C = O.prism_forward(A, B, R, gs, rs, act, internal_bias=ibx, shuffle_masks=masks)
        grads = O.prism_backward(dC, A, B, R, gs, rs, act, internal_bias=ibx, shuffle_masks=masks)
        assert O.rel_err(C, _t(z[f"C_{tag}"])) < 1e-12
        assert O.rel_err(grads[0], _t(z[f"dA_{tag}"])) < 1e-12
        assert O.rel_err(grads[1], _t(z[f"dR_{tag}"])) < 1e-12
        if act:
            assert O.rel_err(grads[2], _t(z[f"dB_{tag}"])) < 1e-12
            assert O.rel_err(grads[3], _t(z[f"dib_{tag}"])) < 1e-12
        # the shuffle really changes the result
        assert O.rel_err(O.prism_forward(A, B, R, gs, rs, act, internal_bias=ibx), _t(z[f"C_{tag}"])) > 1e-2


@pytest.mark.parametrize("seed", [0, 1])
def test_oracle_matches_reference_config0(seed):
    z = np.load(os.path.join(GOLD, f"config0_seed{seed}.npz"))
    M, K, N, gs, rs, s = [int(v) for v in z["meta"]]
    assert s == seed
    A, B, R, dC = O.make_inputs(M, K, N, gs, rs, seed=seed)
    chk = np.array([A.double().sum().item(), B.double().sum().item(), R.double().sum().item(),
                    dC.double().sum().item()])
    np.testing.assert_allclose(chk, z["input_checksum"], rtol=1e-9, atol=1e-9)
    for act, tag in ((None, "plain"), ("silu_gate", "gated"), ("sigmoid_gate", "sgate")):
        C = O.prism_forward(A, B, R, gs, rs, act)
        dA, dR, dB = O.prism_backward(dC, A, B, R, gs, rs, act)
        assert O.rel_err(C[::16, ::16], _t(z[f"C_{tag}"])) < 2e-5
        assert O.rel_err(dA[::16, ::4], _t(z[f"dA_{tag}"])) < 2e-5
        assert O.rel_err(dR, _t(z[f"dR_{tag}"])) < 2e-5
        if act is not None:
            assert O.rel_err(dB[::16, ::4], _t(z[f"dB_{tag}"])) < 2e-5


@pytest.mark.parametrize("act", [None, "silu_gate", "sigmoid_gate"])
@pytest.mark.parametrize("rs", [8, 16])
def test_oracle_backward_matches_autograd_fp64(act, rs):
    M, K, N, gs = 32, 128, 128, 32
    A, B, R, dC = [t.double() for t in O.make_inputs(M, K, N, gs, rs, seed=3, r_kind="gaussian")]
    A.requires_grad_(True); B.requires_grad_(True); R.requires_grad_(True)
    C = O.prism_forward(A, B, R, gs, rs, act)
    C.backward(dC)
    dA, dR, dB = O.prism_backward(dC, A.detach(), B.detach(), R.detach(), gs, rs, act)
    # only the entries of R inside the diagonal blocks take part; compare those
    assert (dA - A.grad).abs().max() < 1e-9
    assert (dR - R.grad).abs().max() < 1e-9
    if act is not None:
        assert (dB - B.grad).abs().max() < 1e-9


def test_known_answers():
    M, K, N, gs, rs = 16, 64, 64, 32, 8
    A, B, _, _ = O.make_inputs(M, K, N, gs, rs, seed=5)
    G, nb = N // gs, K // rs
    eye = torch.eye(rs).repeat(G, nb)  # identity blocks
    # identity R: plain forward is a dense linear layer
    assert torch.allclose(O.prism_forward(A, B, eye, gs, rs), A @ B.T, atol=1e-5)
    # R = 0: gated forward is exactly zero
    assert O.prism_forward(A, B, torch.zeros_like(eye), gs, rs, "silu_gate").abs().max() == 0
    # permutation blocks: S is a column permutation of A inside each block
    perm = torch.randperm(rs, generator=torch.Generator().manual_seed(0))
    P = torch.eye(rs)[perm]
    Rp = P.repeat(G, nb)
    S = O.rotate(A, O._blocks(Rp, G, rs)[0])
    assert torch.equal(S.reshape(M, nb, rs), A.reshape(M, nb, rs)[:, :, perm])


def test_flop_model():
    f, d, b = O.flops(16384, 4096, 14336, 256, 16)
    assert abs(f / 1e9 - 2044.4) < 0.5 and abs(d / 1e9 - 2164.7) < 0.5 and abs(b / 1e9 - 1924.2) < 0.5


def test_dropout_hash_matches_the_scalar_definition():
    """The vectorised mask of the oracle against the scalar definition of the reference's kernels
    (cute_prism_dtype.hpp:28-40; the reference's own Python mirror is tests/test_cublas_backend.py:40-51):
    u = top24(splitmix64(splitmix64(seed + 0xdeadbeef) ^ splitmix64(idx))) / 2^24, keep iff u >= p."""
    M64 = (1 << 64) - 1

    def splitmix64(x):
        x = (x + 0x9E3779B97F4A7C15) & M64
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M64
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M64
        return (x ^ (x >> 31)) & M64

    assert splitmix64(0) == 0xE220A8397B1DCDAF          # first output of the published generator seeded with 0
    for seed, M, K, p in ((1, 3, 16, 0.1), (0x0123456789ABCDEF, 7, 24, 0.5), ((1 << 62) - 1, 2, 40, 0.9)):
        mult = O.dropout_multiplier(seed, M, K, p)
        h1 = splitmix64((seed + 0xDEADBEEF) & M64)
        for m in range(M):
            for k in range(K):
                h = splitmix64(h1 ^ splitmix64(m * K + k))
                u = ((h >> 40) & 0xFFFFFF) * (1.0 / 16777216.0)
                want = 1.0 / (1.0 - p) if np.float32(u) >= np.float32(p) else 0.0
                assert abs(mult[m, k].item() - want) < 1e-6, (seed, m, k)
    big = O.dropout_multiplier(12345, 256, 256, 0.25)
    assert abs((big > 0).float().mean().item() - 0.75) < 0.01
