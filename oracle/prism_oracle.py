"""CPU/torch restatement of the reference Prism layer arithmetic -- TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA kernels: it is imported by the tests, by the
smoke check and by the benchmark's CPU-baseline leg, and by nothing in the shipped
package.  It restates, in plain torch tensor algebra, what the reference computes in
``src/cute_prism/_pytorch_backend.py``:

* forward  (``pytorch_forward``,  lines 78-176):  per output group g
  ``S_g = A . blockdiag(R_g)^T``;  plain mode ``H_g = S_g``; gated modes
  ``H_g = A * silu(S_g)`` (silu_gate) or ``H_g = A * 2 sigmoid(S_g)`` (sigmoid_gate, lines 157-163);
  ``C[:, g] = H_g @ B_g^T``.
* backward (``pytorch_backward``, lines 179-321):  ``dH_g = dC_g @ B_g``;
  gated: ``dS = dH * A * gate'(S)``, ``dA += dH * gate(S) + blockdiag(dS) . R_g``,
  ``dB_g = dC_g^T @ H_g`` (gate = silu, or 2 sigmoid with derivative 2 sigmoid (1 - sigmoid), lines 250-262);
  plain: ``dS = dH``, ``dA += blockdiag(dS) . R_g``, no dB;
  both: ``dR_g[block b] = dS_b^T @ A_b``.

Parity pin: ``tests/golden/make_golden.py`` imports the reference package itself,
runs its pytorch backend on seeded inputs and stores inputs + outputs under
``tests/golden/``; ``tests/test_oracle.py`` checks this file against those vectors
(and against torch autograd in float64).  Only the features on the accelerated path
are restated: mode ``ar`` with ``silu_gate`` / ``sigmoid_gate``, the internal bias and the kernels' hash dropout
(the pytorch backend's own dropout draws its masks with torch.rand instead); no shuffle or rw mode.
"""
from __future__ import annotations

import math

import torch


def _blocks(R: torch.Tensor, n_groups: int, rs: int) -> torch.Tensor:
    """R (G*rs, K) -> (G, nb, rs_i, rs_j): block b of group g is R[g*rs+i, b*rs+j]."""
    K = R.shape[1]
    return R.reshape(n_groups, rs, K // rs, rs).permute(0, 2, 1, 3)


def rotate(A: torch.Tensor, Rg_blocks: torch.Tensor) -> torch.Tensor:
    """S = A . blockdiag(R_g)^T for one group: S[:, b*rs+i] = sum_j A[:, b*rs+j] R_g[b,i,j]."""
    M, K = A.shape
    nb, rs, _ = Rg_blocks.shape
    Ab = A.reshape(M, nb, rs)
    return torch.einsum("mbj,bij->mbi", Ab, Rg_blocks).reshape(M, K)


def rotate_t(dS: torch.Tensor, Rg_blocks: torch.Tensor) -> torch.Tensor:
    """blockdiag(dS) . R_g: out[:, b*rs+j] = sum_i dS[:, b*rs+i] R_g[b,i,j]."""
    M, K = dS.shape
    nb, rs, _ = Rg_blocks.shape
    return torch.einsum("mbi,bij->mbj", dS.reshape(M, nb, rs), Rg_blocks).reshape(M, K)


GATES = (None, "silu_gate", "sigmoid_gate")


def _gate(S, activation):
    """(gate(S), gate'(S)) of a gated mode."""
    sig = torch.sigmoid(S)
    if activation == "silu_gate":
        return S * sig, sig * (1.0 + S * (1.0 - sig))
    return 2.0 * sig, 2.0 * sig * (1.0 - sig)


_M64 = (1 << 64) - 1


def _splitmix64_int(x: int) -> int:
    """splitmix64 on Python integers (the published mixer; the reference's mirror is
    tests/test_cublas_backend.py:40-44)."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return (x ^ (x >> 31)) & _M64


def _srl(x, n):
    """logical right shift of int64 tensors holding uint64 bit patterns"""
    return (x >> n) & ((1 << (64 - n)) - 1)


def _as_i64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _splitmix64_t(x):
    """splitmix64 on an int64 tensor (two's-complement wrap-around = arithmetic mod 2^64)"""
    x = x + _as_i64(0x9E3779B97F4A7C15)
    x = (x ^ _srl(x, 30)) * _as_i64(0xBF58476D1CE4E5B9)
    x = (x ^ _srl(x, 27)) * _as_i64(0x94D049BB133111EB)
    return x ^ _srl(x, 31)


def dropout_multiplier(seed: int, M: int, K: int, p: float, device="cpu"):
    """(M, K) fp32 multipliers of the reference kernels' hash dropout (cute_prism_dtype.hpp:28-40,
    cute_prism_coop_pc.cu:294-298): 1/(1-p) where u >= p, else 0, with
    u = top24(splitmix64(splitmix64(seed + 0xdeadbeef) ^ splitmix64(m*K + k))) / 2^24."""
    h1 = _as_i64(_splitmix64_int((int(seed) + 0xDEADBEEF) & _M64))
    idx = torch.arange(M * K, dtype=torch.int64, device=device)
    h = _splitmix64_t(_splitmix64_t(idx) ^ h1)
    u = (_srl(h, 40) & 0xFFFFFF).to(torch.float32) * (1.0 / 16777216.0)
    keep = u >= torch.tensor(p, dtype=torch.float32, device=device)
    return (keep.to(torch.float32) * (1.0 / (1.0 - p))).reshape(M, K)


SHUFFLE_SEGMENT_SZ = 2   # src/cute_prism/_pytorch_backend.py:12


def shuffle_elem_perm(masks_g, K, reconn_sz):
    """One group's element permutation, ``A_g[:, i] = A[:, perm[i]]``: inside every chunk of
    K / n_chunks features the 2-element segments go through one round of XOR-partner swaps per delta (the
    powers of two from the block size in segments up), pair p of a round swapped when bit p of the round's
    mask is set (src/cute_prism/_pytorch_backend.py:25-76).  Plain loops: test infrastructure."""
    n_chunks, n_rounds = masks_g.shape
    blk = K // n_chunks
    n_seg = blk // SHUFFLE_SEGMENT_SZ
    block_size = reconn_sz // SHUFFLE_SEGMENT_SZ
    deltas = [1 << r for r in range(n_seg.bit_length() - 1) if (1 << r) >= block_size]
    assert len(deltas) == n_rounds
    perm = list(range(K))
    for c in range(n_chunks):
        seg = list(range(n_seg))
        for r, delta in enumerate(deltas):
            bits = int(masks_g[c, r])
            new = list(seg)
            pair = 0
            for i in range(n_seg):
                partner = i ^ delta
                if partner > i and partner < n_seg:
                    if (bits >> pair) & 1:
                        new[i], new[partner] = new[partner], new[i]
                    pair += 1
            seg = new
        for dst, src in enumerate(seg):
            for e in range(SHUFFLE_SEGMENT_SZ):
                perm[c * blk + dst * SHUFFLE_SEGMENT_SZ + e] = c * blk + src * SHUFFLE_SEGMENT_SZ + e
    return torch.tensor(perm, dtype=torch.long)


def prism_forward(A, B, R, group_size, reconn_sz, activation=None, bias=None, internal_bias=None,
                  dropout_seeds=None, dropout_p=0.0, shuffle_masks=None):
    """C (M, N) in the dtype of A.  Follows ``pytorch_forward`` (ar mode, optional gate; the internal bias
    (G, K) is added to S before the gate, lines 154-156)."""
    if activation not in GATES:
        raise ValueError(f"oracle restates {GATES} only, got {activation!r}")
    M, K = A.shape
    N = B.shape[0]
    G = N // group_size
    Rb = _blocks(R, G, reconn_sz)
    C = torch.empty(M, N, dtype=A.dtype, device=A.device)
    A_in = A
    for g in range(G):
        if shuffle_masks is not None:   # this group's permuted view of the input (lines 143-149); all that follows lives in it
            A = A_in.index_select(1, shuffle_elem_perm(shuffle_masks[g].cpu(), K, reconn_sz).to(A_in.device))
        S = rotate(A, Rb[g])
        if activation is not None and internal_bias is not None:
            S = S + internal_bias[g]
        H = A * _gate(S, activation)[0] if activation is not None else S
        if activation is not None and dropout_seeds is not None and dropout_p > 0.0:
            H = H * dropout_multiplier(int(dropout_seeds[g]), M, K, dropout_p, A.device).to(H.dtype)
        C[:, g * group_size:(g + 1) * group_size] = H @ B[g * group_size:(g + 1) * group_size].T
    if bias is not None:
        C = C + bias
    return C


def prism_backward(dC, A, B, R, group_size, reconn_sz, activation=None, internal_bias=None,
                   dropout_seeds=None, dropout_p=0.0, shuffle_masks=None):
    """(dA, dR, dB-or-None), plus d_internal_bias (G, K) = sum over tokens of dS as a fourth element when an
    internal bias is given (lines 246-248, 271-272).  Follows ``pytorch_backward``."""
    if activation not in GATES:
        raise ValueError(f"oracle restates {GATES} only, got {activation!r}")
    M, K = A.shape
    N = B.shape[0]
    G = N // group_size
    rs = reconn_sz
    nb = K // rs
    gated = activation is not None
    Rb = _blocks(R, G, rs)
    dA = torch.zeros_like(A)
    dR = torch.empty_like(R)
    dB = torch.empty_like(B) if gated else None
    d_ib = torch.empty_like(internal_bias) if (gated and internal_bias is not None) else None
    A_in = A
    Ab = A.reshape(M, nb, rs)
    for g in range(G):
        sl = slice(g * group_size, (g + 1) * group_size)
        dC_g = dC[:, sl]
        dH = dC_g @ B[sl]
        perm = None
        if shuffle_masks is not None:   # gradients in the group's permuted space, dA added back through the permutation (lines 233-240, 300-304)
            perm = shuffle_elem_perm(shuffle_masks[g].cpu(), K, reconn_sz).to(A_in.device)
            A = A_in.index_select(1, perm)
            Ab = A.reshape(M, nb, rs)
        dA_g = torch.zeros_like(A)
        if gated:
            S = rotate(A, Rb[g])
            if internal_bias is not None:
                S = S + internal_bias[g]
            gate, gate_d = _gate(S, activation)
            H = A * gate
            if dropout_seeds is not None and dropout_p > 0.0:   # the forward's mask on H and on dH (lines 264-276)
                mult = dropout_multiplier(int(dropout_seeds[g]), M, K, dropout_p, A.device).to(H.dtype)
                H = H * mult
                dH = dH * mult
            dB[sl] = dC_g.T @ H
            dS = dH * A * gate_d
            if d_ib is not None:
                d_ib[g] = dS.sum(dim=0)
            dA_g += dH * gate
        else:
            dS = dH
        dA_g += rotate_t(dS, Rb[g])
        if perm is None:
            dA += dA_g
        else:
            dA.index_add_(1, perm, dA_g)
        # dR block (g, b)[i, j] = sum_m dS[m, b*rs+i] * A[m, b*rs+j]
        dRg = torch.einsum("mbi,mbj->ibj", dS.reshape(M, nb, rs), Ab)
        dR[g * rs:(g + 1) * rs] = dRg.reshape(rs, K)
    if d_ib is not None:
        return dA, dR, dB, d_ib
    return dA, dR, dB


# ---------------------------------------------------------------------------
# seeded synthetic inputs (shapes and value distributions of the benchmark configs)
# ---------------------------------------------------------------------------
def orthogonal_R(n_groups, K, rs, gen):
    """Seeded block-orthogonal R: every rs x rs block is the Q factor of a Gaussian QR."""
    nb = K // rs
    Z = torch.randn(n_groups, nb, rs, rs, generator=gen, dtype=torch.float64)
    Q, _ = torch.linalg.qr(Z)
    return Q.permute(0, 2, 1, 3).reshape(n_groups * rs, K).to(torch.float32).contiguous()


def make_inputs(M, K, N, group_size, reconn_sz, seed=0, a_std=1.0, b_std=1.0, dc_std=1.0,
                r_kind="orthogonal"):
    """fp32 CPU tensors drawn in the fixed order A, B, R, dC from one seeded generator."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randn(M, K, generator=gen) * a_std
    B = torch.randn(N, K, generator=gen) * b_std
    G = N // group_size
    if r_kind == "orthogonal":
        R = orthogonal_R(G, K, reconn_sz, gen)
    elif r_kind == "gaussian":
        R = torch.randn(G * reconn_sz, K, generator=gen) / math.sqrt(reconn_sz)
    else:
        raise ValueError(r_kind)
    dC = torch.randn(M, N, generator=gen) * dc_std
    return A, B, R, dC


def rel_err(val, ref):
    """The reference tests' metric: max|val-ref| / (max|ref| + 1e-6)  (tests/test_correctness.py:24-31)."""
    wide = torch.float64 if torch.float64 in (val.dtype, ref.dtype) else torch.float32
    val = val.to(wide)
    ref = ref.to(wide)
    return ((val - ref).abs().max().double() / (ref.abs().max().double() + 1e-6)).item()


def mean_rel_err(val, ref, floor=1e-4):
    """The reference tests' second metric: mean of |val-ref| / |ref| over the elements with
    |ref| > floor  (tests/test_backward.py:96-108, tests/test_correctness.py:90-100)."""
    val = val.float()
    ref = ref.float()
    mask = ref.abs() > floor
    n = int(mask.sum().item())
    if n == 0:
        return 0.0
    rel = torch.where(mask, (val - ref).abs() / ref.abs().clamp_min(floor), torch.zeros_like(ref))
    return (rel.double().sum() / n).item()


def flops(M, K, N, group_size, reconn_sz):
    """Algorithmic work per call: (fwd, bwd_dadr, bwd_db) in FLOP; recompute is not counted."""
    dense = 2.0 * M * N * K
    bd = 2.0 * M * K * reconn_sz * (N // group_size)
    return dense + bd, dense + 2 * bd, dense
