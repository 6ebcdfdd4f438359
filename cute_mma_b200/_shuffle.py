"""Input shuffle of the Prism layer, folded into the parameters.

The reference lets every output group see its own permutation of the input features: inside each chunk
of ``shuffle_blk_k`` = 64 features, 2-element segments are exchanged between the chunk's 16-wide rotation
blocks by a butterfly of XOR-partner swaps, one packed bit mask per (group, chunk, round)
(src/cute_prism/_module.py:225-270; src/cute_prism/_pytorch_backend.py:31-76).  Its kernels and backends
gather a permuted copy of A per group (a ``(G, M, K)`` buffer, torch_ext/prism_fwd_torch.cu:122-139).

Here nothing is gathered per token.  With ``A_g[:, c] = A[:, perm_g[c]]`` the group's rotation in the
permuted space, ``S_g = A_g . blockdiag(R_g)^T``, is the same numbers as ``A . R64_g^T`` read in physical
feature order, where ``R64_g = P_g . blockdiag(R_g) . P_g^T`` is block diagonal with 64 x 64 blocks (the
permutation never leaves a chunk): a Prism rotation with ``reconn_sz = 64``, which the sm_100a kernels run
at the cost of the 16-wide one (a ``tcgen05.mma`` with N = 64 takes the time of one with N = 16).  The gate
is elementwise, so ``H`` comes out in physical order too, and ``C_g = H_g . B_g^T`` holds with the columns
of ``B_g`` (and of the internal bias) put into physical order once per call.  The gradients come back
through the same index maps; dA needs none.
"""
from __future__ import annotations

import math

import torch

SHUFFLE_SEGMENT_SZ = 2   # elements per exchanged segment (src/cute_prism/_module.py:13)
_M64 = 0xFFFFFFFFFFFFFFFF


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return (x ^ (x >> 31)) & _M64


def partition_deltas(n_segments: int, block_size: int) -> list[int]:
    """XOR deltas (in segments) that move a segment to another rotation block: the powers of two from the
    block size up (src/cute_prism/_module.py:225-233)."""
    return [1 << r for r in range(int(math.log2(n_segments))) if (1 << r) >= block_size]


def build_shuffle_masks(in_features: int, out_features: int, group_size: int, reconn_sz: int,
                        shuffle_blk_k: int = 64) -> tuple[torch.Tensor, list[int]]:
    """The reference's masks: ``(G, K / shuffle_blk_k, rounds)`` int64, group 0 the identity, the others
    hashed from (group, chunk, round) (src/cute_prism/_module.py:236-270)."""
    n_groups = out_features // group_size
    n_chunks = in_features // shuffle_blk_k
    n_segments = shuffle_blk_k // SHUFFLE_SEGMENT_SZ
    deltas = partition_deltas(n_segments, reconn_sz // SHUFFLE_SEGMENT_SZ)
    pair_mask = (1 << (n_segments // 2)) - 1
    masks = torch.zeros(n_groups, n_chunks, len(deltas), dtype=torch.long)
    for g in range(1, n_groups):
        for c in range(n_chunks):
            for r in range(len(deltas)):
                masks[g, c, r] = _splitmix64(g * 0xDEADBEEF + c * 0xCAFEBABE + r * 0x12345678) & pair_mask
    return masks, deltas


def shuffle_perm(shuffle_masks: torch.Tensor, K: int, reconn_sz: int) -> torch.Tensor:
    """``perm`` of shape ``(G, K)`` with ``A_g[:, i] = A[:, perm[g, i]]`` (src/cute_prism/_pytorch_backend.py:31-76),
    for all groups and chunks at once."""
    masks = shuffle_masks.detach().to("cpu", torch.long)
    G, n_chunks, n_rounds = masks.shape
    blk = K // n_chunks
    n_seg = blk // SHUFFLE_SEGMENT_SZ
    deltas = partition_deltas(n_seg, reconn_sz // SHUFFLE_SEGMENT_SZ)
    if len(deltas) != n_rounds:
        raise ValueError(f"shuffle_masks has {n_rounds} rounds, reconn_sz={reconn_sz} with chunks of {blk} needs {len(deltas)}")
    seg = torch.arange(n_seg).expand(G, n_chunks, n_seg).clone()
    for r, delta in enumerate(deltas):
        lo = torch.tensor([i for i in range(n_seg) if (i ^ delta) > i])
        hi = lo ^ delta
        bits = ((masks[:, :, r, None] >> torch.arange(lo.numel())) & 1).bool()   # pair p = the p-th such i
        a, b = seg[:, :, lo], seg[:, :, hi]
        seg[:, :, lo] = torch.where(bits, b, a)
        seg[:, :, hi] = torch.where(bits, a, b)
    e = torch.arange(SHUFFLE_SEGMENT_SZ)
    perm = (torch.arange(n_chunks)[None, :, None, None] * blk + seg[..., None] * SHUFFLE_SEGMENT_SZ + e)
    return perm.reshape(G, K)


class ShuffleFold:
    """Index maps of one set of masks (built once per module, or per functional call)."""

    def __init__(self, shuffle_masks: torch.Tensor, K: int, group_size: int, reconn_sz: int, device):
        if reconn_sz != 16:
            raise ValueError("input_shuffle requires reconn_sz=16")
        G, n_chunks, _ = shuffle_masks.shape
        if n_chunks == 0 or K % n_chunks != 0 or K // n_chunks != 64:
            raise ValueError("input shuffle is built for chunks of 64 features (shuffle_blk_k = 64)")
        self.G, self.K, self.gs, self.rs, self.n_chunks = G, K, group_size, reconn_sz, n_chunks
        perm = shuffle_perm(shuffle_masks, K, reconn_sz)                     # logical -> physical
        inv = torch.empty_like(perm)
        inv.scatter_(1, perm, torch.arange(K).expand(G, K))                   # physical -> logical
        self.perm = perm.to(device)
        self.inv = inv.to(device)
        self.inv_in_chunk = (inv.view(G, n_chunks, 64) % 64).to(device)       # the same, inside its chunk
        self.perm_in_chunk = (perm.view(G, n_chunks, 64) % 64).to(device)

    def fold_R(self, R: torch.Tensor) -> torch.Tensor:
        """``R (G * 16, K)`` -> ``R64 (G * 64, K)``: per chunk ``P . blockdiag(R) . P^T`` (differentiable)."""
        G, nc = self.G, self.n_chunks
        Rb = R.view(G, 16, nc, 4, 16).permute(0, 2, 3, 1, 4)                  # g, chunk, block, i, j
        bd = R.new_zeros(G, nc, 4, 16, 4, 16)
        for b in range(4):
            bd[:, :, b, :, b, :] = Rb[:, :, b]
        bd = bd.view(G, nc, 64, 64)                                            # logical rows (S columns) x logical columns
        idx = self.inv_in_chunk
        r64 = bd.gather(2, idx[:, :, :, None].expand(-1, -1, -1, 64)).gather(3, idx[:, :, None, :].expand(-1, -1, 64, -1))
        return r64.permute(0, 2, 1, 3).reshape(G * 64, self.K).contiguous()

    def unfold_dR(self, dR64: torch.Tensor) -> torch.Tensor:
        """Gradient of ``fold_R``: the diagonal 16 x 16 blocks of ``P^T . dR64 . P``."""
        G, nc = self.G, self.n_chunks
        d = dR64.view(G, 64, nc, 64).permute(0, 2, 1, 3)
        idx = self.perm_in_chunk
        d = d.gather(2, idx[:, :, :, None].expand(-1, -1, -1, 64)).gather(3, idx[:, :, None, :].expand(-1, -1, 64, -1))
        d = d.view(G, nc, 4, 16, 4, 16)
        out = torch.stack([d[:, :, b, :, b, :] for b in range(4)], dim=2)      # g, chunk, block, i, j
        return out.permute(0, 3, 1, 2, 4).reshape(G * 16, self.K).contiguous()

    def fold_cols(self, X: torch.Tensor, rows_per_group: int) -> torch.Tensor:
        """Columns of a per-group matrix (``B``: ``(G * gs, K)``; internal bias: ``(G, K)``) into physical order."""
        Xg = X.view(self.G, rows_per_group, self.K)
        return Xg.gather(2, self.inv[:, None, :].expand(-1, rows_per_group, -1)).reshape(X.shape).contiguous()

    def unfold_cols(self, dX: torch.Tensor, rows_per_group: int) -> torch.Tensor:
        dXg = dX.view(self.G, rows_per_group, self.K)
        return dXg.gather(2, self.perm[:, None, :].expand(-1, rows_per_group, -1)).reshape(dX.shape).contiguous()
