"""Host-side logic that needs no GPU: argument validation (same rules as the reference's
src/cute_prism/_validate.py), the tile table, PrismLinear construction / state / R construction,
and the token-sharded gradient all-reduce on two gloo ranks."""
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cute_mma_b200 as cp
from cute_mma_b200 import _functional as F
from cute_mma_b200 import _tile_table
from oracle import prism_oracle as O


def test_validate_kernel_params():
    F.validate_kernel_params(256, 8)
    for gs, rs in ((0, 8), (256, 0), (256, 12), (100, 8), (2.5, 8)):
        with pytest.raises(ValueError):
            F.validate_kernel_params(gs, rs)


def test_forward_rejects_cpu_and_bad_options():
    A, B, R = torch.randn(8, 64), torch.randn(64, 64), torch.randn(16, 64)
    with pytest.raises(ValueError, match="CUDA"):
        cp.forward(A.half(), B.half(), R.half(), 32, 8)
    with pytest.raises(ValueError, match="activation"):
        cp.forward(A, B, R, 32, 8, activation="relu")
    with pytest.raises(ValueError, match="CUDA"):
        cp.forward(A, B, R, 32, 8, activation="sigmoid_gate")   # a known activation: fails on the device check
    with pytest.raises(ValueError, match="mode"):
        cp.forward(A, B, R, 32, 8, mode="wr")
    with pytest.raises(ValueError, match="gated"):
        cp.forward(A, B, R, 32, 8, mode="rw", activation="silu_gate")
    with pytest.raises(ValueError, match="gated"):
        F._check_internal_bias(torch.zeros(2, 64), A, 64, 64, 32, 0)      # plain mode has no internal bias
    with pytest.raises(ValueError, match="internal_bias must"):
        F._check_internal_bias(torch.zeros(3, 64), A, 64, 64, 32, 1)      # wrong shape
    with pytest.raises(ValueError):
        cp.backward(torch.randn(8, 64), A, B, R, 32, 12)


def test_tile_table_lookup(tmp_path):
    path = tmp_path / "tt.json"
    path.write_text(json.dumps({"entries": [
        {"kernel": "fwd", "dtype": "bf16", "gate": 1, "M": 0, "N": 14336, "K": 4096, "gs": 256, "rs": 16, "cfg": [64, 16]},
        {"kernel": "fwd", "dtype": "bf16", "gate": 1, "M": 1024, "N": 14336, "K": 4096, "gs": 256, "rs": 16, "cfg": [256, 16]},
        {"kernel": "bwd_db", "dtype": "*", "gate": "*", "M": 0, "N": "*", "K": "*", "gs": "*", "rs": "*", "cfg": [128, 2]},
    ]}))
    _tile_table.load(str(path))
    try:
        look = _tile_table.lookup
        assert look("fwd", torch.bfloat16, 1, 16, 14336, 4096, 256, 16) == [64, 16]
        assert look("fwd", torch.bfloat16, 1, 16384, 14336, 4096, 256, 16) == [256, 16]
        assert look("fwd", torch.float16, 1, 16384, 14336, 4096, 256, 16) is None
        assert look("bwd_db", torch.float16, 1, 77, 512, 512, 64, 8) == [128, 2]
        assert look("bwd_dadr", torch.float16, 1, 77, 512, 512, 64, 8) is None
    finally:
        _tile_table.load()  # restore the shipped table
    assert isinstance(_tile_table.load(), list)


def test_prism_linear_construction_and_state():
    m = cp.PrismLinear(64, 128, group_size=32, reconn_sz=8)
    assert sorted(m.state_dict()) == ["bias", "reconn", "weight"]
    assert m.weight.shape == (128, 64) and m.reconn.shape == (32, 64) and m.bias.shape == (128,)
    assert not m.weight.requires_grad and m.reconn.requires_grad
    assert m._bwd_scale == 1.0
    g = cp.PrismLinear(64, 128, group_size=32, reconn_sz=16, activation="silu_gate", bias=False)
    assert g.weight.requires_grad and g.bias is None
    assert abs(g._bwd_scale - 1 / 1.437) < 1e-12
    # gated R is block skew-symmetric at init
    Rb = g._build_R().reshape(4, 16, 4, 16).permute(0, 2, 1, 3)
    assert torch.allclose(Rb, -Rb.transpose(-1, -2))
    m2 = cp.PrismLinear(64, 128, group_size=32, reconn_sz=8)
    m2.load_state_dict(m.state_dict())
    assert torch.equal(m2.weight, m.weight)
    sg = cp.PrismLinear(64, 128, group_size=32, reconn_sz=16, activation="sigmoid_gate")
    assert sg.weight.requires_grad and abs(sg._bwd_scale - 1 / 1.15) < 1e-12
    ibl = cp.PrismLinear(64, 128, group_size=32, reconn_sz=16, activation="silu_gate", internal_bias=True)
    assert ibl._internal_bias.shape == (4, 64) and "_internal_bias" in ibl.state_dict()
    assert cp.PrismLinear(64, 128, group_size=32, reconn_sz=16, internal_bias=True)._internal_bias is None   # plain mode: none
    dl = cp.PrismLinear(64, 128, group_size=32, reconn_sz=16, activation="silu_gate", dropout=0.1)
    assert dl.dropout == pytest.approx(0.1)
    with pytest.raises(ValueError):
        cp.PrismLinear(64, 128, group_size=32, reconn_sz=32, activation="silu_gate", dropout=0.1)   # 8 / 16 only
    sh = cp.PrismLinear(128, 128, group_size=32, reconn_sz=16, activation="silu_gate", input_shuffle=True)
    assert sh._shuffle_masks.shape == (4, 2, 2) and "_shuffle_masks" in sh.state_dict()
    assert int(sh._shuffle_masks[0].abs().sum()) == 0          # group 0 keeps the natural order
    for bad in (dict(input_shuffle=True, reconn_sz=8), dict(input_shuffle=True, shuffle_blk_k=32),
                dict(input_shuffle=True, activation="silu_gate", dropout=0.1), dict(activation="tanh")):
        kw = dict(reconn_sz=16)
        kw.update(bad)
        with pytest.raises(ValueError):
            cp.PrismLinear(128, 128, 32, **kw)
    with pytest.raises(ValueError):
        cp.PrismLinear(64, 100, 32, 8)


def test_build_R_identity_and_orthogonal():
    m = cp.PrismLinear(64, 64, group_size=32, reconn_sz=8)
    R = m._build_R()
    assert torch.allclose(R, torch.eye(8).repeat(2, 8))  # reconn = 0  ->  identity blocks
    with torch.no_grad():
        m.reconn.normal_(0, 0.3)
    for order in (float("inf"), 2):
        m.cayley_order = order
        Rb = m._build_R().reshape(2, 8, 8, 8).permute(0, 2, 1, 3)
        if order == float("inf"):
            assert torch.allclose(Rb @ Rb.transpose(-1, -2), torch.eye(8).expand_as(Rb), atol=1e-5)
    # 16-bit parameters: solved in fp32, returned in the parameter dtype
    mb = cp.PrismLinear(64, 64, group_size=32, reconn_sz=8).to(torch.bfloat16)
    assert mb._build_R().dtype == torch.bfloat16


def test_from_linear_copies_weights():
    lin = torch.nn.Linear(64, 128)
    m = cp.PrismLinear.from_linear(lin, group_size=32, reconn_sz=8)
    assert torch.equal(m.weight, lin.weight) and torch.equal(m.bias, lin.bias)


def test_shard_rows():
    assert [cp.shard_rows(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert cp.shard_rows(65536, 7, 8) == (57344, 65536)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import prism_oracle as O
        M, K, N, gs, rs = 64, 64, 64, 32, 8
        A, B, R, dC = O.make_inputs(M, K, N, gs, rs, seed=2)
        lo, hi = cp.shard_rows(M, rank, world)
        # each rank computes the gradients of its token rows (here with the CPU oracle standing in
        # for the kernels), then the parameter gradients are summed over ranks
        dA, dR, dB = O.prism_backward(dC[lo:hi], A[lo:hi], B, R, gs, rs, "silu_gate")
        dbias = dC[lo:hi].sum(0)
        cp.allreduce_grads([dR, dB, dbias, dR.double()])
        fA, fR, fB = O.prism_backward(dC, A, B, R, gs, rs, "silu_gate")
        ok = (torch.allclose(dR, fR, atol=1e-4) and torch.allclose(dB, fB, atol=1e-4)
              and torch.allclose(dbias, dC.sum(0), atol=1e-4) and torch.allclose(dA, fA[lo:hi], atol=1e-4))
        # async form
        t = torch.full((5,), float(rank + 1))
        fin = cp.allreduce_grads([t], average=True, async_op=True)
        fin()
        ok = ok and torch.allclose(t, torch.full((5,), (1 + world) / 2))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_token_sharded_gradients_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_dp_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(out) == {0: True, 1: True}


def test_allreduce_is_a_noop_without_process_group():
    t = torch.ones(3)
    assert cp.allreduce_grads([t]) is None
    assert torch.equal(t, torch.ones(3))


def test_input_shuffle_fold_is_the_reference_shuffle():
    """The per-group butterfly permutation folded into a 64-wide rotation and a column order of B (what the
    kernels are given) is the shuffled layer itself: checked with the oracle in float64 on the CPU, forward and
    every gradient, against the oracle's own per-group gather (which follows the reference)."""
    from cute_mma_b200 import _shuffle as S
    M, K, N, gs, rs = 20, 192, 384, 128, 16
    masks, deltas = S.build_shuffle_masks(K, N, gs, rs)
    assert deltas == [8, 16] and masks.shape == (3, 3, 2) and int(masks[1:].abs().sum()) > 0
    fold = S.ShuffleFold(masks, K, gs, rs, "cpu")
    for g in range(3):
        assert torch.equal(fold.perm[g], O.shuffle_elem_perm(masks[g], K, rs))
        assert torch.equal(fold.perm[g][fold.inv[g]], torch.arange(K))
    gen = torch.Generator().manual_seed(5)
    A = torch.randn(M, K, generator=gen, dtype=torch.float64)
    B = torch.randn(N, K, generator=gen, dtype=torch.float64) * K ** -0.5
    R = O.orthogonal_R(N // gs, K, rs, gen).double()
    dC = torch.randn(M, N, generator=gen, dtype=torch.float64)
    ib = torch.randn(N // gs, K, generator=gen, dtype=torch.float64) * 0.3
    for act in (None, "silu_gate", "sigmoid_gate"):
        ibx = ib if act else None
        C = O.prism_forward(A, B, R, gs, rs, act, internal_bias=ibx, shuffle_masks=masks)
        grads = O.prism_backward(dC, A, B, R, gs, rs, act, internal_bias=ibx, shuffle_masks=masks)
        R64, B2 = fold.fold_R(R), fold.fold_cols(B, gs)
        ib2 = fold.fold_cols(ib, 1) if act else None
        assert (O.prism_forward(A, B2, R64, gs, 64, act, internal_bias=ib2) - C).abs().max() < 1e-12
        gf = O.prism_backward(dC, A, B2, R64, gs, 64, act, internal_bias=ib2)
        assert (gf[0] - grads[0]).abs().max() < 1e-12
        assert (fold.unfold_dR(gf[1]) - grads[1]).abs().max() < 1e-12
        if act:
            assert (fold.unfold_cols(gf[2], gs) - grads[2]).abs().max() < 1e-12
            assert (fold.unfold_cols(gf[3], 1) - grads[3]).abs().max() < 1e-12
        # the fold is differentiable: autograd through it gives the same dR as the explicit unfold
        Rq = R.clone().requires_grad_(True)
        (fold.fold_R(Rq) * gf[1]).sum().backward()
        assert (Rq.grad - fold.unfold_dR(gf[1])).abs().max() < 1e-12
