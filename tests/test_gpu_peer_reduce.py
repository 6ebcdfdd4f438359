"""The gradient exchange over peer memory (prism_peer_reduce / PeerGradReducer).

On one GPU the ranks are emulated: every "rank" has its own buffers on the same device and its kernel is
launched in turn -- the kernel waits for nobody, so this exercises slicing, the rank-order sum, scaling and
casts completely.  With two or more GPUs the real thing runs as one process per GPU over symmetric memory.
"""
import ctypes
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from cute_mma_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("out", [torch.bfloat16, torch.float16, torch.float32])
def test_peer_reduce_emulated_ranks(world, out):
    L = _lib.lib()
    n = 4 * 12345 * world + 4 * 7          # not a multiple of the slice granularity times world
    g = torch.Generator(device=DEV).manual_seed(world)
    ins = [torch.randn(n, device=DEV, generator=g) for _ in range(world)]
    outs = [torch.full((n,), float("nan"), dtype=out, device=DEV) for _ in range(world)]
    vp = ctypes.c_void_p
    in_ptrs = (vp * world)(*[vp(t.data_ptr()) for t in ins])
    out_ptrs = (vp * world)(*[vp(t.data_ptr()) for t in outs])
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out]
    stream = vp(torch.cuda.current_stream().cuda_stream)
    for rank in range(world):
        _lib.check(L.prism_peer_reduce(in_ptrs, out_ptrs, world, rank, n, code, ctypes.c_float(0.5), 4 + rank, stream))
    torch.cuda.synchronize()
    ref = ins[0].clone()
    for t in ins[1:]:
        ref += t                            # rank order, fp32
    ref = (ref * 0.5).to(out)
    for o in outs:
        assert torch.equal(o, ref)          # every rank holds the same bits
    # bad arguments are refused before anything is launched
    assert L.prism_peer_reduce(in_ptrs, out_ptrs, world, world, n, code, ctypes.c_float(1.0), 0, stream) != 0
    assert L.prism_peer_reduce(in_ptrs, out_ptrs, world, 0, n + 2, code, ctypes.c_float(1.0), 0, stream) != 0


def _find_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    import cute_mma_b200 as cp
    shapes = [(512, 256), (32, 256), (512,)]
    red = cp.PeerGradReducer(shapes, out_dtype=torch.bfloat16, ctas=8)
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    grads = [torch.randn(s, device=dev, generator=g) for s in shapes]
    ok = True
    for _ in range(3):
        red.stage(grads)
        outs = [o.clone() for o in red.reduce()]
        torch.cuda.synchronize()
        for o, x in zip(outs, grads):
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            exact = parts[0].clone()
            for t in parts[1:]:
                exact += t
            ok = ok and torch.equal(o, exact.to(torch.bfloat16))
    # a module's gradients through the same exchange, averaged like DistributedDataParallel
    torch.manual_seed(7)
    lin = torch.nn.Linear(64, 32).to(dev)
    lin(torch.randn(16, 64, device=dev, generator=torch.Generator(device=dev).manual_seed(rank))).square().sum().backward()
    want = [p.grad.clone() for p in lin.parameters()]
    for w_ in want:
        dist.all_reduce(w_)
        w_ /= world
    cp.sync_module_grads(lin, reducer=cp.PeerGradReducer.for_module(lin, ctas=4))
    torch.cuda.synchronize()
    ok = ok and all(torch.allclose(p.grad, w_, rtol=1e-5, atol=1e-6) for p, w_ in zip(lin.parameters(), want))
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_grad_reducer_two_gpus():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _find_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    assert res == [(0, True), (1, True)]
