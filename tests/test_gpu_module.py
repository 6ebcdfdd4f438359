"""PrismLinear / custom-op autograd wiring on the GPU against torch autograd of the oracle."""
import pytest
import torch

import cute_mma_b200 as cp
from oracle import prism_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-2
DEV = "cuda"


def _oracle_module(layer, x):
    """fp32 autograd restatement of PrismLinear.forward, with the reference's backward rescale."""
    A = x.reshape(-1, layer.in_features).float().detach().requires_grad_(True)
    W = layer.weight.float().detach().requires_grad_(True)
    reconn = layer.reconn.float().detach().requires_grad_(True)
    b = layer.bias.float().detach().requires_grad_(True) if layer.bias is not None else None
    if layer.activation == "silu_gate":
        R = reconn
    else:
        G, r, nb = layer.out_features // layer.group_size, layer.reconn_sz, layer.in_features // layer.reconn_sz
        Mb = reconn.reshape(G, r, nb, r).permute(0, 2, 1, 3)
        S = Mb - Mb.transpose(-1, -2)
        eye = torch.eye(r, device=S.device).expand_as(S)
        R = torch.linalg.solve(eye - S, eye + S).permute(0, 2, 1, 3).reshape(G * r, layer.in_features)
    C = O.prism_forward(A, W, R, layer.group_size, layer.reconn_sz, layer.activation)
    scale = layer._bwd_scale
    C = C * scale + (C * (1 - scale)).detach()  # identity forward, gradient scaled
    if b is not None:
        C = C + b
    return C, A, W, reconn, b


@pytest.mark.parametrize("act", [None, "silu_gate"])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_module_forward_backward(act, dt):
    torch.manual_seed(0)
    layer = cp.PrismLinear(256, 512, group_size=256, reconn_sz=8, activation=act).to(DEV)
    if act is None:
        with torch.no_grad():
            layer.reconn.normal_(0, 0.05)
    layer = layer.to(dt)
    x = torch.randn(4, 96, 256, device=DEV).to(dt).requires_grad_(True)
    y = layer(x)
    assert y.shape == (4, 96, 512) and y.dtype == dt
    dy = torch.randn_like(y)
    y.backward(dy)
    cp.check_device_status()
    ry, rA, rW, rreconn, rb = _oracle_module(layer, x)
    ry.backward(dy.reshape(-1, 512).float())
    assert O.rel_err(y.reshape(-1, 512).float(), ry) < TOL
    assert O.rel_err(x.grad.reshape(-1, 256).float(), rA.grad) < TOL
    assert O.rel_err(layer.reconn.grad.float(), rreconn.grad) < 3e-2   # through the Cayley solve in plain mode
    assert O.rel_err(layer.bias.grad.float(), rb.grad) < TOL
    if act is None:
        assert layer.weight.grad is None            # frozen B gets no gradient tensor
    else:
        assert O.rel_err(layer.weight.grad.float(), rW.grad) < TOL


def test_plain_mode_trainable_B_gets_exact_zeros():
    """The reference's frozen-B contract (src/cute_prism/_module.py:92-104,
    tests/test_module_integration.py:123-130)."""
    A = torch.randn(128, 64, device=DEV).half().requires_grad_(True)
    B = torch.randn(64, 64, device=DEV).half().requires_grad_(True)
    R = torch.eye(8, device=DEV).repeat(2, 8).half().requires_grad_(True)
    C = cp.prism_linear(A, B, R, None, 32, 8, None)
    C.sum().backward()
    assert B.grad is not None and B.grad.abs().max() == 0
    assert A.grad is not None and R.grad is not None


def test_from_linear_reproduces_linear():
    lin = torch.nn.Linear(256, 512).to(DEV).half()
    layer = cp.PrismLinear.from_linear(lin, group_size=128, reconn_sz=16)
    x = torch.randn(200, 256, device=DEV).half()
    assert O.rel_err(layer(x).float(), lin(x).float()) < 5e-3


def test_torch_compile_fullgraph():
    layer = cp.PrismLinear(128, 256, group_size=128, reconn_sz=16, activation="silu_gate").to(DEV).to(torch.bfloat16)
    x = torch.randn(64, 128, device=DEV, dtype=torch.bfloat16)
    ref = layer(x)
    out = torch.compile(layer, fullgraph=True, backend="eager")(x)
    assert torch.equal(out, ref)
