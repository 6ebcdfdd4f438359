"""``PrismLinear`` and the autograd wiring of the sm_100a Prism kernels.

Mirrors the reference module (src/cute_prism/_module.py): the custom ops with fake
implementations (lines 38-141), the constant backward rescale of the gated layer
(``_BwdScaleFn``, lines 20-30 and 462-470), parameter names / shapes / initialisation
(lines 415-532), the Cayley construction of R in fine-tuning mode (lines 534-577),
``load_pretrained_weight`` / ``from_linear`` (lines 599-688) and ``forward`` (lines 690-739).

Differences, all on the fast path:
* the output bias is added in the forward kernel's epilogue instead of a separate op;
* the backward rescale is passed to the backward kernels as ``dc_scale`` instead of an extra
  pass over dC (the bias gradient, taken after the rescale point, stays unscaled as in the
  reference) and the bias gradient is a fixed-order column sum kernel of the library;
* in plain mode a frozen ``weight`` gets no gradient tensor at all; a trainable ``weight``
  in plain mode gets exact zeros, which is the reference's contract
  (src/cute_prism/_module.py:92-104);
* the exact Cayley transform of CUDA parameters with ``reconn_sz`` 8 or 16 is one launch of the
  library's batched kernel (fp32 inside, its own backward); elsewhere it is solved by
  ``torch.linalg.solve`` in fp32 for fp16/bf16 parameters (which has no 16-bit kernels) and cast back;
* the internal bias (``internal_bias=True``, gated modes) is added inside the kernels and its gradient
  comes out of the dA+dR kernel; ``dropout`` (gated modes, training) is the reference kernels' hash
  dropout, regenerated in the backward from per-group seeds;
* ``input_shuffle=True`` (``reconn_sz`` 16, chunks of 64 features, no dropout) builds the reference's per-group
  butterfly masks and folds every group's permutation into a 64-wide rotation and a column order of the
  weight (``_shuffle``): the same kernels, no per-group copy of the input.
"""
from __future__ import annotations

import math
from typing import Literal

import torch
import torch.nn as nn

from . import _functional as F

_GATED_SILU_BWD_GAIN = 1.437     # same constants as the reference (src/cute_prism/_module.py:14-15)
_GATED_SIGMOID_BWD_GAIN = 1.15
_GATED = ("silu_gate", "sigmoid_gate")


def gated_name(activation) -> bool:
    return activation in _GATED


# ---------------------------------------------------------------------------
# custom ops: opaque to torch.compile, with fake-tensor and autograd support
# ---------------------------------------------------------------------------
@torch.library.custom_op("prism_b200::forward", mutates_args=())
def _prism_forward_op(A: torch.Tensor, B: torch.Tensor, R: torch.Tensor, bias: torch.Tensor | None,
                      group_size: int, reconn_sz: int, activation: str, bwd_scale: float,
                      internal_bias: torch.Tensor | None = None,
                      dropout_seeds: torch.Tensor | None = None, dropout_p: float = 0.0) -> torch.Tensor:
    C, _ = F.forward(A.contiguous(), B.contiguous(), R.contiguous(), group_size, reconn_sz,
                     activation=activation or None, bias=bias, internal_bias=internal_bias,
                     dropout_p=dropout_p, training=dropout_seeds is not None, dropout_seeds=dropout_seeds)
    return C


@_prism_forward_op.register_fake
def _(A, B, R, bias, group_size, reconn_sz, activation, bwd_scale, internal_bias=None, dropout_seeds=None,
      dropout_p=0.0):
    return A.new_empty(A.shape[0], B.shape[0])


@torch.library.custom_op("prism_b200::backward", mutates_args=())
def _prism_backward_op(dC: torch.Tensor, A: torch.Tensor, B: torch.Tensor, R: torch.Tensor,
                       group_size: int, reconn_sz: int, activation: str, bwd_scale: float,
                       need_dB: bool, need_dbias: bool, internal_bias: torch.Tensor | None = None,
                       dropout_seeds: torch.Tensor | None = None, dropout_p: float = 0.0
                       ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    dC = dC.contiguous()
    A, B, R = A.contiguous(), B.contiguous(), R.contiguous()
    gate = F._gate_code(activation or None)
    ib = internal_bias.contiguous() if internal_bias is not None else None
    out = F._backward_dadr(dC, A, B, R, group_size, reconn_sz, gate, bwd_scale, internal_bias=ib,
                           dropout_seeds=dropout_seeds, dropout_p=dropout_p)
    dA, dR = out[0], out[1]
    d_ib = out[2] if ib is not None else dC.new_empty(0)
    if not need_dB:
        dB = B.new_empty(0)
    elif gate:
        dB = F._backward_db(dC, A, R, group_size, reconn_sz, gate, bwd_scale, internal_bias=ib,
                            dropout_seeds=dropout_seeds, dropout_p=dropout_p)
    else:
        dB = torch.zeros_like(B)  # frozen-B contract of the reference's plain mode
    # the bias is added after the rescale point: its gradient is the plain column sum of dC
    dbias = F.bias_grad(dC) if need_dbias else dC.new_empty(0)
    return dA, dR, dB, dbias, d_ib


@_prism_backward_op.register_fake
def _(dC, A, B, R, group_size, reconn_sz, activation, bwd_scale, need_dB, need_dbias, internal_bias=None,
      dropout_seeds=None, dropout_p=0.0):
    return (A.new_empty(A.shape), R.new_empty(R.shape), (B.new_empty(B.shape) if need_dB else B.new_empty(0)),
            (dC.new_empty(dC.shape[1]) if need_dbias else dC.new_empty(0)),
            (internal_bias.new_empty(internal_bias.shape) if internal_bias is not None else dC.new_empty(0)))


@torch.library.custom_op("prism_b200::cayley", mutates_args=())
def _cayley_op(M: torch.Tensor, reconn_sz: int) -> torch.Tensor:
    return F.cayley(M, reconn_sz)


@_cayley_op.register_fake
def _(M, reconn_sz):
    return M.new_empty(M.shape)


@torch.library.custom_op("prism_b200::cayley_backward", mutates_args=())
def _cayley_bwd_op(M: torch.Tensor, dR: torch.Tensor, reconn_sz: int) -> torch.Tensor:
    return F.cayley_backward(M, dR, reconn_sz)


@_cayley_bwd_op.register_fake
def _(M, dR, reconn_sz):
    return M.new_empty(M.shape)


def _cayley_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])
    ctx.reconn_sz = inputs[1]


def _cayley_backward(ctx, dR):
    (M,) = ctx.saved_tensors
    return _cayley_bwd_op(M, dR, ctx.reconn_sz), None


_cayley_op.register_autograd(_cayley_backward, setup_context=_cayley_setup)


def _setup_context(ctx, inputs, output):
    A, B, R, bias, group_size, reconn_sz, activation, bwd_scale, internal_bias, dropout_seeds, dropout_p = inputs
    ctx.save_for_backward(A, B, R, *(() if internal_bias is None else (internal_bias,)))
    ctx.has_ib = internal_bias is not None
    ctx.dropout_seeds, ctx.dropout_p = dropout_seeds, dropout_p
    ctx.has_bias = bias is not None
    ctx.group_size, ctx.reconn_sz = group_size, reconn_sz
    ctx.activation, ctx.bwd_scale = activation, bwd_scale


def _backward(ctx, dC):
    A, B, R = ctx.saved_tensors[:3]
    ib = ctx.saved_tensors[3] if ctx.has_ib else None
    need_dB = bool(ctx.needs_input_grad[1])
    need_dbias = bool(ctx.has_bias and ctx.needs_input_grad[3])
    dA, dR, dB, dbias, d_ib = _prism_backward_op(dC, A, B, R, ctx.group_size, ctx.reconn_sz, ctx.activation,
                                                 ctx.bwd_scale, need_dB, need_dbias, ib, ctx.dropout_seeds,
                                                 ctx.dropout_p)
    return (dA, (dB if need_dB else None), dR, (dbias if need_dbias else None), None, None, None, None,
            (d_ib if ctx.has_ib else None), None, None)


_prism_forward_op.register_autograd(_backward, setup_context=_setup_context)


def prism_linear(A, B, R, bias=None, group_size=256, reconn_sz=8, activation=None, bwd_scale=1.0,
                 internal_bias=None, dropout_seeds=None, dropout_p=0.0):
    """Differentiable functional form: C = prism(A, B, R) + bias; gradients of A/B/R (and of the
    internal bias) are multiplied by ``bwd_scale`` (the output-bias gradient is not).  ``dropout_seeds``
    (int64, one per group) switches the hash dropout of the gated activation on."""
    return _prism_forward_op(A, B, R, bias, group_size, reconn_sz, activation or "", float(bwd_scale), internal_bias,
                             dropout_seeds, float(dropout_p))


# ---------------------------------------------------------------------------
# module
# ---------------------------------------------------------------------------
class PrismLinear(nn.Module):
    """Drop-in for the reference ``cute_prism.PrismLinear`` on the accelerated path.

    ``C = (A . blockdiag(R_g)^T) @ B_g^T`` per output group (``activation=None``: B frozen, R is
    the Cayley transform of the skew-symmetric part of ``reconn``), or
    ``C = (A * silu(A . blockdiag(R_g)^T)) @ B_g^T`` (``activation="silu_gate"``; ``"sigmoid_gate"`` uses
    ``2 sigmoid`` in place of ``silu``: B and R trained, R = ``reconn``).  Parameter names and shapes match the reference, so its checkpoints load:
    ``weight (N, K)``, ``reconn (N/group_size*reconn_sz, K)``, ``bias (N)``, optional ``ar_scale``.
    """

    def __init__(self, in_features: int, out_features: int, group_size: int = 256, reconn_sz: int = 8,
                 bias: bool = True, activation: Literal["silu_gate"] | None = None,
                 cayley_order: int | float = float("inf"), input_shuffle: bool = False,
                 shuffle_blk_k: int = 64, backend: str | None = None, autotuning: bool = False,
                 force_rebenchmark: bool = False, comp_params=None, bwd_dadr_params=None,
                 bwd_db_params=None, internal_bias: bool = False, dropout: float = 0.0,
                 r_init_scale=1.0, ar_scale_init: float | None = None):
        super().__init__()
        if activation not in (None,) + _GATED:
            raise ValueError(f"Unknown activation {activation!r}, must be one of (None, 'silu_gate', 'sigmoid_gate')")
        if input_shuffle:
            # reference: src/cute_prism/_module.py:368-375; here additionally chunks of 64 features and no dropout
            if reconn_sz != 16:
                raise ValueError("input_shuffle requires reconn_sz=16")
            if shuffle_blk_k != 64:
                raise ValueError("input_shuffle is built for shuffle_blk_k=64")
            if in_features % shuffle_blk_k != 0:
                raise ValueError(f"in_features ({in_features}) must be divisible by shuffle_blk_k ({shuffle_blk_k})")
            if dropout > 0.0:
                raise ValueError("input_shuffle together with dropout is not supported by the sm_100a kernels")
        if dropout > 0.0 and gated_name(activation) and reconn_sz not in (8, 16):
            raise ValueError("dropout is supported for reconn_sz 8 and 16")
        self.dropout = float(dropout)
        if out_features % group_size != 0:
            raise ValueError(f"out_features ({out_features}) must be divisible by group_size ({group_size})")
        if in_features % reconn_sz != 0:
            raise ValueError(f"in_features ({in_features}) must be divisible by reconn_sz ({reconn_sz})")
        F.validate_kernel_params(group_size, reconn_sz)

        self.in_features, self.out_features = in_features, out_features
        self.group_size, self.reconn_sz = group_size, reconn_sz
        self.input_shuffle, self.shuffle_blk_k = bool(input_shuffle), shuffle_blk_k
        self._shuffle_fold = None
        if input_shuffle:
            from ._shuffle import build_shuffle_masks
            masks, self._shuffle_deltas = build_shuffle_masks(in_features, out_features, group_size, reconn_sz, shuffle_blk_k)
            self.register_buffer("_shuffle_masks", masks)
        self.activation = activation
        self.cayley_order = cayley_order
        self.r_init_scale = r_init_scale
        # accepted for signature compatibility; there is one backend and no autotuner
        self.backend, self.autotuning, self.force_rebenchmark = backend, autotuning, force_rebenchmark

        gated = activation in _GATED
        n_groups = out_features // group_size
        self.weight = nn.Parameter(torch.empty(out_features, in_features), requires_grad=gated)
        self.reconn = nn.Parameter(torch.empty(n_groups * reconn_sz, in_features))
        if ar_scale_init is not None:
            self.ar_scale = nn.Parameter(torch.tensor(float(ar_scale_init)))
        else:
            self.register_parameter("ar_scale", None)
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        # bias added to A . blockdiag(R_g)^T before the gate (gated modes only), one row per group
        if internal_bias and gated:
            self._internal_bias = nn.Parameter(torch.empty(n_groups, in_features))
        else:
            self.register_parameter("_internal_bias", None)
        self._bwd_scale = {"silu_gate": 1.0 / _GATED_SILU_BWD_GAIN, "sigmoid_gate": 1.0 / _GATED_SIGMOID_BWD_GAIN}.get(activation, 1.0)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Same initialisation as the reference (src/cute_prism/_module.py:474-532)."""
        K, r = self.in_features, self.reconn_sz
        nn.init.normal_(self.weight, std=1.0 / math.sqrt(K))
        if self.activation in _GATED:
            n_groups = self.out_features // self.group_size
            sigma = 4.0 / math.sqrt(2 * (r - (2 if self._internal_bias is not None else 1))) * self.r_init_scale
            Mb = torch.randn(n_groups, K // r, r, r, device=self.reconn.device, dtype=self.reconn.dtype) * sigma
            S = Mb - Mb.transpose(-1, -2)
            with torch.no_grad():
                self.reconn.copy_(S.permute(0, 2, 1, 3).reshape(n_groups * r, K))
        else:
            nn.init.zeros_(self.reconn)
        if self.bias is not None:
            bound = 1 / math.sqrt(K) if K > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)
        if self._internal_bias is not None:
            nn.init.normal_(self._internal_bias, std=1.0 / math.sqrt(r - 1))

    def _build_R(self) -> torch.Tensor:
        """R from the stored parameter (reference: src/cute_prism/_module.py:534-577)."""
        if self.activation in _GATED:
            return self.reconn if self.ar_scale is None else self.ar_scale * self.reconn
        n_groups = self.out_features // self.group_size
        r = self.reconn_sz
        nb = self.in_features // r
        out_dtype = self.reconn.dtype
        if self.cayley_order == float("inf") and F.cayley_supported(self.reconn, r):
            # the library's batched Cayley kernel: one launch, fp32 inside, any parameter dtype,
            # differentiable, capturable in a CUDA graph
            return _cayley_op(self.reconn, r)
        Mb = self.reconn.reshape(n_groups, r, nb, r).permute(0, 2, 1, 3)
        if out_dtype in (torch.float16, torch.bfloat16):
            Mb = Mb.float()
        S = Mb - Mb.transpose(-1, -2)
        eye = torch.eye(r, device=S.device, dtype=S.dtype).expand_as(S)
        if self.cayley_order == float("inf"):
            Rb = torch.linalg.solve(eye - S, eye + S)
        else:
            Rb = eye.clone()
            Sp = S
            for _ in range(int(self.cayley_order)):
                Rb = Rb + 2 * Sp
                Sp = Sp @ S
        return Rb.permute(0, 2, 1, 3).reshape(n_groups * r, self.in_features).to(out_dtype)

    def reconn_diag_sq_sum(self) -> torch.Tensor:
        """Sum over all rotation blocks of the squared diagonal entries of R (a scalar tensor):
        0 for skew-symmetric blocks, about ``n_groups * n_blocks * reconn_sz`` for orthogonal
        blocks close to the identity (reference: src/cute_prism/_module.py:579-597)."""
        r = self.reconn_sz
        R = self._build_R().reshape(self.out_features // self.group_size, r, self.in_features // r, r)
        return torch.diagonal(R, dim1=1, dim2=3).pow(2).sum()

    def load_pretrained_weight(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        if weight.shape != self.weight.shape:
            raise ValueError(f"Weight shape mismatch: expected {self.weight.shape}, got {weight.shape}")
        with torch.no_grad():
            self.weight.copy_(weight)
        if bias is not None:
            if self.bias is None:
                raise ValueError("This layer has no bias, but bias was provided")
            if bias.shape != self.bias.shape:
                raise ValueError(f"Bias shape mismatch: expected {self.bias.shape}, got {bias.shape}")
            with torch.no_grad():
                self.bias.copy_(bias)

    @classmethod
    def from_linear(cls, linear: nn.Linear, group_size: int = 256, reconn_sz: int = 8, activation=None,
                    backend=None, autotuning: bool = False, **kwargs) -> "PrismLinear":
        layer = cls(linear.in_features, linear.out_features, group_size=group_size, reconn_sz=reconn_sz,
                    bias=linear.bias is not None, activation=activation, backend=backend,
                    autotuning=autotuning, **kwargs)
        layer.to(device=linear.weight.device, dtype=linear.weight.dtype)
        layer.load_pretrained_weight(linear.weight.data, linear.bias.data if linear.bias is not None else None)
        return layer

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        A = input.reshape(-1, self.in_features)
        seeds = None
        if self.training and self.dropout > 0.0 and self.activation in _GATED:
            # one seed per group and call; forward and backward regenerate the mask from them
            seeds = torch.randint(1, 1 << 62, (self.out_features // self.group_size,), dtype=torch.int64,
                                  device=A.device)
        weight, R, rs, ib = self.weight, self._build_R(), self.reconn_sz, self._internal_bias
        if self.input_shuffle:
            # every group's permutation of the input features, folded into the parameters: a 64-wide rotation
            # on the same kernels (``_shuffle``); autograd carries dR, dB and the bias gradient back through the fold
            fold = self._shuffle_fold
            if fold is None or fold.perm.device != A.device:
                from ._shuffle import ShuffleFold
                fold = self._shuffle_fold = ShuffleFold(self._shuffle_masks, self.in_features, self.group_size,
                                                        self.reconn_sz, A.device)
            weight, R, rs = fold.fold_cols(weight, self.group_size), fold.fold_R(R), 64
            ib = None if ib is None else fold.fold_cols(ib, 1)
        C = _prism_forward_op(A, weight, R, self.bias, self.group_size, rs,
                              self.activation or "", float(self._bwd_scale), ib, seeds,
                              self.dropout)
        return C.reshape(input.shape[:-1] + (self.out_features,))

    def extra_repr(self) -> str:
        parts = [f"in_features={self.in_features}", f"out_features={self.out_features}",
                 f"group_size={self.group_size}", f"reconn_sz={self.reconn_sz}",
                 f"bias={self.bias is not None}"]
        if self._internal_bias is not None:
            parts.append("internal_bias=True")
        if self.input_shuffle:
            parts.append(f"input_shuffle=True, shuffle_blk_k={self.shuffle_blk_k}")
        if self.activation is not None:
            parts.append(f"activation={self.activation!r}")
        else:
            parts.append(f"cayley_order={self.cayley_order}")
        return ", ".join(parts)


def mup_fix_prism_shapes(model: nn.Module) -> None:
    """For models set up with the ``mup`` package: give the ``reconn`` parameter of every
    ``PrismLinear`` a width multiplier of 1, because a rotation block's fan-in is ``reconn_sz``
    whatever the model width (reference: src/cute_prism/_module.py:806-870).  Call it after
    ``mup.set_base_shapes`` and before the optimizer is built; needs ``mup`` installed."""
    from mup.infshape import InfDim, InfShape

    for module in model.modules():
        if not isinstance(module, PrismLinear):
            continue
        p = module.reconn
        if hasattr(p, "infshape"):
            dims = list(p.infshape)
            dims[-1] = InfDim(dims[-1].dim, dims[-1].dim)
            p.infshape = InfShape(dims)
