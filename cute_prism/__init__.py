"""``cute_prism``: the reference package's import name, served by the sm_100a kernels.

A model or script written against the reference (``import cute_prism``;
``cute_prism.forward / backward / PrismLinear``; ``torch.ops.cute_prism.forward / backward``)
runs unedited on top of ``cute_mma_b200``.  There is one backend: ``backend=``, ``comp_params=``,
``autotuning=`` and the other tuning keywords of the reference are accepted and ignored, the
compile / autotune cache helpers are no-ops, and what the accelerated path does not cover raises
``ValueError`` (see ``cute_mma_b200._functional``).

The custom ops registered here have the reference's schemas
(src/cute_prism/_module.py:38-141): ``cute_prism::forward(A, B, R, group_size, reconn_sz, backend,
activation, autotuning, force_rebenchmark) -> C`` and ``cute_prism::backward(dC, A, B, R, ...) ->
(dA, dR, dB)`` with the frozen-B contract of the plain mode (dB is returned as zeros).
"""
from __future__ import annotations

import torch

import cute_mma_b200 as _impl
from cute_mma_b200 import (PrismLinear, backward, forward, mup_fix_prism_shapes,  # noqa: F401
                           validate_kernel_params, validate_tensor_params)

BACKENDS = ("cute", "cublas", "pytorch")   # accepted, all served by the one sm_100a backend
MODES = ("ar", "rw")
ACTIVATIONS = (None, "silu_gate", "sigmoid_gate")


class CompilationError(RuntimeError):
    """Kept for ``except cute_prism.CompilationError``: nothing is compiled at run time here."""


def clear_cache() -> None:
    """No-op: the kernels are built ahead of time, there is no JIT cache."""


def clear_autotune_cache() -> None:
    """No-op: launch parameters come from the shipped tile table, not from an autotuner."""


def get_autotune_cache() -> dict:
    return {}


@torch.library.custom_op("cute_prism::forward", mutates_args=())
def _forward_op(A: torch.Tensor, B: torch.Tensor, R: torch.Tensor, group_size: int, reconn_sz: int,
                backend: str, activation: str, autotuning: bool, force_rebenchmark: bool) -> torch.Tensor:
    C, _ = _impl.forward(A.contiguous(), B.contiguous(), R.contiguous(), group_size, reconn_sz,
                         activation=activation or None)
    return C


@_forward_op.register_fake
def _(A, B, R, group_size, reconn_sz, backend, activation, autotuning, force_rebenchmark):
    return A.new_empty(A.shape[0], B.shape[0])


@torch.library.custom_op("cute_prism::backward", mutates_args=())
def _backward_op(dC: torch.Tensor, A: torch.Tensor, B: torch.Tensor, R: torch.Tensor, group_size: int,
                 reconn_sz: int, backend: str, activation: str, autotuning: bool,
                 force_rebenchmark: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dA, dR, dB, _ = _impl.backward(dC.contiguous(), A.contiguous(), B.contiguous(), R.contiguous(),
                                   group_size, reconn_sz, activation=activation or None)
    if dB is None:   # plain mode: B is the frozen pretrained weight
        dB = torch.zeros_like(B)
    return dA, dR, dB


@_backward_op.register_fake
def _(dC, A, B, R, group_size, reconn_sz, backend, activation, autotuning, force_rebenchmark):
    return A.new_empty(A.shape), R.new_empty(R.shape), B.new_empty(B.shape)


def _setup_context(ctx, inputs, output):
    A, B, R, ctx.group_size, ctx.reconn_sz, _backend, ctx.activation, _at, _fr = inputs
    ctx.save_for_backward(A, B, R)


def _op_backward(ctx, dC):
    A, B, R = ctx.saved_tensors
    dA, dR, dB = _backward_op(dC, A, B, R, ctx.group_size, ctx.reconn_sz, "cute", ctx.activation, False, False)
    return dA, dB, dR, None, None, None, None, None, None


_forward_op.register_autograd(_op_backward, setup_context=_setup_context)

__all__ = ["forward", "backward", "PrismLinear", "mup_fix_prism_shapes", "validate_kernel_params",
           "validate_tensor_params", "clear_cache", "clear_autotune_cache", "get_autotune_cache",
           "CompilationError", "BACKENDS", "MODES", "ACTIVATIONS"]
