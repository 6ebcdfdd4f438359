"""prism-b200: the Prism linear layer (forward + backward) as hand-written sm_100a kernels.

Public surface (same names and argument meaning as the reference package ``cute_prism``):
``forward``, ``backward``, ``PrismLinear``; plus ``prism_linear`` (differentiable functional
form), ``check_device_status`` and the data-parallel helpers in ``cute_mma_b200._dp``.
"""
from ._functional import forward, backward, bias_grad, fold_weight, cayley, check_device_status  # noqa: F401
from ._functional import validate_kernel_params, validate_tensor_params  # noqa: F401
from ._module import PrismLinear, prism_linear, mup_fix_prism_shapes  # noqa: F401
from ._dp import PeerGradReducer, allreduce_grads, shard_rows, sync_module_grads  # noqa: F401

__all__ = ["forward", "backward", "bias_grad", "fold_weight", "cayley", "PrismLinear", "prism_linear", "mup_fix_prism_shapes",
           "validate_kernel_params", "validate_tensor_params", "check_device_status",
           "allreduce_grads", "shard_rows", "sync_module_grads"]
