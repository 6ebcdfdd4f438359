"""prism-b200: the Prism linear layer (forward + backward) as hand-written sm_100a kernels."""
from ._functional import forward, backward, check_device_status  # noqa: F401

__all__ = ["forward", "backward", "check_device_status"]
