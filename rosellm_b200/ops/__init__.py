"""Hand-written sm_100a kernels (``csrc/``) behind checked Python functions."""
from . import build, kernels

__all__ = ["build", "kernels"]
