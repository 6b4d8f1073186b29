"""Hand-written CUDA kernels for sm_100a: building (`build`) and calling (`ops`)."""
from . import build, ops
from .ops import KernelError

__all__ = ["build", "ops", "KernelError"]
