"""Symmetric int4 weight-only GEMM in Marlin order (reference: fast_dequant/simple_marlin/)."""
from .marlin_cuda import mul  # noqa: F401
from .utils import QuantUtils  # noqa: F401
