"""B200-native (sm_100a) expert-parallel quantized MoE layer.

Python host code over a C-ABI CUDA library (include/b200moe.h).  The modules
under `moe/` and `quantization/` keep the names and call signatures of the
reference's moe/all2all_moe.py, moe/group_gemm_kernel.py,
quantization/fp8_kernel.py and quantization/bitpack.py.

There is no CPU path: importing is free, but every operator raises if the CUDA
library cannot be loaded or the tensors are not on a CUDA device.
"""
from . import _native  # noqa: F401

__all__ = ["_native"]
