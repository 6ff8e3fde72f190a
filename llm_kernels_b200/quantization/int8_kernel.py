"""int8 blockwise quantizers with the call surface of the reference's quantization/int8_kernel.py:
act_quant (:34-56; with rounding='floor_half' the variant of quantization/w4a8_kernel.py:171-193),
weight_quant (:91-113) and weight_dequant (:145-170), as CUDA kernels."""
from typing import Tuple

import torch

from .. import _native as N


def act_quant(x: torch.Tensor, block_size: int = 128, rounding: str = "half_away") -> Tuple[torch.Tensor, torch.Tensor]:
    N.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert block_size == 128, 'block_size must be 128'
    assert x.size(-1) % block_size == 0, f'Last dimension size must be divisible by block_size (block_size={block_size})'
    y = torch.empty_like(x, dtype=torch.int8)
    s = x.new_empty(*x.size()[:-1], x.size(-1) // block_size, dtype=torch.float16)
    cols = x.size(-1)
    rows = x.numel() // cols if cols else 0
    N.check(N.lib().b200moe_act_quant_int8(N.ptr(x), N.dtype_code(x.dtype), rows, cols, N.ptr(y), N.ptr(s),
                                           {"half_away": 0, "floor_half": 1}[rounding], N.stream()))
    return y, s


def weight_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M,N] -> (int8 [M,N], f16 scales [ceil(M/128), ceil(N/128)]); per block s = amax/127,
    y = round-half-away(x / s) (reference :59-113)."""
    N.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert x.dim() == 2, 'Input tensors must have 2 dimensions'
    assert block_size == 128, 'block_size must be 128'
    M, Nn = x.size()
    y = torch.empty_like(x, dtype=torch.int8)
    s = x.new_empty(((M + block_size - 1) // block_size, (Nn + block_size - 1) // block_size), dtype=torch.float16)
    N.check(N.lib().b200moe_weight_quant_int8(N.ptr(x), N.dtype_code(x.dtype), N.ptr(y), N.ptr(s), M, Nn, 127.0, 0,
                                              N.stream()))
    return y, s


def weight_dequant(x: torch.Tensor, s: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """y = x * s[i/128, j/128] in the default dtype (reference :145-170)."""
    N.require_cuda(x, s)
    assert x.is_contiguous() and s.is_contiguous(), 'Input tensors must be contiguous'
    assert x.dim() == 2 and s.dim() == 2, 'Input tensors must have 2 dimensions'
    assert block_size == 128 and x.dtype == torch.int8 and s.dtype == torch.float16
    M, Nn = x.size()
    y = torch.empty_like(x, dtype=torch.get_default_dtype())
    N.check(N.lib().b200moe_weight_dequant_int8(N.ptr(x), N.ptr(s), N.ptr(y), N.dtype_code(y.dtype), M, Nn, N.stream()))
    return y
