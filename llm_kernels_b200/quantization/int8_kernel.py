"""int8 per-token-group activation quantizer (reference: quantization/int8_kernel.py:34-56;
with rounding='floor_half' the variant of quantization/w4a8_kernel.py:171-193)."""
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
