"""fp8 e4m3 block quantization and blockwise GEMM.

Same call surface as the reference's quantization/fp8_kernel.py (act_quant :33-52,
weight_dequant :84-105, fp8_gemm :170-190) plus `weight_quant`, the 128x128 e4m3
weight quantizer the reference only ships for int8 (quantization/int8_kernel.py:91-113).
"""
from typing import Tuple

import torch

from .. import _native as N


def act_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-(1 x block_size) quantization: returns (y e4m3 same shape, s f32 [..., D/block_size])."""
    N.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert block_size == 128, 'block_size must be 128'
    assert x.size(-1) % block_size == 0, f'Last dimension size must be divisible by block_size (block_size={block_size})'
    y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = x.new_empty(*x.size()[:-1], x.size(-1) // block_size, dtype=torch.float32)
    cols = x.size(-1)
    rows = x.numel() // cols if cols else 0
    N.check(N.lib().b200moe_act_quant_fp8(N.ptr(x), N.dtype_code(x.dtype), rows, cols, N.ptr(y), cols,
                                          N.ptr(s), cols // block_size, N.stream()))
    return y, s


def weight_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128-block quantization of a 2-D weight: (y e4m3 [M,N], s f32 [ceil(M/128), ceil(N/128)])."""
    N.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert x.dim() == 2, 'Input tensors must have 2 dimensions'
    assert block_size == 128, 'block_size must be 128'
    M, Nn = x.size()
    y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = x.new_empty(((M + 127) // 128, (Nn + 127) // 128), dtype=torch.float32)
    N.check(N.lib().b200moe_weight_quant_fp8(N.ptr(x), N.dtype_code(x.dtype), N.ptr(y), N.ptr(s), M, Nn, N.stream()))
    return y, s


def weight_dequant(x: torch.Tensor, s: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """y = x * s[block] in the default dtype."""
    N.require_cuda(x, s)
    assert x.is_contiguous() and s.is_contiguous(), 'Input tensors must be contiguous'
    assert x.dim() == 2 and s.dim() == 2, 'Input tensors must have 2 dimensions'
    assert block_size == 128, 'block_size must be 128'
    M, Nn = x.size()
    y = torch.empty_like(x, dtype=torch.get_default_dtype())
    N.check(N.lib().b200moe_weight_dequant_fp8(N.ptr(x), N.ptr(s.float() if s.dtype != torch.float32 else s),
                                               N.ptr(y), N.dtype_code(y.dtype), M, Nn, N.stream()))
    return y


_partials = {}


def _split_k(M: int, Nn: int, K: int) -> int:
    """K splits for a small-M product: enough tiles to occupy the 148 SMs, every split non-empty."""
    if M > 128:
        return 1
    tiles = -(-M // 128) * -(-Nn // 256)
    kb = K // 128
    ks = max(1, min(8, 148 // tiles, kb))
    while ks > 1 and -(-kb // ks) * (ks - 1) >= kb:
        ks -= 1
    return ks


def fp8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor,
             out_dtype: torch.dtype = None, ksplits: int = None) -> torch.Tensor:
    """c[..., N] = a[..., K] . b[N, K]^T with 1x128 / 128x128 f32 block scales, in the
    default dtype unless out_dtype is given (tcgen05 kernel).  ksplits (None = chosen from the shape):
    M <= 128 splits the K loop over several sets of tiles whose f32 partial products are added in
    split order by a second kernel, so that the weights stream on all SMs."""
    N.require_cuda(a, a_s, b, b_s)
    assert a.is_contiguous() and b.is_contiguous(), 'Input tensors must be contiguous'
    assert a_s.is_contiguous() and b_s.is_contiguous(), 'Scaling factor tensors must be contiguous'
    assert a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn, 'operands must be float8_e4m3fn'
    assert a_s.dtype == torch.float32 and b_s.dtype == torch.float32, 'scales must be float32'
    K = a.size(-1)
    M = a.numel() // K
    Nn = b.size(0)
    c = a.new_empty(*a.size()[:-1], Nn, dtype=out_dtype or torch.get_default_dtype())
    ks = _split_k(M, Nn, K) if ksplits is None else int(ksplits)
    if ks > 1 and M > 0:
        key = (a.device, torch.cuda.current_stream(a.device).cuda_stream)
        part = _partials.get(key)
        if part is None or part.numel() < ks * M * Nn:
            part = _partials[key] = torch.empty(ks * M * Nn, dtype=torch.float32, device=a.device)
        N.check(N.lib().b200moe_gemm_fp8_block_splitk(N.ptr(a), N.ptr(a_s), N.ptr(b), N.ptr(b_s), N.ptr(c),
                                                      N.dtype_code(c.dtype), M, Nn, K, ks, N.ptr(part),
                                                      part.numel() * 4, N.stream()))
        return c
    N.check(N.lib().b200moe_gemm_fp8_block(N.ptr(a), N.ptr(a_s), N.ptr(b), N.ptr(b_s), N.ptr(c),
                                           N.dtype_code(c.dtype), M, Nn, K, N.stream()))
    return c
