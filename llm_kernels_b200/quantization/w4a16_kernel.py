"""Asymmetric group-128 int4 weights with bf16 activations (w4a16).

The reference's w4a16 is the dense symmetric "simple Marlin" kernel
(fast_dequant/simple_marlin/marlin_w4a16_gemm.cu:86-280, quantizer utils.py:98-136).  This module
extends that quantizer with a zero-point and bf16 scales, stores the nibbles in the order of
quantization/bitpack.py:38-67 (8 consecutive k per int32), and runs the matrix product on the
tcgen05 bf16 path after a CUDA expansion kernel."""
from typing import Tuple

import torch

from .. import _native as N


def weight_quant(w: torch.Tensor, groupsize: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """w [N,K] (nn.Linear layout) -> (packed int32 [N,K/8], scale bf16 [N,K/128], zero bf16 [N,K/128]).
    scale = (max-min)/15, zero = round(-min/scale), q = clamp(round(w/scale) + zero, 0, 15)."""
    N.require_cuda(w)
    assert w.dim() == 2 and groupsize == 128 and w.shape[1] % 128 == 0
    w = w.contiguous()
    Nn, K = w.shape
    packed = torch.empty(Nn, K // 8, dtype=torch.int32, device=w.device)
    scale = torch.empty(Nn, K // 128, dtype=torch.bfloat16, device=w.device)
    zero = torch.empty(Nn, K // 128, dtype=torch.bfloat16, device=w.device)
    N.check(N.lib().b200moe_weight_quant_w4a16(N.ptr(w), N.dtype_code(w.dtype), N.ptr(packed), N.ptr(scale),
                                               N.ptr(zero), Nn, K, N.stream()))
    return packed, scale, zero


def expand_bf16(packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """packed int32 [..., N, K/8] -> bf16 [..., N, K] = (q - zero) * scale."""
    N.require_cuda(packed, scale, zero)
    assert packed.is_contiguous() and scale.is_contiguous() and zero.is_contiguous()
    assert scale.dtype == torch.bfloat16 and zero.dtype == torch.bfloat16
    K = packed.shape[-1] * 8
    rows = packed.numel() // packed.shape[-1]
    out = torch.empty(*packed.shape[:-1], K, dtype=torch.bfloat16, device=packed.device)
    N.check(N.lib().b200moe_w4a16_expand_bf16(N.ptr(packed), N.ptr(scale), N.ptr(zero), N.ptr(out), rows, K, N.stream()))
    return out


def w4a16_gemm(a: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """c[..., N] = a[..., K] (bf16) . dequant(packed)^T, f32 accumulation."""
    from ..moe.group_gemm_kernel import grouped_gemm_bf16
    assert a.is_contiguous() and a.dtype == torch.bfloat16
    K = a.size(-1)
    M = a.numel() // K
    w = expand_bf16(packed, scale, zero)
    c = a.new_empty(*a.size()[:-1], w.shape[0], dtype=out_dtype)
    seg = torch.tensor([0, M], dtype=torch.int64, device=a.device)
    grouped_gemm_bf16(a.view(M, K), w.unsqueeze(0), seg, None, c.view(M, -1))
    return c
