"""Two-level int4 weights with int8 activations; call surface of the reference's
quantization/w4a8_kernel.py (weight_quant :265-309, weight_dequant :104-142, act_quant :171-193,
w4a8_gemm :406-448).

The GEMM expands the packed int4 weights to int8 with a CUDA kernel and runs the tcgen05 int8
GEMM with per-K-block f32 promotion.  weight_quant is one CUDA kernel (both levels and the packing).
"""
from typing import Tuple

import torch

from .. import _native as N
from . import int8_kernel

PACKING_BITS = 32
W_BITS = 4


def weight_quant(x: torch.Tensor, block_size: int = 128, group_size_int4: int = 128,
                 pack_direction: str = "row") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """x [M,N] -> (packed int32 [M/8,N], s f16 [M/128,N/128], s4 int8 [M,N/128], z4 int8 [M,N/128])."""
    N.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert x.dim() == 2, 'Input tensors must have 2 dimensions'
    assert block_size == 128 and group_size_int4 == 128
    assert x.size(-1) % block_size == 0, f'Last dimension size must be divisible by block_size (block_size={block_size})'
    assert pack_direction == "row", "Only row packing is supported"
    M, Nn = x.shape
    assert M % 128 == 0, 'row count must be divisible by 128'
    dev = x.device
    packed = torch.empty(M // (PACKING_BITS // W_BITS), Nn, dtype=torch.int32, device=dev)
    s = torch.empty(M // 128, Nn // 128, dtype=torch.float16, device=dev)
    s4 = torch.empty(M, Nn // 128, dtype=torch.int8, device=dev)
    z4 = torch.empty(M, Nn // 128, dtype=torch.int8, device=dev)
    N.check(N.lib().b200moe_weight_quant_w4a8(N.ptr(x), N.dtype_code(x.dtype), N.ptr(packed), N.ptr(s), N.ptr(s4),
                                              N.ptr(z4), M, Nn, N.stream()))
    return packed, s, s4, z4


def expand_int8(packed: torch.Tensor, s4: torch.Tensor, z4: torch.Tensor) -> torch.Tensor:
    """packed int32 [..., N/8, K] + s4/z4 int8 [..., N, K/128] -> int8 [..., N, K] (reference :44-101)."""
    N.require_cuda(packed, s4, z4)
    assert packed.is_contiguous() and s4.is_contiguous() and z4.is_contiguous()
    K = packed.shape[-1]
    Nn = packed.shape[-2] * 8
    W = packed.numel() // (packed.shape[-2] * K)
    out = torch.empty(*packed.shape[:-2], Nn, K, dtype=torch.int8, device=packed.device)
    N.check(N.lib().b200moe_w4a8_expand_int8(N.ptr(packed), N.ptr(s4), N.ptr(z4), N.ptr(out), W, Nn, K, N.stream()))
    return out


def weight_dequant(y: torch.Tensor, s: torch.Tensor, s4: torch.Tensor, z4: torch.Tensor, block_size: int = 128,
                   group_size_int4: int = 128, pack_direction: str = "row") -> torch.Tensor:
    assert pack_direction == "row", "Only row packing is supported for dequantization"
    w8 = expand_int8(y, s4, z4).float()
    M, Nn = w8.shape
    se = s.float().repeat_interleave(block_size, 0)[:M].repeat_interleave(block_size, 1)[:, :Nn]
    return (w8 * se).to(torch.float16)


def act_quant(x: torch.Tensor, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """int8 per 1x128 group, floor(v + 0.5) rounding, f16 scales (reference :171-193)."""
    return int8_kernel.act_quant(x, block_size, rounding="floor_half")


def w4a8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor, b_s4: torch.Tensor,
              b_z4: torch.Tensor, GROUP_SIZE_INT4: int = 128, elements_per_sample: int = 8,
              pack_direction: str = "row", out_dtype: torch.dtype = None) -> torch.Tensor:
    """c[..., N] = a[..., K] (int8) . dequant(b)^T with per-K-block scales (reference :406-448)."""
    from ..moe.group_gemm_kernel import grouped_gemm_i8
    assert a.is_contiguous() and b.is_contiguous(), 'Input tensors must be contiguous'
    assert a_s.is_contiguous() and b_s.is_contiguous(), 'Scaling factor tensors must be contiguous'
    assert b_s4.is_contiguous() and b_z4.is_contiguous(), 'Scaling factor and zero point tensors must be contiguous'
    assert pack_direction == "row" and GROUP_SIZE_INT4 == 128 and elements_per_sample == 8
    K = a.size(-1)
    M = a.numel() // K
    w8 = expand_int8(b, b_s4, b_z4)
    Nn = w8.shape[0]
    c = a.new_empty(*a.size()[:-1], Nn, dtype=out_dtype or torch.get_default_dtype())
    seg = torch.tensor([0, M], dtype=torch.int64, device=a.device)
    grouped_gemm_i8(a.view(M, K), a_s.reshape(M, -1).float(), w8.unsqueeze(0), b_s.float().unsqueeze(0), seg, None,
                    c.view(M, Nn))
    return c
