"""n-bit pack / unpack of quantized weights; call surface of the reference's
quantization/bitpack.py (module-level aliases at :376-379)."""
from typing import Tuple

import torch

from .. import _native as N

_WORD = {8: torch.uint8, 16: torch.int16, 32: torch.int32}


def _check(W_nbits: int, packing_bitwidth: int):
    assert packing_bitwidth in [8, 16, 32], "Unsuported bitpacking width"
    assert W_nbits in [8, 4, 2, 1], "Unsuported nbits"


def _pack(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int, transpose: bool, over_rows: bool):
    _check(W_nbits, packing_bitwidth)
    N.require_cuda(W_q)
    assert W_q.dim() == 2
    w = W_q.to(torch.uint8).contiguous()
    e = packing_bitwidth // W_nbits
    R, Cc = w.shape
    shape = (R // e, Cc) if over_rows else (R, Cc // e)
    out = torch.empty(shape, dtype=_WORD[packing_bitwidth], device=w.device)
    N.check(N.lib().b200moe_pack_bits(N.ptr(w), N.ptr(out), R, Cc, W_nbits, packing_bitwidth,
                                      1 if over_rows else 0, N.stream()))
    return (out.t() if transpose else out), e


def pack_weights_over_rows(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int, transpose: bool = False) -> Tuple[torch.Tensor, int]:
    return _pack(W_q, W_nbits, packing_bitwidth, transpose, True)


def pack_weights_over_cols(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int, transpose: bool = False) -> Tuple[torch.Tensor, int]:
    return _pack(W_q, W_nbits, packing_bitwidth, transpose, False)


def _unpack(packed: torch.Tensor, W_nbits: int, n_out: int, dtype, over_rows: bool):
    N.require_cuda(packed)
    assert packed.dim() == 2 and packed.is_contiguous()
    width = packed.element_size() * 8
    _check(W_nbits, width)
    R, Cc = (n_out, packed.shape[1]) if over_rows else (packed.shape[0], n_out)
    out = torch.empty((R, Cc), dtype=torch.uint8, device=packed.device)
    N.check(N.lib().b200moe_unpack_bits(N.ptr(packed), N.ptr(out), R, Cc, W_nbits, width,
                                        1 if over_rows else 0, N.stream()))
    return out if dtype == torch.uint8 else out.to(dtype)


def unpack_over_rows(W_q_packed: torch.Tensor, W_nbits: int, num_output_rows: int, dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    return _unpack(W_q_packed, W_nbits, num_output_rows, dtype, True)


def unpack_over_cols(W_q_packed: torch.Tensor, W_nbits: int, num_output_cols: int, dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    return _unpack(W_q_packed, W_nbits, num_output_cols, dtype, False)
