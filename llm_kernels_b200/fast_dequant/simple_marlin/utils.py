"""Offline int4 quantization and Marlin-order packing (reference: fast_dequant/simple_marlin/utils.py).

`QuantUtils.fake_quantize` and `QuantUtils.pack` keep the reference's signatures and produce the same
tensors bit for bit.  `pack` of CUDA tensors is a CUDA kernel; host tensors are packed on the host with
torch ops, as the reference packs them through numpy."""
from typing import List, Tuple

import torch


def _get_perms() -> Tuple[torch.Tensor, List[int], List[int]]:
    """utils.py:20-46.  perm[i] = index, inside a block of four 16x16 tiles stored tile-major, of the
    element that packed position i holds: positions are ordered so that the eight nibbles of one int32
    are the values one tensor-core lane consumes, with even/odd nibbles interleaved."""
    lane_rows = lambda q: (2 * q, 2 * q + 1, 2 * (q + 4), 2 * (q + 4) + 1)
    perm = []
    for lane in range(32):
        col, quad = divmod(lane, 4)
        one_tile = [16 * row + col + 8 * half for half in (0, 1) for row in lane_rows(quad)]
        for tile in range(4):
            perm += [256 * tile + p for p in one_tile]
    perm = torch.tensor(perm, dtype=torch.int64).view(-1, 8)[:, [0, 2, 4, 6, 1, 3, 5, 7]].reshape(-1)
    scale_perm = [i + 8 * j for i in range(8) for j in range(8)]
    scale_perm_single = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return perm, scale_perm, scale_perm_single


_perm, _scale_perm, _scale_perm_single = _get_perms()


def scale_perm_for(groupsize: int) -> List[int]:
    return _scale_perm if groupsize != -1 else _scale_perm_single


class QuantUtils:

    @staticmethod
    def pack(weight: torch.Tensor, scale: torch.Tensor, groupsize: int = -1) -> tuple:
        """utils.py:53-95.  weight int32 [K, N] with values 0..15, scale [K/groupsize, N] ->
        (packed int32 [K/16, N*16/8], scale permuted [K/groupsize, N])."""
        assert weight.dtype == torch.int, f"weight dtype {weight.dtype} != torch.int"
        assert weight.shape[0] % groupsize == 0, "Weight shape must be divisible by groupsize"
        k, n = weight.shape
        if weight.is_cuda:
            from ... import _native as N
            assert scale.dtype == torch.half and scale.is_cuda and k % 16 == 0 and n % 64 == 0
            weight, scale = weight.contiguous(), scale.contiguous()
            packed = torch.empty(k // 16, n * 2, dtype=torch.int32, device=weight.device)
            scale_out = torch.empty(scale.numel() // n, n, dtype=torch.half, device=weight.device)
            N.check(N.lib().b200moe_marlin_pack(N.ptr(weight), N.ptr(packed), N.ptr(scale), N.ptr(scale_out), k, n,
                                                groupsize, N.stream()))
            return packed, scale_out
        sp = scale_perm_for(groupsize)
        scale = scale.reshape(-1, len(sp))[:, sp].reshape(-1, n).contiguous()
        tiles = weight.reshape(k // 16, 16, n // 16, 16).permute(0, 2, 1, 3).reshape(k // 16, n * 16)
        perm = _perm.to(weight.device)
        nib = tiles.reshape(-1, perm.numel())[:, perm].reshape(k // 16, n * 2, 8).to(torch.int64)
        shifts = torch.arange(0, 32, 4, device=weight.device, dtype=torch.int64)
        word = (nib << shifts).sum(-1)                     # disjoint bit fields: sum == or
        word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
        return word.to(torch.int32), scale

    @staticmethod
    def fake_quantize(weight: torch.Tensor, groupsize: int = -1) -> tuple:
        """utils.py:98-136.  weight f16 [K, N] -> (dequantized f16 [K, N], q int32 [K, N] in 0..15,
        scale f16 [K/groupsize, N]); scale = max|w| * (2/15) per (group along K, column), all
        arithmetic in f16 as in the reference."""
        assert weight.dtype == torch.half, f"weight dtype {weight.dtype} != torch.half"
        assert weight.shape[0] % groupsize == 0, "Weight shape must be divisible by groupsize"
        k, n = weight.shape
        g = k if groupsize == -1 else groupsize
        w = weight.reshape(k // g, g, n)
        scale = w.abs().amax(dim=1, keepdim=True)
        scale = scale * (2 / 15)
        q = torch.clamp(torch.round(w / scale).int() + 8, 0, 15)
        ref = (q - 8).half() * scale
        return ref.reshape(k, n).contiguous(), q.reshape(k, n).contiguous(), scale.reshape(k // g, n).contiguous()
