"""`mul`: f16 activations x Marlin-order int4 weights (reference: the pybind11 module `marlin_cuda`,
fast_dequant/simple_marlin/marlin_w4a16_gemm.cpp:23-129, kernel marlin_w4a16_gemm.cu:86-280).

The reference streams the packed weights through mma.sync fragments.  Here a CUDA kernel expands the
nibbles to f16 in nn.Linear layout, `(q - 8) * scale` rounded to f16 exactly as the reference's
dequantization (marlin_w4a16_gemm.cu:44-64), and the product runs on the tcgen05 f16 path with f32
accumulation.  The expansion is cached per packed tensor, keyed on storage and version."""
from typing import Dict, Tuple

import torch

from ... import _native as N

_cache: Dict[Tuple[int, int, int, int], torch.Tensor] = {}


def expand(B: torch.Tensor, s: torch.Tensor, K: int, Nn: int, groupsize: int) -> torch.Tensor:
    """packed int32 [K/16, N*2] + permuted scales f16 [K/g, N] -> f16 [N, K].  groupsize -1: one group,
    scales in the single-group permutation; otherwise the grouped permutation (also when groupsize == K)."""
    N.require_cuda(B, s)
    assert B.dtype == torch.int32 and s.dtype == torch.half and B.is_contiguous() and s.is_contiguous()
    assert tuple(B.shape) == (K // 16, Nn * 2), f"packed shape {tuple(B.shape)} for K={K} N={Nn}"
    assert s.numel() == (1 if groupsize == -1 else K // groupsize) * Nn
    out = torch.empty(Nn, K, dtype=torch.half, device=B.device)
    N.check(N.lib().b200moe_marlin_expand_f16(N.ptr(B), N.ptr(s), N.ptr(out), K, Nn, groupsize, N.stream()))
    return out


def mul(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, s: torch.Tensor, workspace: torch.Tensor = None,
        thread_k: int = -1, thread_n: int = -1, sms: int = -1, max_par: int = 16) -> None:
    """C[M, N] = A[M, K] @ dequant(B).  Errors follow marlin_w4a16_gemm.cpp:38-108 (RuntimeError with the
    same messages).  workspace, thread_k, thread_n, sms, max_par are accepted and unused, as in the
    reference binding.  As there, a 2-D `s` [K/g, N] means groups of g = K / rows packed with
    QuantUtils.pack(..., groupsize=g); a 1-D `s` [N] means QuantUtils.pack(..., groupsize=-1)."""
    M, K = A.shape
    Nn = C.shape[1]
    if M % 16 or Nn % 16 or K % 16:
        raise RuntimeError(f"Matrix dimensions must be divisible by 16. Got M={M}, N={Nn}, K={K}")
    if not (A.is_cuda and B.device == A.device and C.device == A.device and s.device == A.device):
        raise RuntimeError("All tensors must be on the same CUDA device")
    if A.dtype != torch.half or C.dtype != torch.half:
        raise RuntimeError("A and C matrices must be of type torch.float16")
    if s.dtype != torch.half:
        raise RuntimeError("Scale tensor must be of type torch.float16")
    if B.dtype != torch.int32:
        raise RuntimeError("B matrix must be packed INT4 data (torch.int32)")
    if s.dim() == 2:
        if s.shape[1] != Nn:
            raise RuntimeError(f"Scale tensor N dimension mismatch: expected {Nn} but got {s.shape[1]}")
        if K % s.shape[0]:
            raise RuntimeError(f"K dimension not divisible by groupsize: K={K}, groupsize={K // s.shape[0]}")
    if Nn % 64 or K % 64:
        # one permutation block spans 64 output columns; the tcgen05 K step is 64 f16 values
        raise RuntimeError("Matrix dimensions not compatible with Marlin kernel requirements")
    A, B, s = A.contiguous(), B.contiguous(), s.contiguous()
    key = (B.data_ptr(), B._version, s.data_ptr(), s._version)
    w = _cache.get(key)
    if w is None or w.shape[1] != K or w.shape[0] < Nn or w.device != B.device:
        if len(_cache) >= 64:
            _cache.clear()
        w = expand(B, s, K, Nn, K // s.shape[0] if s.dim() == 2 else -1)
        if Nn % 128:                       # the GEMM tiles N by 128: pad with zero rows once
            w = torch.cat([w, w.new_zeros(128 - Nn % 128, K)])
        _cache[key] = w
    from ...moe.group_gemm_kernel import grouped_gemm_bf16
    direct = C.is_contiguous() and w.shape[0] == Nn
    out = C if direct else torch.empty(M, w.shape[0], dtype=torch.half, device=A.device)
    seg = torch.tensor([0, M], dtype=torch.int64, device=A.device)
    grouped_gemm_bf16(A, w.unsqueeze(0), seg, None, out)
    if not direct:
        C.copy_(out[:, :Nn])
