"""Grouped-GEMM MoE operators with the call surface of the reference's
moe/group_gemm_kernel.py, implemented by sm_100a CUDA kernels.

The reference launches its Triton kernels as ``kernel[(grid,)](args, BLOCK_SIZE=...)``
(e.g. moe/sglang_moe_all_gather_all_reduce.py:312, 375, 429).  The objects
exported here accept the same syntax; the grid and BLOCK_SIZE are ignored because
the CUDA launchers size themselves.
"""
import contextlib
import ctypes as C
import threading
from typing import List, Optional

import torch

from .. import _native as N

_workspaces = {}
_tls = threading.local()


@contextlib.contextmanager
def gemm_options(max_ctas: int = 0, pair_mode: int = 0):
    """Launch options for the grouped GEMMs called inside the `with` block by this thread (b200moe_gemm_opts:
    grid cap, CTA pairs).  They are passed with every call; the library keeps no such state."""
    prev = getattr(_tls, "opts", None)
    _tls.opts = N.GemmOpts(int(max_ctas), int(pair_mode))
    try:
        yield
    finally:
        _tls.opts = prev


def _opts():
    o = getattr(_tls, "opts", None)
    return None if o is None else C.byref(o)


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def run_moe_ep_preproess(topk_ids: torch.Tensor, num_experts: int):
    """Stable sort of the flat expert ids (reference :48-78).

    Returns (reorder_topk_ids int64 [T*k], src2dst int32 [T*k], seg_indptr int64 [E+1])."""
    N.require_cuda(topk_ids)
    assert topk_ids.dtype == torch.int64, "topk_ids must be int64"
    flat = topk_ids.contiguous().view(-1)
    n = flat.numel()
    dev = flat.device
    reorder_topk_ids = torch.empty(n, dtype=torch.int64, device=dev)
    src2dst = torch.empty(n, dtype=torch.int32, device=dev)
    seg_indptr = torch.empty(num_experts + 1, dtype=torch.int64, device=dev)
    need = N.lib().b200moe_route_metadata_workspace_bytes(n, num_experts)
    ws = _workspace(dev, need)
    N.check(N.lib().b200moe_route_metadata(N.ptr(flat), n, num_experts, N.ptr(reorder_topk_ids), N.ptr(src2dst),
                                           N.ptr(seg_indptr), N.ptr(ws), ws.numel(), N.stream()))
    return reorder_topk_ids, src2dst, seg_indptr


class _Launcher:
    """Accepts the Triton launch form ``obj[grid](*args, **meta)``."""

    def __init__(self, fn):
        self._fn = fn
        self.__doc__ = fn.__doc__
        self.__name__ = fn.__name__

    def __getitem__(self, grid):
        return self._fn

    def __call__(self, *args, **kwargs):
        return self._fn(*args, **kwargs)


def _f32_or_none(t):
    if t is None:
        return None
    return t if t.dtype == torch.float32 else t.float()


def _pre_reorder(input_ptr, gateup_input_ptr, src2dst_ptr, topk_ids_ptr, a1_scales_ptr,
                 start_expert_id, end_expert_id, topk, hidden_size, BLOCK_SIZE=512):
    """reference :81-117"""
    N.require_cuda(input_ptr, gateup_input_ptr, src2dst_ptr, topk_ids_ptr)
    assert input_ptr.is_contiguous() and gateup_input_ptr.is_contiguous()
    sc = _f32_or_none(a1_scales_ptr)
    T = input_ptr.numel() // hidden_size
    N.check(N.lib().b200moe_pre_reorder(N.ptr(input_ptr), N.dtype_code(input_ptr.dtype), N.ptr(gateup_input_ptr),
                                        N.dtype_code(gateup_input_ptr.dtype), N.ptr(src2dst_ptr), N.ptr(topk_ids_ptr),
                                        N.ptr(sc), int(start_expert_id), int(end_expert_id), T, int(topk),
                                        int(hidden_size), N.stream()))


def _act_and_mul(act):
    def run(gateup_output, down_input, hidden_size, reorder_topk_ids, scales, start_expert_id,
            end_expert_id, BLOCK_SIZE=512):
        N.require_cuda(gateup_output, down_input)
        assert gateup_output.is_contiguous() and down_input.is_contiguous()
        sc = _f32_or_none(scales)
        rows = gateup_output.numel() // hidden_size
        N.check(N.lib().b200moe_act_and_mul(N.ptr(gateup_output), N.dtype_code(gateup_output.dtype), N.ptr(down_input),
                                            N.dtype_code(down_input.dtype), rows, int(hidden_size),
                                            N.ptr(reorder_topk_ids), N.ptr(sc), int(start_expert_id),
                                            int(end_expert_id), act, N.stream()))
    run.__name__ = "silu_and_mul" if act == 0 else "gelu_and_mul"
    run.__doc__ = "reference :120-168" if act == 0 else "reference :176-235"
    return run


def _post_reorder(down_output_ptr, output_ptr, src2dst_ptr, topk_ids_ptr, topk_weights_ptr,
                  start_expert_id, end_expert_id, topk, hidden_size, BLOCK_SIZE=512):
    """reference :238-288 (f32 accumulation)"""
    N.require_cuda(down_output_ptr, output_ptr)
    assert down_output_ptr.is_contiguous() and output_ptr.is_contiguous()
    assert down_output_ptr.dtype == output_ptr.dtype
    w = _f32_or_none(topk_weights_ptr)
    T = output_ptr.numel() // hidden_size
    N.check(N.lib().b200moe_post_reorder(N.ptr(down_output_ptr), N.dtype_code(down_output_ptr.dtype), N.ptr(output_ptr),
                                         N.ptr(src2dst_ptr), N.ptr(topk_ids_ptr), N.ptr(w), int(start_expert_id),
                                         int(end_expert_id), T, int(topk), int(hidden_size), N.stream()))


pre_reorder_triton_kernel = _Launcher(_pre_reorder)
silu_and_mul_triton_kernel = _Launcher(_act_and_mul(0))
gelu_and_mul_triton_kernel = _Launcher(_act_and_mul(1))
post_reorder_triton_kernel = _Launcher(_post_reorder)


def permute_quant_fp8(x, src2dst, topk_ids, start_expert_id, end_expert_id, out_q, out_s):
    """Fused pre_reorder (:81-117) + 1x128 e4m3 act_quant.  out_q is a 2-D uint8/e4m3 view
    [S, >=H] and out_s a 2-D f32 view [S, >=H/128]; both may be strided views of one packed
    record buffer."""
    N.require_cuda(x, out_q, out_s)
    T, H = x.shape
    k = topk_ids.shape[1]
    assert x.is_contiguous() and out_q.stride(1) == 1 and out_s.stride(1) == 1
    N.check(N.lib().b200moe_permute_quant_fp8(N.ptr(x), N.dtype_code(x.dtype), N.ptr(src2dst), N.ptr(topk_ids),
                                              int(start_expert_id), int(end_expert_id), T, k, H,
                                              N.ptr(out_q), out_q.stride(0) * out_q.element_size(),
                                              N.ptr(out_s), out_s.stride(0), N.stream()))


def permute_quant_int8(x, src2dst, topk_ids, start_expert_id, end_expert_id, out_q, out_s, rounding="floor_half"):
    """Fused pre_reorder (:81-117) + 1x128 int8 act_quant; out_q int8/uint8 view [S, >=H], out_s f32 view
    [S, >=H/128] (the f16-rounded scale stored as f32)."""
    N.require_cuda(x, out_q, out_s)
    T, H = x.shape
    k = topk_ids.shape[1]
    assert x.is_contiguous() and out_q.stride(1) == 1 and out_s.stride(1) == 1 and out_s.dtype == torch.float32
    N.check(N.lib().b200moe_permute_quant_int8(N.ptr(x), N.dtype_code(x.dtype), N.ptr(src2dst), N.ptr(topk_ids),
                                               int(start_expert_id), int(end_expert_id), T, k, H,
                                               N.ptr(out_q), out_q.stride(0) * out_q.element_size(),
                                               N.ptr(out_s), out_s.stride(0),
                                               {"half_away": 0, "floor_half": 1}[rounding], N.stream()))


def gather_rows(src, dst, row_map):
    """dst[i] = src[row_map[i]] for 2-D byte-addressable row buffers (row size a multiple of 16 bytes)."""
    N.require_cuda(src, dst, row_map)
    assert src.is_contiguous() and dst.is_contiguous() and row_map.dtype == torch.int32
    rb = src.shape[1] * src.element_size()
    assert dst.shape[1] * dst.element_size() == rb
    N.check(N.lib().b200moe_gather_rows(N.ptr(src), N.ptr(dst), N.ptr(row_map), row_map.numel(), rb, N.stream()))
    return dst


def grouped_gemm_fp8(a, a_s, b, b_s, seg_indptr, weight_indices, c, c_s=None, epilogue: int = 0,
                     status_word=None, c_row_map=None, c_row_addr=None):
    """tcgen05 grouped blockwise GEMM on already-quantized activations.
    a [M,K] e4m3/uint8 (row-strided view allowed), a_s [M,K/128] f32 (row-strided view allowed),
    b [W,N,K] e4m3, b_s [W,N/128,K/128] f32, seg_indptr int64 [G+1], weight_indices int64 [G] or
    None.  epilogue 0: c [M,N] bf16/f16/f32; epilogue 1 (SiLU(gate)*up + requant) / 4 (GELU(gate)*up +
    requant): c [M,N/2] e4m3, c_s [M,N/256] f32.  c_row_map int32 [M] / c_row_addr int64 [M] (epilogue 0): row r is stored
    at row c_row_map[r] of c / at byte address c_row_addr[r] (possibly on another GPU)."""
    N.require_cuda(a, a_s, b, b_s, c)
    assert b.is_contiguous() and b_s.is_contiguous() and a.stride(1) == 1 and a_s.stride(1) == 1
    assert b_s.dtype == torch.float32 and a_s.dtype == torch.float32
    M, K = a.shape
    W, Nn, Kb = b.shape
    assert Kb == K
    G = seg_indptr.numel() - 1
    c_dtype = N.FP8_E4M3 if epilogue in (1, 4) else N.dtype_code(c.dtype)
    N.check(N.lib().b200moe_grouped_gemm_fp8(
        N.ptr(a), a.stride(0) * a.element_size(), N.ptr(a_s), a_s.stride(0), N.ptr(b), N.ptr(b_s),
        N.ptr(c), c_dtype, c.stride(0) * c.element_size(),
        N.ptr(c_s), 0 if c_s is None else c_s.stride(0), M, Nn, K, G, W,
        N.ptr(seg_indptr), N.ptr(weight_indices), epilogue, N.ptr(c_row_map), N.ptr(c_row_addr),
        N.ptr(status_word), _opts(), N.stream()))
    return c


def ep_plan(counts_all, rank, ep_size, cap_rows, recv_base, rec_bytes, back_base, back_row_bytes, out=None):
    """Device-side plan of the exchange that is folded into the permute and down-projection kernels
    (replaces the host-side split lists of moe/all2all_moe.py:150-200).  counts_all int64
    [ep_size, E]; recv_base / back_base int64 [ep_size] peer-mapped buffer addresses.
    Returns (dst_base [E], local_seg [E/ep+1], back_addr [cap_rows], info int32 [2])."""
    N.require_cuda(counts_all, recv_base, back_base)
    assert counts_all.dtype == torch.int64 and counts_all.is_contiguous()
    E = counts_all.numel() // ep_size
    dev = counts_all.device
    if out is None:
        out = (torch.empty(E, dtype=torch.int64, device=dev), torch.empty(E // ep_size + 1, dtype=torch.int64, device=dev),
               torch.empty(cap_rows, dtype=torch.int64, device=dev), torch.empty(2, dtype=torch.int32, device=dev))
    dst_base, local_seg, back_addr, info = out
    need = N.lib().b200moe_ep_plan_workspace_bytes(ep_size, E)
    assert need > 0, "num_experts must be a multiple of ep_size"
    ws = _workspace(dev, need)
    N.check(N.lib().b200moe_ep_plan(N.ptr(counts_all), rank, ep_size, E, cap_rows, N.ptr(recv_base), rec_bytes,
                                    N.ptr(back_base), back_row_bytes, N.ptr(dst_base), N.ptr(local_seg),
                                    N.ptr(back_addr), N.ptr(info), N.ptr(ws), ws.numel(), N.stream()))
    return out


def permute_quant_fp8_push(x, src2dst, topk_ids, seg_indptr, dst_base, rec_bytes, back_local=None):
    """permute_quant_fp8 storing every record at its owner: record of expert e at sorted position d
    -> dst_base[e] + (d - seg_indptr[e]) * rec_bytes (payload, then f32 scales at byte H).  back_local
    [slots, H] (this rank's return buffer): rows of dropped slots (dst_base[e] == 0) are cleared."""
    N.require_cuda(x, src2dst, topk_ids, seg_indptr, dst_base)
    T, H = x.shape
    assert x.is_contiguous() and topk_ids.dtype == torch.int64 and dst_base.dtype == torch.int64
    N.check(N.lib().b200moe_permute_quant_fp8_push(N.ptr(x), N.dtype_code(x.dtype), N.ptr(src2dst), N.ptr(topk_ids),
                                                   N.ptr(seg_indptr), N.ptr(dst_base), dst_base.numel(), T,
                                                   topk_ids.shape[1], H, rec_bytes, N.ptr(back_local),
                                                   0 if back_local is None else back_local.stride(0) * back_local.element_size(),
                                                   N.stream()))


def grouped_gemm_i8(a, a_s, b, b_s, seg_indptr, weight_indices, c, status_word=None):
    """tcgen05 grouped int8 GEMM with blockwise f32 scales (the w4a8 path once the weights are
    int8).  a int8 [M,K], a_s f32 [M,K/128], b int8 [W,N,K], b_s f32 [W,N/128,K/128]."""
    N.require_cuda(a, a_s, b, b_s, c)
    assert a.dtype == torch.int8 and b.dtype == torch.int8 and a_s.dtype == torch.float32 and b_s.dtype == torch.float32
    assert b.is_contiguous() and b_s.is_contiguous() and a.stride(1) == 1 and a_s.stride(1) == 1
    M, K = a.shape
    W, Nn, Kb = b.shape
    assert Kb == K
    N.check(N.lib().b200moe_grouped_gemm_i8(
        N.ptr(a), a.stride(0), N.ptr(a_s), a_s.stride(0), N.ptr(b), N.ptr(b_s), N.ptr(c), N.dtype_code(c.dtype),
        c.stride(0) * c.element_size(), M, Nn, K, seg_indptr.numel() - 1, W, N.ptr(seg_indptr),
        N.ptr(weight_indices), N.ptr(status_word), _opts(), N.stream()))
    return c


def pair_scales_t(s4: torch.Tensor, z4: torch.Tensor) -> torch.Tensor:
    """s4, z4 [..., N, K/128] -> [..., K/128, N, 2]: the (s4, z4) int8 pairs (or the (scale, zero) bf16 pairs of the
    w4a16 format) with one K group's pairs contiguous, the layout the fused-dequantization GEMMs read (built once per
    weight)."""
    return torch.stack([s4, z4], dim=-1).transpose(-3, -2).contiguous()


def grouped_gemm_w4a8(a, a_s, b_packed, s4z4_t, b_s, seg_indptr, weight_indices, c, c_s=None, epilogue: int = 0,
                      status_word=None):
    """tcgen05 grouped w4a8 GEMM with the int4 -> int8 step inside the kernel (reference w4a8_gemm,
    quantization/w4a8_kernel.py:317-448).  a int8 [M,K] and a_s f32 [M,K/128] (row-strided views allowed),
    b_packed int32 [W,N/8,K], s4z4_t int8 [W,K/128,N,2] (pair_scales_t), b_s f32 [W,N/128,K/128].
    epilogue 0: c [M,N]; epilogue 1 / 4: act(gate)*up + int8 re-quantization, c int8 [M,N/2], c_s f32 [M,N/256]."""
    N.require_cuda(a, a_s, b_packed, s4z4_t, b_s, c)
    assert a.dtype in (torch.int8, torch.uint8) and b_packed.dtype == torch.int32 and s4z4_t.dtype == torch.int8
    assert a_s.dtype == torch.float32 and b_s.dtype == torch.float32
    assert b_packed.is_contiguous() and s4z4_t.is_contiguous() and b_s.is_contiguous()
    assert a.stride(1) == 1 and a_s.stride(1) == 1
    M, K = a.shape
    W, N8, Kb = b_packed.shape
    Nn = N8 * 8
    assert Kb == K and tuple(s4z4_t.shape) == (W, K // 128, Nn, 2)
    c_dtype = N.I8 if epilogue in (1, 4) else N.dtype_code(c.dtype)
    N.check(N.lib().b200moe_grouped_gemm_w4a8(
        N.ptr(a), a.stride(0), N.ptr(a_s), a_s.stride(0), N.ptr(b_packed), N.ptr(s4z4_t), N.ptr(b_s),
        N.ptr(c), c_dtype, c.stride(0) * c.element_size(), N.ptr(c_s), 0 if c_s is None else c_s.stride(0),
        M, Nn, K, seg_indptr.numel() - 1, W, N.ptr(seg_indptr), N.ptr(weight_indices), epilogue,
        N.ptr(status_word), N.stream()))
    return c


def grouped_gemm_w4a16(a, b_packed, scale_zero_t, seg_indptr, weight_indices, c, epilogue: int = 0, status_word=None):
    """tcgen05 grouped w4a16 GEMM with the int4 -> bf16 dequantization inside the kernel.  a bf16 [M,K] (row-strided
    view allowed), b_packed int32 [W,N,K/8], scale_zero_t bf16 [W,K/128,N,2] (pair_scales_t(scale, zero)).
    epilogue 0: c [M,N]; 2 / 5: SiLU(gate)*up / GELU(gate)*up, c bf16 [M,N/2]."""
    N.require_cuda(a, b_packed, scale_zero_t, c)
    assert a.dtype == torch.bfloat16 and b_packed.dtype == torch.int32 and scale_zero_t.dtype == torch.bfloat16
    assert b_packed.is_contiguous() and scale_zero_t.is_contiguous() and a.stride(1) == 1
    M, K = a.shape
    W, Nn, K8 = b_packed.shape
    assert K8 * 8 == K and tuple(scale_zero_t.shape) == (W, K // 128, Nn, 2)
    N.check(N.lib().b200moe_grouped_gemm_w4a16(
        N.ptr(a), a.stride(0) * 2, N.ptr(b_packed), N.ptr(scale_zero_t), N.ptr(c), N.dtype_code(c.dtype),
        c.stride(0) * c.element_size(), M, Nn, K, seg_indptr.numel() - 1, W, N.ptr(seg_indptr),
        N.ptr(weight_indices), epilogue, N.ptr(status_word), N.stream()))
    return c


def grouped_gemm_bf16(a, b, seg_indptr, weight_indices, c, epilogue: int = 0, status_word=None):
    """tcgen05 grouped bf16 or f16 GEMM (reference: the scale-free branch of grouped_gemm_triton,
    :410-412).  epilogue 0: c [M,N]; epilogue 2 / 5 (bf16 operands only): SiLU(gate)*up / GELU(gate)*up fused,
    c bf16 [M,N/2]; epilogue 3: c = round(c + round(a @ b^T)) for a 16-bit c."""
    N.require_cuda(a, b, c)
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    assert b.is_contiguous() and a.stride(1) == 1
    M, K = a.shape
    W, Nn, Kb = b.shape
    assert Kb == K
    if a.dtype == torch.float16:
        assert epilogue in (0, 3), "the fused SwiGLU epilogue takes bf16 operands"
        assert epilogue == 0, "b200moe_grouped_gemm_f16 has the plain epilogue only"
        N.check(N.lib().b200moe_grouped_gemm_f16(
            N.ptr(a), a.stride(0) * 2, N.ptr(b), N.ptr(c), N.dtype_code(c.dtype), c.stride(0) * c.element_size(),
            M, Nn, K, seg_indptr.numel() - 1, W, N.ptr(seg_indptr), N.ptr(weight_indices),
            N.ptr(status_word), _opts(), N.stream()))
        return c
    N.check(N.lib().b200moe_grouped_gemm_bf16(
        N.ptr(a), a.stride(0) * 2, N.ptr(b), N.ptr(c), N.dtype_code(c.dtype), c.stride(0) * c.element_size(),
        M, Nn, K, seg_indptr.numel() - 1, W, N.ptr(seg_indptr), N.ptr(weight_indices), epilogue,
        N.ptr(status_word), _opts(), N.stream()))
    return c


def grouped_gemm_triton(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, batch_size: int,
                        weight_column_major: bool, seg_indptr: Optional[torch.Tensor] = None,
                        weight_indices: Optional[torch.Tensor] = None, use_fp8_w8a8: bool = False,
                        scale_a: torch.Tensor = None, scale_b: torch.Tensor = None,
                        block_shape: Optional[List[int]] = None):
    """reference :442-513.  b must be e4m3 with block_shape == [128, 128].  As in the
    reference, `a` arrives unquantized (f16/bf16) and is quantized 1x128 inside the call
    (the reference does it with its int8 quantizer, :459-469); pass an e4m3 `a` together
    with scale_a to skip that."""
    assert weight_column_major == True  # noqa: E712  (same assert as the reference)
    assert seg_indptr is not None
    if block_shape is None:
        # scale-free branch (:410-412): f16 or bf16 operands, f32 accumulation
        assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16), "the unquantized branch takes f16 or bf16"
        seg = seg_indptr if seg_indptr.is_contiguous() else seg_indptr.contiguous()
        return grouped_gemm_bf16(a, b, seg[: batch_size + 1], weight_indices, c, epilogue=0)
    assert list(block_shape) == [128, 128], "only block_shape=[128,128] is supported"
    assert b.dtype == torch.float8_e4m3fn, "the B200 grouped GEMM takes e4m3 weights"
    assert seg_indptr is not None
    if a.dtype != torch.float8_e4m3fn:
        from ..quantization.fp8_kernel import act_quant
        a, scale_a = act_quant(a.contiguous(), block_shape[1])
    assert scale_a is not None and scale_b is not None
    assert -(-a.shape[-1] // block_shape[1]) == scale_a.shape[-1]
    assert -(-b.shape[-2] // block_shape[0]) == scale_b.shape[-2]
    assert -(-b.shape[-1] // block_shape[1]) == scale_b.shape[-1]
    seg = seg_indptr if seg_indptr.is_contiguous() else seg_indptr.contiguous()
    grouped_gemm_fp8(a, scale_a, b, _f32_or_none(scale_b).contiguous(), seg[: batch_size + 1],
                     weight_indices, c, epilogue=0)
    return c


def dequant_sum(payload: torch.Tensor, scales: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [R, H] = sum over sources of dequantized chunks (each rounded to out's dtype, f32 accumulation).
    payload [n, R, H] e4m3 (f32 scales [n, R, H/128]) or int8 (f16 scales); the middle and last steps of the
    quantized all-reduce (reference quant_communication/quant_all2all_allreduce.py:73-80, 96-99)."""
    N.require_cuda(payload, scales, out)
    assert payload.is_contiguous() and scales.is_contiguous() and out.is_contiguous()
    n, R, H = payload.shape
    assert tuple(scales.shape) == (n, R, H // 128) and tuple(out.shape) == (R, H)
    qd = N.FP8_E4M3 if payload.dtype == torch.float8_e4m3fn else N.dtype_code(payload.dtype)
    N.check(N.lib().b200moe_dequant_sum(N.ptr(payload), qd, H, R * H, N.ptr(scales), N.dtype_code(scales.dtype),
                                        H // 128, R * (H // 128), n, R, H, N.ptr(out), N.dtype_code(out.dtype),
                                        N.stream()))
    return out
