"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The library is built in-tree by `python -m llm_kernels_b200.build` and is loaded
lazily on first use.  Nothing here falls back to another implementation: a
missing library or a non-zero status raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200moe.so")

OK = 0
F32, F16, BF16, FP8_E4M3, I8 = 0, 1, 2, 3, 4
_DTYPES = {  # torch dtype -> B200MOE_* code
   torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16,
           torch.float8_e4m3fn: FP8_E4M3, torch.int8: I8}

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); every exported symbol of include/b200moe.h
SIGNATURES = {
    "b200moe_status_string": (C.c_char_p, [_i]),
    "b200moe_last_error": (C.c_char_p, []),
    "b200moe_abi_version": (_i, []),
    "b200moe_act_quant_fp8": (_i, [_p, _i, _i64, _i64, _p, _i64, _p, _i64, _p]),
    "b200moe_weight_dequant_fp8": (_i, [_p, _p, _p, _i, _i64, _i64, _p]),
    "b200moe_weight_quant_fp8": (_i, [_p, _i, _p, _p, _i64, _i64, _p]),
    "b200moe_gemm_fp8_block": (_i, [_p, _p, _p, _p, _p, _i, _i64, _i64, _i64, _p]),
    "b200moe_gemm_fp8_block_splitk": (_i, [_p, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _p, _i64, _p]),
    "b200moe_act_quant_int8": (_i, [_p, _i, _i64, _i64, _p, _p, _i, _p]),
    "b200moe_dequant_sum": (_i, [_p, _i, _i64, _i64, _p, _i, _i64, _i64, _i, _i64, _i64, _p, _i, _p]),
    "b200moe_router_topk": (_i, [_p, _i, _p, _p, _i64, _i64, _i, _i, _i, _i, _i, _i, _f, _p, _p, _p]),
    "b200moe_router_logits_bf16x3": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p]),
    "b200moe_router_select": (_i, [_p, _i, _i64, _p, _i64, _i, _i, _i, _i, _i, _i, _f, _p, _p, _p]),
    "b200moe_route_metadata_workspace_bytes": (_sz, [_i64, _i]),
    "b200moe_route_metadata": (_i, [_p, _i64, _i, _p, _p, _p, _p, _sz, _p]),
    "b200moe_route_metadata_noalloc": (_i, [_p, _i64, _i, _p, _p, _p, _p]),
    "b200moe_pre_reorder": (_i, [_p, _i, _p, _i, _p, _p, _p, _i, _i, _i64, _i, _i64, _p]),
    "b200moe_permute_quant_fp8": (_i, [_p, _i, _p, _p, _i, _i, _i64, _i, _i64, _p, _i64, _p, _i64, _p]),
    "b200moe_permute_quant_int8": (_i, [_p, _i, _p, _p, _i, _i, _i64, _i, _i64, _p, _i64, _p, _i64, _i, _p]),
    "b200moe_act_and_mul": (_i, [_p, _i, _p, _i, _i64, _i64, _p, _p, _i, _i, _i, _p]),
    "b200moe_post_reorder": (_i, [_p, _i, _p, _p, _p, _p, _i, _i, _i64, _i, _i64, _p]),
    "b200moe_grouped_gemm_fp8": (_i, [_p, _i64, _p, _i64, _p, _p, _p, _i, _i64, _p, _i64,
                                      _i64, _i64, _i64, _i, _i, _p, _p, _i, _p, _p, _p, _p, _p]),
    "b200moe_ep_plan_workspace_bytes": (_i64, [_i, _i]),
    "b200moe_ep_plan": (_i, [_p, _i, _i, _i, _i64, _p, _i64, _p, _i64, _p, _p, _p, _p, _p, _i64, _p]),
    "b200moe_permute_quant_fp8_push": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i, _i64, _i64, _p, _i64, _p]),
    "b200moe_gather_rows": (_i, [_p, _p, _p, _i64, _i64, _p]),
    "b200moe_w4a8_expand_int8": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "b200moe_w4a16_expand_bf16": (_i, [_p, _p, _p, _p, _i64, _i64, _p]),
    "b200moe_grouped_gemm_i8": (_i, [_p, _i64, _p, _i64, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _i,
                                     _p, _p, _p, _p, _p]),
    "b200moe_grouped_gemm_w4a8": (_i, [_p, _i64, _p, _i64, _p, _p, _p, _p, _i, _i64, _p, _i64, _i64, _i64, _i64,
                                       _i, _i, _p, _p, _i, _p, _p]),
    "b200moe_grouped_gemm_w4a16": (_i, [_p, _i64, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _i, _p, _p, _i, _p, _p]),
    "b200moe_grouped_gemm_bf16": (_i, [_p, _i64, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _i, _p, _p, _i, _p, _p, _p]),
    "b200moe_grouped_gemm_f16": (_i, [_p, _i64, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _i, _p, _p, _p, _p, _p]),
    "b200moe_marlin_expand_f16": (_i, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "b200moe_marlin_pack": (_i, [_p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "b200moe_weight_quant_int8": (_i, [_p, _i, _p, _p, _i64, _i64, _f, _i, _p]),
    "b200moe_weight_dequant_int8": (_i, [_p, _p, _p, _i, _i64, _i64, _p]),
    "b200moe_weight_quant_w4a8": (_i, [_p, _i, _p, _p, _p, _p, _i64, _i64, _p]),
    "b200moe_weight_quant_w4a16": (_i, [_p, _i, _p, _p, _p, _i64, _i64, _p]),
    "b200moe_pack_bits": (_i, [_p, _p, _i64, _i64, _i, _i, _i, _p]),
    "b200moe_unpack_bits": (_i, [_p, _p, _i64, _i64, _i, _i, _i, _p]),
}

class GemmOpts(C.Structure):
    """b200moe_gemm_opts: per-call launch options of the grouped GEMMs."""
    _fields_ = [("max_ctas", C.c_int32), ("pair_mode", C.c_int32)]


_lib = None
_lock = threading.Lock()


class B200MoeError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200moe status {status}: {message}")
        self.status = status


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m llm_kernels_b200.build` "
                        "(there is no CPU or PyTorch fallback)")
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


def check(status: int) -> None:
    """Maps a non-zero status to an exception.  Shape/argument problems raise
    AssertionError (the reference's wrappers use bare asserts for those), the
    rest B200MoeError."""
    if status == OK:
        return
    msg = lib().b200moe_last_error().decode() or lib().b200moe_status_string(status).decode()
    if status in (1, 2, 3, 4):
        raise AssertionError(msg)
    raise B200MoeError(status, msg)


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DTYPES[t]
    except KeyError:
        raise AssertionError(f"unsupported dtype {t}") from None


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors) -> None:
    """Every tensor must live on the CURRENT CUDA device: the launchers take the current device's stream and
    the library looks its device up with cudaGetDevice, so a tensor of another GPU would have its pointer
    dereferenced on the wrong device.  Select the device first (torch.cuda.set_device / torch.cuda.device)."""
    cur = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("b200moe operators run on CUDA tensors only (no CPU path)")
        if cur is None:
            cur = torch.cuda.current_device()
        if t.device.index != cur:
            raise RuntimeError(f"tensor on cuda:{t.device.index} but the current device is cuda:{cur}: make the "
                               "tensor's device current before calling (torch.cuda.set_device or torch.cuda.device)")
