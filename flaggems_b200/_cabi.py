"""ctypes binding of the C-ABI library (include/flaggems_b200.h).

The library is the only compute path: if it is missing or an entry point fails,
the caller gets an exception; there is no fallback of any kind.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_uint, c_uint64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libflaggems_b200.so")

FG_OK = 0
DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
DTYPE_E4M3 = 3  # output of fg_scaled_mm_fp8 only
SCALE_SCALAR, SCALE_VECTOR, SCALE_BLOCK = 0, 1, 2

_P = c_void_p
_SIGS = {
    "fg_version": (c_int, []),
    "fg_last_error": (c_char_p, []),
    "fg_device_status": (c_int, [ctypes.POINTER(c_uint)]),
    "fg_launch_count": (c_uint64, []),
    "fg_selftest_bounded_wait": (c_int, [c_int64, c_int, _P]),
    "fg_act_quant_bf16_e4m3": (c_int, [_P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_int, _P]),
    "fg_per_token_group_quant_fp8": (
        c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_int, _P]),
    "fg_per_token_quant_fp8": (
        c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int32, c_int32, _P, _P]),
    "fg_per_token_quant_int8": (
        c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int32, c_int32, _P, _P]),
    "fg_per_tensor_quant_fp8": (
        c_int, [_P, c_int, _P, _P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int32, c_int32, _P, _P]),
    "fg_abs_max": (c_int, [_P, c_int, c_int64, c_int64, c_int64, _P, _P, _P]),
    "fg_per_token_group_quant_fp8_gather": (
        c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64, _P, c_int32, c_int32, _P, _P]),
    "fg_moe_align_block_size": (
        c_int, [_P, c_int, c_int64, c_int, c_int, _P, c_int, _P, c_int64, _P, c_int64, _P, _P]),
    "fg_silu_and_mul": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "fg_moe_sum": (c_int, [_P, _P, c_int64, c_int, c_int64, c_int, _P]),
    "fg_moe_sum_indexed": (c_int, [_P, _P, c_int64, c_int, c_int64, c_int, _P, _P, _P]),
    "fg_gather_rows_fp8": (
        c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, _P, c_int32, c_int32, _P, _P]),
    "fg_moe_align_block_size_ex": (
        c_int, [_P, c_int, c_int64, c_int, c_int, _P, c_int, _P, c_int64, _P, c_int64, _P, c_int64, c_int, _P, _P,
                _P]),
    "fg_ep_pack_rows_fp8_peer": (
        c_int, [_P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P, c_int64,
                _P, _P, _P, c_int, c_int64, _P]),
    "fg_moe_align_block_size_regions": (
        c_int, [_P, c_int, c_int64, c_int, c_int, _P, c_int, _P, c_int64, _P, c_int64, _P, c_int64, c_int, _P, _P,
                c_int64, _P, c_int64, _P]),
    "fg_ep_pack_rows_fp8": (
        c_int, [_P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P, c_int64,
                _P, _P]),
    "fg_moe_routed_workspace_bytes": (c_int64, [c_int64, c_int, c_int64, c_int64]),
    "fg_moe_routed_block_fp8_local": (
        c_int, [_P, _P, c_int, _P, c_int, _P, c_int, c_int64, c_int, _P, _P, _P, _P, c_int, c_int64, c_int64,
                _P, c_int64, _P]),
    "fg_moe_routed_block_fp8_local_noalloc": (
        c_int, [_P, _P, c_int, _P, c_int, _P, c_int, c_int64, c_int, _P, _P, _P, _P, c_int, c_int64, c_int64, _P]),
    "fg_moe_routed_block_fp8_packed": (
        c_int, [_P, _P, c_int64, c_int64, _P, _P, _P, _P, c_int, c_int64, c_int64, _P, c_int64, c_int, _P, c_int,
                c_int64, _P, c_int64, _P, c_int64, _P]),
    "fg_moe_grouped_gemm_fp8_peer": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int64, _P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int64, _P, c_int, c_int64,
                _P]),
    "fg_scaled_grouped_mm_workspace_bytes": (c_int64, [c_int64, c_int, c_int64]),
    "fg_scaled_grouped_mm_fp8": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                _P, c_int64, _P]),
    "fg_group_ids_from_offsets": (c_int, [_P, c_int, c_int64, _P, _P]),
    "fg_grouped_gemm_fp8_bias": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int64, _P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64, c_int64,
                c_int64, c_int, _P]),
    "fg_symm_alloc": (c_int, [c_int64, ctypes.POINTER(c_void_p), _P]),
    "fg_symm_open": (c_int, [_P, ctypes.POINTER(c_void_p)]),
    "fg_symm_close": (c_int, [_P]),
    "fg_symm_free": (c_int, [_P]),
    "fg_scaled_mm_fp8": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                c_int, c_int, c_int, c_int, _P]),
    "fg_block_scaled_mm_fp8": (
        c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                c_int64, c_int64, c_int64, c_int, _P]),
    "fg_topk_softmax": (
        c_int, [_P, _P, c_int, _P, _P, c_int, c_int64, c_int, c_int, c_int, _P, _P]),
    "fg_grouped_topk": (
        c_int, [_P, _P, _P, _P, c_int, c_int64, c_int, c_int64, c_int, c_int, c_int, c_int, ctypes.c_float, c_int,
                _P, _P]),
    "fg_moe_grouped_gemm_16bit": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int64, _P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "fg_moe_grouped_gemm_int8": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int64, _P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "fg_moe_grouped_gemm_fp8": (
        c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int64, _P, _P, _P, c_int64, c_int64, c_int, c_int64, c_int64,
                c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGS)

_lib = None


class FlagGemsB200Error(RuntimeError):
    pass


def lib():
    """Load the shared library once; raise (never fall back) when it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlagGemsB200Error(
                f"{LIB_PATH} not found: build it with `python -m flaggems_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    if rc != FG_OK:
        msg = lib().fg_last_error().decode(errors="replace")
        if rc == -1:
            raise AssertionError(msg)
        if rc == -2:
            raise NotImplementedError(msg)
        raise FlagGemsB200Error(f"flaggems_b200 error {rc}: {msg}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NO_GUARD = _NoGuard()


def device_guard(t):
    """Context that makes t's device current; free when it already is."""
    idx = t.device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(idx)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise FlagGemsB200Error(
                "flaggems_b200 runs on CUDA tensors only (sm_100a); got a tensor on "
                f"{t.device}. There is no CPU path."
            )


def device_status():
    """Read-and-clear the device status word; raises if a kernel reported a failed bounded wait."""
    v = c_uint(0)
    rc = lib().fg_device_status(ctypes.byref(v))
    check(rc)
    return v.value


def launch_count():
    return int(lib().fg_launch_count())
