"""cutlass_scaled_mm: c = (a_scale * b_scale) * (a @ b) [+ bias] for FP8 operands.

Mirrors src/flag_gems/fused/cutlass_scaled_mm.py:475-526 (checks) and :371-431
(dispatch on the scale shapes) of the reference.  Where the reference raises
NotImplementedError on compute capability 10.x (:459-460), this runs the tcgen05
kernels of ``fg_scaled_mm_fp8`` / ``fg_block_scaled_mm_fp8``.
"""
import logging
from typing import Optional

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def _cdiv(a, b):
    return (a + b - 1) // b


def cutlass_scaled_mm(
    c: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
) -> None:
    logger.debug("GEMS CUTLASS SCALED MM")
    assert a.dim() == 2 and b.dim() == 2 and c.dim() == 2, "All inputs must be 2D tensors"
    assert c.size(0) == a.size(0), "Number of rows in c must equal number of rows in a"
    assert a.size(1) == b.size(0), "Number of columns in a must equal number of rows in b"
    assert b.size(1) == c.size(1), "Number of columns in b must equal number of columns in c"
    assert a.stride(1) == 1 and c.stride(1) == 1, "a and c must be row-major"
    assert b.stride(0) == 1, "b must be column-major"
    assert c.stride(0) % 16 == 0, "Row stride of c must be 16-byte aligned"
    assert b.stride(1) % 16 == 0, "Column stride of b must be 16-byte aligned"
    if bias is not None:
        assert bias.numel() == b.size(1), f"Bias size {bias.numel()} must equal number of columns in b {b.size(1)}"
        assert bias.is_contiguous(), "Bias must be contiguous"
        assert bias.dim() == 1, "Bias must be a 1D tensor"
    assert a_scale.dtype == torch.float32, "a_scale must be float32"
    assert b_scale.dtype == torch.float32, "b_scale must be float32"
    _cabi.require_cuda(c, a, b, a_scale, b_scale, bias)

    m, k = a.shape
    n = b.size(1)
    if a.dtype != torch.float8_e4m3fn or b.dtype != torch.float8_e4m3fn:
        if a.dtype == torch.int8:
            raise RuntimeError("Int8 not supported on SM100. Use FP8 quantization instead, or run on older arch (SM < 100).")
        raise AssertionError(f"Unsupported dtype: {a.dtype}")
    if c.dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported output dtype {c.dtype}")
    L = _cabi.lib()
    stream = _cabi.stream_ptr(a.device)

    vector_scales = (a_scale.numel() == 1 or a_scale.numel() == m) and (b_scale.numel() == 1 or b_scale.numel() == n)
    with _cabi.device_guard(a):
        if vector_scales:
            assert a_scale.is_contiguous(), "a_scale must be contiguous"
            assert b_scale.is_contiguous(), "b_scale must be contiguous"
            if bias is not None and bias.dtype != c.dtype:
                bias = bias.to(c.dtype)
            _cabi.check(
                L.fg_scaled_mm_fp8(
                    _cabi.ptr(c), _cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(a_scale), _cabi.ptr(b_scale), _cabi.ptr(bias),
                    m, n, k, a.stride(0), b.stride(1), c.stride(0),
                    _cabi.SCALE_VECTOR if a_scale.numel() > 1 else _cabi.SCALE_SCALAR,
                    _cabi.SCALE_VECTOR if b_scale.numel() > 1 else _cabi.SCALE_SCALAR,
                    _cabi.DTYPE_CODE[c.dtype], 1, stream,
                )
            )
        else:
            assert a_scale.dim() == 2, "a_scale must be 2D tensor for blockwise scaling"
            assert b_scale.dim() == 2, "b_scale must be 2D tensor for blockwise scaling"
            assert a.size(0) == a_scale.size(0), (
                f"a_scale must have same first dimension as a: a.shape[0]={a.size(0)}, a_scale.shape[0]={a_scale.size(0)}"
            )
            assert _cdiv(a.size(1), 128) == a_scale.size(1), (
                f"a_scale second dimension mismatch: cdiv({a.size(1)}, 128)={_cdiv(a.size(1), 128)} != "
                f"a_scale.shape[1]={a_scale.size(1)}"
            )
            assert _cdiv(b.size(0), 128) == b_scale.size(0), (
                f"b_scale first dimension mismatch: cdiv({b.size(0)}, 128)={_cdiv(b.size(0), 128)} != "
                f"b_scale.shape[0]={b_scale.size(0)}"
            )
            assert _cdiv(b.size(1), 128) == b_scale.size(1), (
                f"b_scale second dimension mismatch: cdiv({b.size(1)}, 128)={_cdiv(b.size(1), 128)} != "
                f"b_scale.shape[1]={b_scale.size(1)}"
            )
            assert bias is None, "Bias not yet supported for blockwise scaled_mm"
            # b_scale is [K/128, N/128] here: block (n, k) sits at k*stride(0) + n*stride(1)
            _cabi.check(
                L.fg_block_scaled_mm_fp8(
                    _cabi.ptr(c), _cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(a_scale), _cabi.ptr(b_scale),
                    m, n, k, a.stride(0), b.stride(1), c.stride(0), a_scale.stride(0), a_scale.stride(1),
                    b_scale.stride(1), b_scale.stride(0), _cabi.DTYPE_CODE[c.dtype], stream,
                )
            )
    return None
