"""w8a8_block_fp8_matmul: FP8 GEMM with 1x128 activation and 128x128 weight scales.

Mirrors src/flag_gems/ops/w8a8_block_fp8_matmul.py:173-232 of the reference.
"""
import logging
from typing import List

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def _cdiv(a, b):
    return (a + b - 1) // b


def w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: List[int],
    output_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    logger.debug("GEMS W8A8_BLOCK_FP8_MATMUL")
    assert len(block_size) == 2
    block_n, block_k = block_size[0], block_size[1]
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1] and A.is_contiguous()
    assert _cdiv(A.shape[-1], block_k) == As.shape[-1]
    m = A.numel() // A.shape[-1]
    assert B.ndim == 2 and Bs.ndim == 2
    n, k = B.shape
    assert _cdiv(n, block_n) == Bs.shape[0]
    assert _cdiv(k, block_k) == Bs.shape[1]
    if block_n != 128 or block_k != 128:
        raise NotImplementedError(f"block_size {block_size}: only [128, 128] is implemented")
    if A.dtype != torch.float8_e4m3fn or B.dtype != torch.float8_e4m3fn:
        raise NotImplementedError(f"operands must be float8_e4m3fn, got {A.dtype} and {B.dtype}")
    if output_dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported output dtype {output_dtype}")
    _cabi.require_cuda(A, B, As, Bs)

    c = A.new_empty(A.shape[:-1] + (n,), dtype=output_dtype)
    if m == 0 or n == 0:
        return c
    if B.stride(1) != 1 or B.stride(0) % 16 != 0:
        B = B.contiguous()
    As2 = As.reshape(m, As.shape[-1])  # any strides: row-major or the column-major scale layout
    if As2.dtype != torch.float32:
        As2 = As2.float()
    if Bs.dtype != torch.float32:
        Bs = Bs.float()
    with _cabi.device_guard(A):
        _cabi.check(
            _cabi.lib().fg_block_scaled_mm_fp8(
                _cabi.ptr(c), _cabi.ptr(A), _cabi.ptr(B), _cabi.ptr(As2), _cabi.ptr(Bs),
                m, n, k, k, B.stride(0), n, As2.stride(0), As2.stride(1), Bs.stride(0), Bs.stride(1),
                _cabi.DTYPE_CODE[output_dtype], _cabi.stream_ptr(A.device),
            )
        )
    return c
