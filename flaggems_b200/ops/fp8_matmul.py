"""fp8_matmul: block-wise scaled FP8 matrix product with bf16 output.

Mirrors src/flag_gems/ops/fp8_matmul.py:137-205 of the reference (the C++ twin is
cpp/lib/fp8_matmul.cpp:25-102).
"""
import logging

import torch

from .w8a8_block_fp8_matmul import w8a8_block_fp8_matmul

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def fp8_matmul(a, a_s, b, b_s, scale_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    logger.debug("GEMS FP8_MATMUL")
    assert b.ndim == 2
    assert a.is_contiguous() and b.is_contiguous()
    assert a_s.is_contiguous() and b_s.is_contiguous()
    assert a.size(-1) == b.size(1)
    if scale_dtype != torch.float32:
        a_s = a_s.to(torch.float32)
        b_s = b_s.to(torch.float32)
    return w8a8_block_fp8_matmul(a, b, a_s, b_s, [128, 128], torch.bfloat16)
