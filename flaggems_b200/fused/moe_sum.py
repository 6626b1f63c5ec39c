"""moe_sum: out[t, :] = sum_k input[t, k, :] in fp32.

Mirrors src/flag_gems/fused/moe_sum.py:70-90 of the reference.
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def moe_sum(input: torch.Tensor, output: torch.Tensor):
    logger.debug("GEMS MOE SUM")
    assert input.dim() == 3 and output.dim() == 2, "input must be [M, topk, K] and output [M, K]"
    m, topk, k = input.shape
    assert output.shape == (m, k), "output shape mismatch"
    assert input.dtype == output.dtype, "dtype mismatch"
    _cabi.require_cuda(input, output)
    if input.dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported dtype {input.dtype}")
    src = input if input.is_contiguous() else input.contiguous()
    dst = output if output.is_contiguous() else torch.empty_like(output, memory_format=torch.contiguous_format)
    with _cabi.device_guard(input):
        _cabi.check(
            _cabi.lib().fg_moe_sum(_cabi.ptr(src), _cabi.ptr(dst), m, topk, k, _cabi.DTYPE_CODE[input.dtype],
                                   _cabi.stream_ptr(input.device))
        )
    if dst is not output:
        output.copy_(dst)
    return output
