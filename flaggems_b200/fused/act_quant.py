"""act_quant: block-wise FP8 e4m3 activation quantisation.

Mirrors src/flag_gems/fused/act_quant.py:111-174 of the reference (same name,
arguments, asserts and return values); the device work is the hand-written
sm_100a kernel behind ``fg_act_quant_bf16_e4m3``.
"""
import logging
from typing import Optional, Tuple

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def act_quant_triton(
    x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``x`` (bf16, contiguous, last dim divisible by ``block_size``) per block.

    Returns ``(y, s)``: ``y`` float8_e4m3fn with the shape of ``x`` and ``s`` float32 of
    shape ``x.shape[:-1] + (N // block_size,)``.  ``scale_fmt`` not None rounds every
    scale up to a power of two.  (The name keeps the reference's ``_triton`` suffix;
    no Triton is involved.)
    """
    logger.debug("GEMS ACT_QUANT")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    assert (
        x.size(-1) % block_size == 0
    ), f"Last dimension size must be divisible by block_size (block_size={block_size})"
    _cabi.require_cuda(x)
    if x.dtype != torch.bfloat16:
        raise NotImplementedError(f"act_quant supports bfloat16 input, got {x.dtype}")

    n = x.size(-1)
    x2 = x.view(-1, n)
    m = x2.size(0)
    n_blocks = n // block_size
    y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = x.new_empty(*x.size()[:-1], n_blocks, dtype=torch.float32)
    with _cabi.device_guard(x):
        _cabi.check(
            _cabi.lib().fg_act_quant_bf16_e4m3(
                _cabi.ptr(x2), _cabi.ptr(y), _cabi.ptr(s), m, n, block_size,
                n, n, n_blocks, 0 if scale_fmt is None else 1, _cabi.stream_ptr(x.device),
            )
        )
    return y, s
