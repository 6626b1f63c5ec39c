"""per_token_group_quant_fp8 with vLLM semantics.

Mirrors src/flag_gems/ops/per_token_group_quant_fp8.py:227-336 of the reference.
"""
import logging
from typing import Optional, Tuple

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))

SUPPORTED_FP8_DTYPE = torch.float8_e4m3fn


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    dtype: Optional[torch.dtype] = None,
    column_major_scales: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    logger.debug("GEMS PER TOKEN GROUP QUANT FP8")
    fp8_dtype = SUPPORTED_FP8_DTYPE if dtype is None else dtype
    assert x.shape[-1] % group_size == 0, (
        f"the last dimension of `x` {x.shape[-1]} must be divisible "
        f"by `group_size` {group_size}"
    )
    assert x.stride(-1) == 1, "`x` groups must be contiguous"
    if fp8_dtype != torch.float8_e4m3fn:
        raise NotImplementedError(f"only float8_e4m3fn output is supported, got {fp8_dtype}")
    _cabi.require_cuda(x)

    x_q = torch.empty(x.shape, device=x.device, dtype=fp8_dtype)
    k = x.shape[-1]
    if column_major_scales:
        shape = (k // group_size,) + x.shape[:-1]
        x_s = torch.empty(shape, device=x.device, dtype=torch.float32).permute(-1, -2)
    else:
        shape = x.shape[:-1] + (k // group_size,)
        x_s = torch.empty(shape, device=x.device, dtype=torch.float32)
    if x.numel() == 0:
        return x_q, x_s

    # Rows are addressed through one stride: collapse the leading dimensions.
    if x.dim() == 2:
        x2, ld_x = x, x.stride(0)
    else:
        x2 = x.reshape(-1, k)  # a view whenever the leading dims are collapsible
        ld_x = x2.stride(0)
    m = x2.shape[0]
    if column_major_scales:
        assert x.dim() == 2, "column-major scales are defined for 2-D inputs"
        s_row, s_col = x_s.stride(0), x_s.stride(1)
    else:
        s_row, s_col = k // group_size, 1
    xq2 = x_q.view(-1, k)
    with _cabi.device_guard(x):
        _cabi.check(
            _cabi.lib().fg_per_token_group_quant_fp8(
                _cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], _cabi.ptr(xq2), _cabi.ptr(x_s),
                m, k, group_size, ld_x, xq2.stride(0), s_row, s_col, float(eps),
                1 if scale_ue8m0 else 0, _cabi.stream_ptr(x.device),
            )
        )
    return x_q, x_s
