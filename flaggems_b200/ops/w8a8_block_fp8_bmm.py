"""w8a8_block_fp8_bmm and fp8_einsum: batched FP8 GEMM with 1x128 activation and 128x128 weight scales.

Mirrors src/flag_gems/runtime/backend/_nvidia/hopper/ops/w8a8_block_fp8_bmm.py:629-760 and
.../hopper/ops/fp8_einsum.py:22-75 of the reference (Hopper-only there): same signatures, asserts
and stride freedom (only the last dimension of x, y and z has to be contiguous, so the permuted
views fp8_einsum passes work without copies).  Every batch entry is one launch of the block-scaled
tcgen05 GEMM (``fg_block_scaled_mm_fp8``) on that entry's pointers and strides.
"""
import logging
from typing import List, Optional

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def w8a8_block_fp8_bmm(
    x: torch.Tensor,
    y: torch.Tensor,
    xs: torch.Tensor,
    ys: torch.Tensor,
    block_size: List[int] = [128, 128],
    z: Optional[torch.Tensor] = None,
    output_dtype: torch.dtype = torch.bfloat16,
):
    """x [B, M, K] fp8, y [B, N, K] fp8, xs [B, M, K/128] fp32, ys [B, N/128, K/128] fp32 -> z [B, M, N]."""
    logger.debug("GEMS W8A8_BLOCK_FP8_BMM")
    assert len(block_size) == 2
    block_n, block_k = block_size
    assert block_n == 128 and block_k == 128, "this kernel assumes 128x128 block-wise FP8 scales"
    assert x.ndim == 3 and y.ndim == 3 and xs.ndim == 3 and ys.ndim == 3
    assert x.shape[0] == y.shape[0] == xs.shape[0] == ys.shape[0]
    assert x.shape[-1] == y.shape[-1]
    assert x.shape[:-1] == xs.shape[:-1]
    assert x.stride(-1) == 1 and y.stride(-1) == 1
    b, m, k = x.shape
    _, n, _ = y.shape
    assert k % block_k == 0 and n % block_n == 0
    if z is None:
        z = torch.empty((b, m, n), device=x.device, dtype=output_dtype)
    else:
        assert z.shape == (b, m, n) and z.device == x.device and z.dtype == output_dtype
        assert z.stride(-1) == 1
    if x.dtype != torch.float8_e4m3fn or y.dtype != torch.float8_e4m3fn:
        raise NotImplementedError(f"operands must be float8_e4m3fn, got {x.dtype} and {y.dtype}")
    if output_dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported output dtype {output_dtype}")
    _cabi.require_cuda(x, y, xs, ys, z)
    if b == 0 or m == 0 or n == 0:
        return z
    # TMA reads rows of x and y: 16-byte aligned rows (strides in bytes = elements for FP8)
    if x.stride(1) % 16 != 0 or x.stride(0) % 16 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    if y.stride(1) % 16 != 0 or y.stride(0) % 16 != 0 or y.data_ptr() % 16 != 0:
        y = y.contiguous()
    xs = xs if xs.dtype == torch.float32 else xs.float()
    ys = ys if ys.dtype == torch.float32 else ys.float()
    L, st, code = _cabi.lib(), _cabi.stream_ptr(x.device), _cabi.DTYPE_CODE[output_dtype]
    esz = z.element_size()
    with _cabi.device_guard(x):
        for i in range(b):
            _cabi.check(L.fg_block_scaled_mm_fp8(
                z.data_ptr() + i * z.stride(0) * esz, x.data_ptr() + i * x.stride(0), y.data_ptr() + i * y.stride(0),
                xs.data_ptr() + i * xs.stride(0) * 4, ys.data_ptr() + i * ys.stride(0) * 4, m, n, k, x.stride(1),
                y.stride(1), z.stride(1), xs.stride(1), xs.stride(2), ys.stride(1), ys.stride(2), code, st))
    return z


def fp8_einsum(
    equation: str,
    x: torch.Tensor,
    xs: torch.Tensor,
    y: torch.Tensor,
    ys: torch.Tensor,
    block_size: List[int] = [128, 128],
    output_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Block-wise FP8 einsum, ``"bhr,hdr->bhd"`` only: out[b,h,d] = sum_r x[b,h,r] * y[h,d,r] with
    xs [b, h, r/128] and ys [h, d/128, r/128]; h is the batch dimension of the underlying bmm."""
    assert equation == "bhr,hdr->bhd", f"fp8_einsum only supports 'bhr,hdr->bhd', got {equation!r}"
    b, h, r = x.shape
    h2, d, r2 = y.shape
    assert h2 == h and r2 == r, f"x {tuple(x.shape)} / y {tuple(y.shape)} mismatch"
    z = torch.empty((b, h, d), device=x.device, dtype=output_dtype)
    w8a8_block_fp8_bmm(x.permute(1, 0, 2), y, xs.permute(1, 0, 2), ys, block_size=block_size,
                       z=z.permute(1, 0, 2), output_dtype=output_dtype)
    return z
