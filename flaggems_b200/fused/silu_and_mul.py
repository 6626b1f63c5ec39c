"""silu_and_mul: out = silu(A) * B with fp32 math.

Mirrors src/flag_gems/fused/silu_and_mul.py:26-31,62-69 of the reference.
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def _as_rows(t):
    n = t.shape[-1]
    if t.dim() == 2 and t.stride(1) == 1:
        return t, t.shape[0], n, t.stride(0)
    t = t.contiguous()
    return t, t.numel() // max(n, 1), n, n


def silu_and_mul_out(A, B, out):
    logger.debug("GEMS SILU AND MUL OUT")
    assert A.shape == B.shape == out.shape, "silu_and_mul: shape mismatch"
    assert A.dtype == B.dtype == out.dtype, "silu_and_mul: dtype mismatch"
    _cabi.require_cuda(A, B, out)
    if A.dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported dtype {A.dtype}")
    if A.numel() == 0:
        return out
    a2, m, n, lda = _as_rows(A)
    b2, _, _, ldb = _as_rows(B)
    if out.dim() == 2 and out.stride(1) == 1:
        o2, ldo = out, out.stride(0)
    else:
        assert out.is_contiguous(), "out must be 2-D row-major or contiguous"
        o2, ldo = out, n
    with _cabi.device_guard(A):
        _cabi.check(
            _cabi.lib().fg_silu_and_mul(
                _cabi.ptr(a2), _cabi.ptr(b2), _cabi.ptr(o2), m, n, lda, ldb, ldo,
                _cabi.DTYPE_CODE[A.dtype], _cabi.stream_ptr(A.device),
            )
        )
    return out


def silu_and_mul(A, B):
    logger.debug("GEMS SILU AND MUL")
    out = torch.empty(A.shape, dtype=torch.promote_types(A.dtype, B.dtype), device=A.device)
    if A.dtype != out.dtype:
        A = A.to(out.dtype)
    if B.dtype != out.dtype:
        B = B.to(out.dtype)
    return silu_and_mul_out(A, B, out)
