"""aten::_scaled_mm / aten::_scaled_mm.out for FP8 e4m3 operands.

Mirrors src/flag_gems/ops/scaled_mm.py:213-452 of the reference: same argument
normalisation and error messages; the product itself is ``fg_scaled_mm_fp8`` with the
bias added in fp32 before the output cast (reference kernel :116-136).  ``out_dtype=None``
resolves to the operands' dtype (:214-220): the result is then FP8 e4m3, rounded to nearest
even and saturated at +-448 (the conversion the reference's ``tl.store`` of an fp32 tile to an
fp8 pointer performs on NVIDIA hardware).
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))

SCALAR_SCALE = 0
VECTOR_SCALE = 1


def _resolve_out_dtype(self, out_dtype, out=None):
    if out_dtype is not None:
        if out is not None and out.dtype != out_dtype:
            raise RuntimeError("out_dtype must be the same as the dtype of the provided out tensor")
        return out_dtype
    if out is not None:
        return out.dtype
    return self.dtype


def _normalize_scale(scale, expected_size, *, is_left_scale):
    if scale.numel() == 1:
        return scale.reshape(1).contiguous(), SCALAR_SCALE
    valid_vector = scale.ndim == 1 and scale.shape[0] == expected_size
    if is_left_scale:
        valid_vector = valid_vector or (scale.ndim == 2 and scale.shape == (expected_size, 1))
    else:
        valid_vector = valid_vector or (scale.ndim == 2 and scale.shape == (1, expected_size))
    if valid_vector:
        return scale.reshape(expected_size).contiguous(), VECTOR_SCALE
    scale_name = "scale_a" if is_left_scale else "scale_b"
    expected_shape = f"({expected_size}, 1)" if is_left_scale else f"(1, {expected_size})"
    raise RuntimeError(f"{scale_name} must be a scalar tensor or have shape {expected_shape}")


def _normalize_bias(bias, cols):
    if bias is None:
        return None
    if bias.numel() != cols:
        raise RuntimeError(f"Bias must be size {cols} but got {bias.numel()}")
    return bias.reshape(cols).contiguous()


def _check_inputs(self, mat2):
    if self.ndim != 2:
        raise RuntimeError("self must be a matrix")
    if mat2.ndim != 2:
        raise RuntimeError("mat2 must be a matrix")
    if self.shape[1] != mat2.shape[0]:
        raise RuntimeError(
            f"mat1 and mat2 shapes cannot be multiplied ({self.shape[0]}x{self.shape[1]} "
            f"and {mat2.shape[0]}x{mat2.shape[1]})"
        )
    if self.dtype != mat2.dtype:
        raise RuntimeError(f"self and mat2 must have the same dtype, but got {self.dtype} and {mat2.dtype}")


def _scaled_mm_impl(self, mat2, scale_a, scale_b, bias, out_dtype, out):
    _check_inputs(self, mat2)
    m, k = self.shape
    _, n = mat2.shape
    output_dtype = _resolve_out_dtype(self, out_dtype, out)
    if out is None:
        out = torch.empty((m, n), dtype=output_dtype, device=self.device)
    elif out.shape != (m, n):
        raise RuntimeError("Incompatible output shape")
    scale_a, mode_a = _normalize_scale(scale_a, m, is_left_scale=True)
    scale_b, mode_b = _normalize_scale(scale_b, n, is_left_scale=False)
    bias = _normalize_bias(bias, n)
    if m == 0 or n == 0:
        return out

    _cabi.require_cuda(self, mat2, scale_a, scale_b, bias, out)
    if self.dtype != torch.float8_e4m3fn:
        raise NotImplementedError(f"_scaled_mm is implemented for float8_e4m3fn operands only, got {self.dtype}")
    fp8_out = output_dtype == torch.float8_e4m3fn
    if output_dtype not in _cabi.DTYPE_CODE and not fp8_out:
        raise NotImplementedError(f"_scaled_mm output dtype {output_dtype} is not supported (e4m3/bf16/fp16/fp32)")
    if scale_a.dtype != torch.float32 or scale_b.dtype != torch.float32:
        scale_a, scale_b = scale_a.float(), scale_b.float()
    # The tensor-core path reads both operands K-contiguous; lay them out that way if needed.
    if self.stride(1) != 1 or self.stride(0) % 16 != 0:
        self = self.contiguous()
    if mat2.stride(0) != 1 or mat2.stride(1) % 16 != 0:
        mat2 = mat2.t().contiguous().t()
    # The kernel reads the bias in the output type; with an FP8 output (out_dtype=None resolves to
    # the operands' type, reference :214-220) it reads fp32 and adds it before the saturating cast.
    bias_dtype = torch.float32 if fp8_out else output_dtype
    if bias is not None and bias.dtype != bias_dtype:
        bias = bias.to(bias_dtype)
    dst = out if out.stride(1) == 1 else torch.empty((m, n), dtype=output_dtype, device=out.device)
    with _cabi.device_guard(self):
        _cabi.check(
            _cabi.lib().fg_scaled_mm_fp8(
                _cabi.ptr(dst), _cabi.ptr(self), _cabi.ptr(mat2), _cabi.ptr(scale_a), _cabi.ptr(scale_b),
                _cabi.ptr(bias), m, n, k, self.stride(0), mat2.stride(1), dst.stride(0),
                mode_a, mode_b, _cabi.DTYPE_E4M3 if fp8_out else _cabi.DTYPE_CODE[output_dtype], 0,
                _cabi.stream_ptr(self.device),
            )
        )
    if dst is not out:
        out.copy_(dst)
    return out


def scaled_mm(self, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None, use_fast_accum=False):
    logger.debug("GEMS SCALED_MM")
    return _scaled_mm_impl(self, mat2, scale_a, scale_b, bias, out_dtype, None)


def scaled_mm_out(self, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None,
                  use_fast_accum=False, *, out):
    logger.debug("GEMS SCALED_MM_OUT")
    return _scaled_mm_impl(self, mat2, scale_a, scale_b, bias, out_dtype, out)
