"""aten::_scaled_grouped_mm for FP8 e4m3 operands.

Mirrors src/flag_gems/ops/scaled_grouped_mm.py:470-583 of the reference: same argument checks
and error messages (:262-366), same four operand forms:

  A 2-D, B 3-D   rows of A grouped by ``offs``, one B per group            -> [M, N]
  A 3-D, B 3-D   one product per group                                     -> [G, M, N]
  A 3-D, B 2-D   columns of B grouped by ``offs``, one A per group         -> [M, N]
  A 2-D, B 2-D   the K range split by ``offs``, one product per K slice    -> [G, M, N]

with ``out = ((A @ B) * scale_a[:, None]) * scale_b[None, :] (+ bias in fp32)`` cast to ``out_dtype``
(bf16 by default for FP8 inputs).  The first form is the device primitive
(``fg_scaled_grouped_mm_fp8``: group ids from the offsets, alignment to 128-row tiles, row gather,
grouped tcgen05 GEMM with the rows scattered back; ``offs`` is read on the device).  The other
three are expressed through it here: the batched form as one grouped product over the flattened
rows, the B-2-D form as the transposed problem, the K-split form as products of A with everything
outside a group's K range zeroed.
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))

FP8 = torch.float8_e4m3fn


def _default_out_dtype(dtype):
    return torch.bfloat16 if dtype == FP8 else dtype


def _check_dims(mat_a, mat_b):
    if mat_a.dim() not in (2, 3):
        raise RuntimeError("mat_a has to be 2D or 3D")
    if mat_b.dim() not in (2, 3):
        raise RuntimeError("mat_b has to be 2D or 3D")
    if mat_a.dtype != mat_b.dtype:
        raise RuntimeError(f"mat_a and mat_b must have the same dtype, got {mat_a.dtype} and {mat_b.dtype}")


def _check_offsets(offs, need_offsets, num_groups):
    if need_offsets:
        if offs is None:
            raise RuntimeError("offs must be provided when either input is 2D")
        if offs.dim() != 1:
            raise RuntimeError("offs has to be 1D")
        if offs.dtype != torch.int32:
            raise RuntimeError("offs has to be int32")
        if offs.numel() != num_groups:
            raise RuntimeError(f"offs length must match the group count, got {offs.numel()} and {num_groups}")
        return offs.contiguous()
    if offs is not None:
        raise RuntimeError("offs must be None when both inputs are 3D")
    return None


def _resolve_shapes(mat_a, mat_b, offs):
    a_is_2d, b_is_2d = mat_a.dim() == 2, mat_b.dim() == 2
    need_offsets = a_is_2d or b_is_2d
    if a_is_2d:
        m, k = mat_a.shape
    else:
        groups_a, m, k = mat_a.shape
    if b_is_2d:
        bk, n = mat_b.shape
    else:
        groups_b, bk, n = mat_b.shape
    if k != bk:
        raise RuntimeError(f"mat_a and mat_b shapes cannot be multiplied ({k} and {bk})")
    if need_offsets:
        if a_is_2d and b_is_2d:
            num_groups = offs.numel() if offs is not None else 0
            out_shape = (num_groups, m, n)
        elif a_is_2d:
            num_groups, out_shape = groups_b, (m, n)
        else:
            num_groups, out_shape = groups_a, (m, n)
    else:
        if groups_a != groups_b:
            raise RuntimeError(f"matrix batch sizes have to match, got {groups_a} and {groups_b}")
        num_groups, out_shape = groups_a, (groups_a, m, n)
    offs = _check_offsets(offs, need_offsets, num_groups)
    return a_is_2d, b_is_2d, num_groups, m, n, k, out_shape, offs


def _normalize_scale(scale, mat, *, dim, num_groups, scale_multiplier, name):
    if scale.dtype != torch.float32:
        raise RuntimeError(f"{name} must be a float32 tensor")
    if mat.dim() == 2:
        expected = mat.shape[dim] * scale_multiplier
        if scale.dim() != 1 or scale.numel() != expected:
            raise RuntimeError(f"{name} must be a 1D tensor with length {expected}")
        return scale.reshape(expected).contiguous()
    expected_shape = (num_groups, mat.shape[1 + dim])
    if scale.dim() != 2 or tuple(scale.shape) != expected_shape:
        raise RuntimeError(f"{name} must have shape {expected_shape}")
    return scale.contiguous()


def _normalize_bias(bias, *, a_is_2d, b_is_2d, num_groups, n):
    if bias is None:
        return None
    if bias.dim() == 1 and bias.numel() == n:
        return bias.contiguous()
    can_use_grouped_bias = not (b_is_2d and not a_is_2d)
    if can_use_grouped_bias and bias.numel() == num_groups * n:
        return bias.reshape(num_groups, n).contiguous()
    expected = f"({n},)"
    if can_use_grouped_bias:
        expected = f"{expected} or ({num_groups}, {n})"
    raise RuntimeError(f"bias must have shape {expected}")


def _k_contiguous(w_gkn):
    """[G, K, N] operand -> its [G, N, K] storage with K contiguous (no copy when the caller passes the
    usual transposed view of a [G, N, K] tensor)."""
    w = w_gkn.transpose(-1, -2)
    return w if w.is_contiguous() else w.contiguous()


def _grouped_rows(a, w_gnk, scale_a, scale_b, offs, bias, out_dtype):
    """Device primitive: a [M, K] fp8 (rows grouped by offs), w_gnk [G, N, K] fp8 contiguous, scale_a [M],
    scale_b [G, N], bias None / fp32 [N] / fp32 [G, N]; returns [M, N]."""
    m, k = a.shape
    g, n, _ = w_gnk.shape
    if a.stride(1) != 1 or a.stride(0) % 16 != 0 or a.data_ptr() % 16 != 0:
        a = a.contiguous()
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if m == 0 or n == 0:
        return out
    L = _cabi.lib()
    need = L.fg_scaled_grouped_mm_workspace_bytes(m, g, k)
    ws = torch.empty(int(need) + 256, dtype=torch.uint8, device=a.device)
    bias_stride = 0
    if bias is not None:
        bias = bias.float().contiguous()
        bias_stride = n if bias.dim() == 2 else 0
    with _cabi.device_guard(a):
        _cabi.check(L.fg_scaled_grouped_mm_fp8(
            _cabi.ptr(out), _cabi.ptr(a), _cabi.ptr(w_gnk), _cabi.ptr(scale_a), _cabi.ptr(scale_b), _cabi.ptr(bias),
            bias_stride, _cabi.ptr(offs), g, m, n, k, a.stride(0), out.stride(0), _cabi.DTYPE_CODE[out_dtype],
            _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(a.device)))
    return out


def scaled_grouped_mm(self, mat2, scale_a, scale_b, offs=None, bias=None, scale_result=None, out_dtype=None,
                      use_fast_accum=False):
    logger.debug("GEMS SCALED_GROUPED_MM")
    if scale_result is not None:
        raise RuntimeError("scale_result is not supported for scaled_grouped_mm")
    _check_dims(self, mat2)
    a_is_2d, b_is_2d, num_groups, m, n, k, out_shape, offs = _resolve_shapes(self, mat2, offs)
    output_dtype = out_dtype or _default_out_dtype(self.dtype)
    scale_multiplier = num_groups if a_is_2d and b_is_2d else 1
    scale_a = _normalize_scale(scale_a, self, dim=0, num_groups=num_groups, scale_multiplier=scale_multiplier,
                               name="scale_a")
    scale_b = _normalize_scale(scale_b, mat2, dim=1, num_groups=num_groups, scale_multiplier=scale_multiplier,
                               name="scale_b")
    bias = _normalize_bias(bias, a_is_2d=a_is_2d, b_is_2d=b_is_2d, num_groups=num_groups, n=n)

    _cabi.require_cuda(self, mat2, scale_a, scale_b, offs, bias)
    if self.dtype != FP8:
        raise NotImplementedError(f"_scaled_grouped_mm is implemented for float8_e4m3fn operands only, got {self.dtype}")
    if output_dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"_scaled_grouped_mm output dtype {output_dtype} is not supported (bf16/fp16/fp32)")
    if k % 16 != 0:
        raise NotImplementedError(f"K = {k} must be a multiple of 16")
    dev = self.device
    if 0 in out_shape:
        return torch.empty(out_shape, dtype=output_dtype, device=dev)

    if a_is_2d and not b_is_2d:
        return _grouped_rows(self, _k_contiguous(mat2), scale_a, scale_b, offs, bias, output_dtype)

    if not a_is_2d and not b_is_2d:
        # one product per group = rows [g*M, (g+1)*M) of the flattened A against B[g]
        ends = torch.arange(1, num_groups + 1, dtype=torch.int32, device=dev) * m
        a2 = self.reshape(num_groups * m, k)
        out = _grouped_rows(a2, _k_contiguous(mat2), scale_a.reshape(-1), scale_b, ends, bias, output_dtype)
        return out.reshape(num_groups, m, n)

    if not a_is_2d and b_is_2d:
        # out[:, n_g] = A[g] @ B[:, n_g]: the transposed problem groups the rows of B^T and uses A[g] [M, K]
        # as the group's K-contiguous weight; the bias runs along the rows there, so it is added afterwards
        bt = mat2.t()
        out_t = _grouped_rows(bt, self.contiguous(), scale_b, scale_a, offs, None,
                              torch.float32 if bias is not None else output_dtype)
        if bias is None:
            return out_t.t().contiguous()
        return (out_t.t() + bias.float().reshape(1, -1)).to(output_dtype)

    # both 2-D: out[g] = A[:, k_g] @ B[k_g, :].  A copy of A per group with the bytes outside the group's K
    # range zeroed (0x00 is +0 in e4m3) turns each slice into a full-K product; offs stays on the device.
    cols = torch.arange(k, device=dev, dtype=torch.int32)
    starts = torch.cat([torch.zeros(1, dtype=torch.int32, device=dev), offs[:-1]])
    mask = ((cols[None, :] >= starts[:, None]) & (cols[None, :] < offs[:, None])).to(torch.uint8)  # [G, K]
    a_masked = (self.contiguous().view(torch.uint8)[None, :, :] * mask[:, None, :]).view(FP8)  # [G, M, K]
    w = _k_contiguous(mat2.unsqueeze(0)).expand(num_groups, n, k).contiguous()
    ends = torch.arange(1, num_groups + 1, dtype=torch.int32, device=dev) * m
    out = _grouped_rows(a_masked.reshape(num_groups * m, k), w, scale_a.reshape(-1), scale_b.reshape(num_groups, n),
                        ends, bias, output_dtype)
    return out.reshape(num_groups, m, n)
