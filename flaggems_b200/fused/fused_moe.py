"""Fused MoE layer on FP8 weights: quantise -> align -> grouped GEMM1 (+SiLU*up) ->
quantise -> grouped GEMM2 (x router weight) -> top-k sum.

Mirrors the FP8 path of src/flag_gems/fused/fused_moe.py of the reference:
``fused_experts_impl`` (:1821-2185), ``inplace_fused_experts`` / ``outplace_fused_experts``
(:2188-2290), ``_fp8_quantize`` / ``moe_kernel_quantize_input`` (:629-698, :749-773),
``MoEActivation`` (:538-577).  The two grouped GEMMs are ``fg_moe_grouped_gemm_fp8``
(tcgen05); rows are first gathered into expert-sorted padded order while they are
quantised, so the GEMMs read their A operand with plain TMA boxes.

Implemented: the FP8 w8a8 modes (block 128x128, per-token x per-channel, per-tensor) and int8
w8a8 with per-token x per-channel scales (tcgen05 kind::i8, int32 accumulation); the weight-only
(w8a16 / w4a16), MX, bias and non-SiLU options of the reference signature raise
NotImplementedError.
"""
import logging
from enum import Enum
from typing import Optional

import torch

from .. import _cabi
from .moe_align_block_size import ceil_div, moe_align_block_size
from .moe_sum import moe_sum
from .silu_and_mul import silu_and_mul_out

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))

# Rows per grouped-GEMM tile; moe_align_block_size is run with this block size inside
# the layer (the public moe_align_block_size accepts any block size).
_TILE_ROWS = 128
_CHUNK_SIZE = 32 * 1024


class MoEActivation(Enum):
    SILU = "silu"
    GELU = "gelu"
    RELU2 = "relu2"
    SWIGLUOAI = "swigluoai"
    SWIGLUSTEP = "swiglustep"
    SILU_NO_MUL = "silu_no_mul"
    GELU_NO_MUL = "gelu_no_mul"
    RELU2_NO_MUL = "relu2_no_mul"

    @property
    def is_gated(self) -> bool:
        return not self.value.endswith("_no_mul")

    @classmethod
    def from_str(cls, s: str) -> "MoEActivation":
        for member in cls:
            if member.value == s:
                return member
        valid = [m.value for m in cls]
        raise ValueError(f"Unknown MoE activation: {s!r}. Valid activations: {valid}")

    @staticmethod
    def adjust_N_for_activation(N: int, activation: "MoEActivation") -> int:
        return N if not activation.is_gated else N // 2


def _per_token_quant(x, row_index=None, index_div=1, index_limit=0, n_rows_dev=None, out_rows=None):
    """Dynamic per-row FP8 quantisation (reference: fused_moe.py:673-684), optionally
    gathering rows through ``row_index``."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    rows = x2.shape[0] if out_rows is None else out_rows
    q = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
    if rows and k:
        _cabi.check(
            _cabi.lib().fg_per_token_quant_fp8(
                _cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], _cabi.ptr(q), _cabi.ptr(s), rows, k,
                x2.stride(0), k, _cabi.ptr(row_index), index_div, index_limit, _cabi.ptr(n_rows_dev),
                _cabi.stream_ptr(x.device),
            )
        )
    return q, s


def _per_token_quant_int8(x, row_index=None, index_div=1, index_limit=0, n_rows_dev=None, out_rows=None):
    """Dynamic per-row INT8 quantisation (reference: fused_moe.py:732-739), optionally gathering rows
    through ``row_index``."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    rows = x2.shape[0] if out_rows is None else out_rows
    q = torch.empty((rows, k), dtype=torch.int8, device=x.device)
    s = torch.empty((rows, 1), dtype=torch.float32, device=x.device)
    if rows and k:
        _cabi.check(
            _cabi.lib().fg_per_token_quant_int8(
                _cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], _cabi.ptr(q), _cabi.ptr(s), rows, k,
                x2.stride(0), k, _cabi.ptr(row_index), index_div, index_limit, _cabi.ptr(n_rows_dev),
                _cabi.stream_ptr(x.device),
            )
        )
    return q, s


def _int8_quantize(A, A_scale, per_act_token, block_shape=None):
    """INT8 quantisation of MoE activations (reference: fused_moe.py:700-747); the per-token form only."""
    _cabi.require_cuda(A)
    if block_shape is not None or not per_act_token:
        raise NotImplementedError("int8 activations: only per-token quantisation is implemented")
    with _cabi.device_guard(A):
        q, s = _per_token_quant_int8(A)
    return q.reshape(A.shape), s.reshape(A.shape[:-1] + (1,))


def _group_quant(x, group, row_index=None, index_div=1, index_limit=0, n_rows_dev=None, out_rows=None):
    """Per-token-group FP8 quantisation (reference: fused_moe.py:647-659), optionally
    gathering rows through ``row_index``."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    rows = x2.shape[0] if out_rows is None else out_rows
    q = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows, k // group), dtype=torch.float32, device=x.device)
    if rows and k:
        _cabi.check(
            _cabi.lib().fg_per_token_group_quant_fp8_gather(
                _cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], _cabi.ptr(q), _cabi.ptr(s), rows, k, group,
                x2.stride(0), k, _cabi.ptr(row_index), index_div, index_limit, _cabi.ptr(n_rows_dev),
                _cabi.stream_ptr(x.device),
            )
        )
    return q, s


def _group_quant_once_then_gather(x, group, row_index, top_k, numel, n_rows_dev, out_rows):
    """The reference's order (fused_moe.py:2016-2023 quantises A once, the kernel gathers rows by
    ``sorted_token_ids // top_k``): every token is quantised once and its FP8 row and scales are
    copied to each of its places in expert order.  Same bits as quantising while gathering."""
    k = x.shape[-1]
    tq, ts = _group_quant(x, group)
    q = torch.empty((out_rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((out_rows, k // group), dtype=torch.float32, device=x.device)
    if out_rows and k:
        _cabi.check(_cabi.lib().fg_gather_rows_fp8(
            _cabi.ptr(tq), _cabi.ptr(ts), _cabi.ptr(q), _cabi.ptr(s), out_rows, k, k // group, k, k // group,
            _cabi.ptr(row_index), top_k, numel, _cabi.ptr(n_rows_dev), _cabi.stream_ptr(x.device)))
    return q, s


def _per_tensor_quant(x, scale=None, row_index=None, index_div=1, index_limit=0, n_rows_dev=None, out_rows=None,
                      amax_rows_dev=None):
    """Per-tensor FP8 quantisation (reference: fused_moe.py:686-698): with a given ``scale``
    q = x / scale; without, scale = max(max|x|, 1e-10) / 448 over the whole tensor and
    q = x * (1 / scale).  Returns (q, scale[1])."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    rows = x2.shape[0] if out_rows is None else out_rows
    q = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    L, st = _cabi.lib(), _cabi.stream_ptr(x.device)
    if scale is not None:
        s_in = scale.float().reshape(-1)[:1].contiguous()
        s_out, dynamic = s_in, 0
    else:
        s_in = torch.zeros(1, dtype=torch.float32, device=x.device)
        s_out, dynamic = torch.empty(1, dtype=torch.float32, device=x.device), 1
        if x2.shape[0] and k:
            _cabi.check(L.fg_abs_max(_cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], x2.shape[0], k, x2.stride(0),
                                     _cabi.ptr(amax_rows_dev), _cabi.ptr(s_in), st))
    if rows and k:
        _cabi.check(L.fg_per_tensor_quant_fp8(
            _cabi.ptr(x2), _cabi.DTYPE_CODE[x.dtype], _cabi.ptr(q), _cabi.ptr(s_in), dynamic, _cabi.ptr(s_out),
            rows, k, x2.stride(0), k, _cabi.ptr(row_index), index_div, index_limit, _cabi.ptr(n_rows_dev), st))
    return q, s_out


def _fp8_quantize(A, A_scale, per_act_token, block_shape=None):
    """FP8 e4m3 quantisation of MoE activations: block-wise, per-token, or per-tensor with a
    given or a dynamic scale (reference: fused_moe.py:629-698)."""
    _cabi.require_cuda(A)
    with _cabi.device_guard(A):
        if block_shape is not None:
            assert not per_act_token
            assert len(block_shape) == 2
            block_k = block_shape[1]
            assert A.size(-1) % block_k == 0
            q, s = _group_quant(A, block_k)
            return q.reshape(A.shape), s.reshape(A.shape[:-1] + (A.size(-1) // block_k,))
        if per_act_token:
            q, s = _per_token_quant(A)
            return q.reshape(A.shape), s.reshape(A.shape[:-1] + (1,))
        q, s = _per_tensor_quant(A, A_scale)
        return q.reshape(A.shape), (A_scale if A_scale is not None else s)


def moe_kernel_quantize_input(A, A_scale, quant_dtype, per_act_token_quant, block_shape=None, ocp_mx_scheme=None):
    """Quantise MoE input activations before a GEMM (reference: fused_moe.py:749-773)."""
    if ocp_mx_scheme is not None:
        raise NotImplementedError("OCP MX schemes are not implemented")
    if quant_dtype is None:
        return A, A_scale
    if quant_dtype == torch.float8_e4m3fn:
        return _fp8_quantize(A, A_scale, per_act_token_quant, block_shape)
    raise NotImplementedError(f"quant dtype {quant_dtype} is not implemented")


def _grouped_gemm(c, a, w, a_scale, w_scale, topk_weights, sorted_ids, expert_ids, num_post_pad, numel,
                  scale_mode, fuse_silu, scatter, mul_weight, block_rows=_TILE_ROWS, a_scale_per_row=None):
    e, n, k = w.shape
    c = c.view(-1, c.shape[-1])
    head = (
        _cabi.ptr(c), _cabi.ptr(a), _cabi.ptr(w), _cabi.ptr(a_scale), _cabi.ptr(w_scale),
        _cabi.ptr(topk_weights), _cabi.DTYPE_CODE.get(topk_weights.dtype, -1) if topk_weights is not None else 0,
        1,
        _cabi.ptr(sorted_ids), _cabi.ptr(expert_ids), _cabi.ptr(num_post_pad),
        a.shape[0], numel, e, n, k, a.stride(0), c.stride(0), block_rows, scale_mode,
        (0 if scale_mode == _cabi.SCALE_SCALAR else 1) if a_scale_per_row is None else int(a_scale_per_row),
        1 if fuse_silu else 0, 1 if scatter else 0, 1 if mul_weight else 0,
    )
    tail = (_cabi.DTYPE_CODE[c.dtype], _cabi.stream_ptr(a.device))
    if w.dtype in (torch.bfloat16, torch.float16):
        assert a.dtype == w.dtype, "16-bit expert GEMMs take both operands in one type"
        _cabi.check(_cabi.lib().fg_moe_grouped_gemm_16bit(*head, _cabi.DTYPE_CODE[w.dtype], *tail))
        return
    entry = _cabi.lib().fg_moe_grouped_gemm_int8 if w.dtype == torch.int8 else _cabi.lib().fg_moe_grouped_gemm_fp8
    _cabi.check(entry(*head, *tail))


def _fused_experts_16bit(hidden_states, w1, w2, topk_weights, topk_ids, inplace, weight_only, w1_scale, w2_scale,
                         global_num_experts, expert_map):
    """Unquantised bf16 / fp16 experts and the weight-only int8 / int4 forms (int4 values in int8
    containers) on the 16-bit tcgen05 grouped GEMM.  The reference converts integer weights to the
    activation type and multiplies them by their per-channel scale before its GEMM
    (fused_moe.py:1976-1983); here the integers are converted exactly and the fp32 scale is applied to
    the fp32 accumulators, one rounding fewer per weight."""
    assert hidden_states.size(1) == w1.size(2), f"Hidden size mismatch {hidden_states.size(1)} != {w1.size(2)}"
    assert topk_weights.size() == topk_ids.size(), "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous() and w2.is_contiguous(), "expert weights must be contiguous"
    assert topk_weights.stride(1) == 1
    _cabi.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, expert_map)
    dtype = hidden_states.dtype
    if dtype not in (torch.bfloat16, torch.float16):
        raise NotImplementedError(f"16-bit expert GEMMs take bf16 or fp16 activations, got {dtype}")
    num_tokens, hidden = hidden_states.shape
    e, n, _ = w1.shape
    k_out = w2.size(1)
    inter = n // 2
    assert w2.size(2) == inter, "w2 inner size must be half of w1's output size"
    if hidden % 8 or inter % 8:
        raise NotImplementedError("hidden and intermediate sizes must be multiples of 8")
    dev = hidden_states.device
    if weight_only:
        if w1.dtype != torch.int8 or w2.dtype != torch.int8:
            raise NotImplementedError("weight-only experts are int8 tensors (int4 values in int8 containers)")
        assert w1_scale is not None and w2_scale is not None, "weight-only experts need w1_scale and w2_scale"
        w1s = w1_scale.float().reshape(e, -1).contiguous()
        w2s = w2_scale.float().reshape(e, -1).contiguous()
        assert w1s.shape == (e, n) and w2s.shape == (e, k_out), "per-channel scales must be [E, N]"
        w1, w2 = w1.to(dtype), w2.to(dtype)  # exact: |v| <= 128
        scale_mode = _cabi.SCALE_VECTOR
    else:
        if w1.dtype != dtype or w2.dtype != dtype:
            raise NotImplementedError(f"unquantised expert weights must have the activation type {dtype}")
        w1s = w2s = torch.ones(e, dtype=torch.float32, device=dev)
        scale_mode = _cabi.SCALE_SCALAR
    if global_num_experts == -1:
        global_num_experts = e
    top_k = topk_ids.size(1)
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if num_tokens == 0:
        return out
    tw = topk_weights if topk_weights.dtype in _cabi.DTYPE_CODE else topk_weights.float()
    tw = tw.contiguous()
    with _cabi.device_guard(hidden_states):
        for begin in range(0, num_tokens, _CHUNK_SIZE):
            end = min(begin + _CHUNK_SIZE, num_tokens)
            h = hidden_states[begin:end]
            ids = topk_ids[begin:end]
            w = tw[begin:end].reshape(-1)
            t = end - begin
            numel = t * top_k
            sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, _TILE_ROWS, global_num_experts, expert_map)
            rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
            # rows into expert order: a byte copy of the 16-bit rows (zeros for padding rows)
            a1 = torch.empty((rows, hidden), dtype=dtype, device=dev)
            _cabi.check(_cabi.lib().fg_gather_rows_fp8(
                _cabi.ptr(h), None, _cabi.ptr(a1), None, rows, 2 * hidden, 0, 2 * h.stride(0), 1,
                _cabi.ptr(sorted_ids), top_k, numel, _cabi.ptr(post_pad), _cabi.stream_ptr(dev)))
            ones = torch.ones(rows if scale_mode == _cabi.SCALE_VECTOR else 1, dtype=torch.float32, device=dev)
            act = torch.empty((rows, inter), dtype=dtype, device=dev)
            _grouped_gemm(act, a1, w1, ones, w1s, None, sorted_ids, expert_ids, post_pad, numel, scale_mode,
                          fuse_silu=True, scatter=False, mul_weight=False)
            routed = torch.empty((t, top_k, k_out), dtype=dtype, device=dev)
            _grouped_gemm(routed, act, w2, ones, w2s, w, sorted_ids, expert_ids, post_pad, numel, scale_mode,
                          fuse_silu=False, scatter=True, mul_weight=True)
            moe_sum(routed, out[begin:end])
    return out


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    ocp_mx_scheme: Optional[str] = None,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    expert_map: Optional[torch.Tensor] = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    w1_zp: Optional[torch.Tensor] = None,
    w2_zp: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    logger.debug("GEMS FUSED MOE")
    assert activation == "silu", f"Only 'silu' activation is supported, got {activation}"
    MoEActivation.from_str(activation)
    if ocp_mx_scheme is not None:
        raise NotImplementedError("OCP MX expert formats are not implemented")
    if use_int8_w8a8 and (use_fp8_w8a8 or not per_channel_quant or block_shape is not None):
        raise NotImplementedError("int8 w8a8 is implemented for per-token x per-channel scales "
                                  "(use_int8_w8a8=True, per_channel_quant=True)")
    if w1_zp is not None or w2_zp is not None or w1_bias is not None or w2_bias is not None:
        raise NotImplementedError("zero points and expert biases are not implemented")
    if apply_router_weight_on_input:
        raise NotImplementedError("apply_router_weight_on_input is not implemented")
    weight_only = use_int8_w8a16 or use_int4_w4a16
    if weight_only or (not use_fp8_w8a8 and not use_int8_w8a8):
        if weight_only and (use_fp8_w8a8 or use_int8_w8a8):
            raise NotImplementedError("weight-only formats cannot be combined with w8a8")
        return _fused_experts_16bit(hidden_states, w1, w2, topk_weights, topk_ids, inplace, weight_only, w1_scale,
                                    w2_scale, global_num_experts, expert_map)
    if (a1_scale is not None or a2_scale is not None) and (block_shape is not None or per_channel_quant):
        raise NotImplementedError("static activation scales are implemented for the per-tensor mode only")

    assert hidden_states.size(1) == w1.size(2), f"Hidden size mismatch {hidden_states.size(1)} != {w1.size(2)}"
    assert topk_weights.size() == topk_ids.size(), "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    assert hidden_states.dtype in [torch.float32, torch.float16, torch.bfloat16]
    assert w1_scale is not None and w2_scale is not None, "FP8 weights need w1_scale and w2_scale"
    assert w1.is_contiguous() and w2.is_contiguous(), "expert weights must be contiguous"
    assert topk_weights.stride(1) == 1
    _cabi.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, expert_map)
    w_dtype = torch.int8 if use_int8_w8a8 else torch.float8_e4m3fn
    if w1.dtype != w_dtype or w2.dtype != w_dtype:
        raise NotImplementedError(f"expert weights must be {w_dtype}")

    num_tokens, hidden = hidden_states.shape
    e, n, _ = w1.shape
    k_out = w2.size(1)
    inter = n // 2
    assert w2.size(2) == inter, "w2 inner size must be half of w1's output size"
    if global_num_experts == -1:
        global_num_experts = e
    top_k = topk_ids.size(1)
    dtype = hidden_states.dtype

    if block_shape is not None:
        assert len(block_shape) == 2
        if list(block_shape) != [128, 128]:
            raise NotImplementedError(f"block_shape {block_shape}: only [128, 128] is implemented")
        assert hidden % 128 == 0 and inter % 128 == 0, "block-FP8 needs hidden and intermediate sizes divisible by 128"
        scale_mode = _cabi.SCALE_BLOCK
        w1s = w1_scale.float().contiguous()
        w2s = w2_scale.float().contiguous()
        assert w1s.shape == (e, (n + 127) // 128, hidden // 128), f"w1_scale shape {tuple(w1s.shape)}"
        assert w2s.shape == (e, (k_out + 127) // 128, inter // 128), f"w2_scale shape {tuple(w2s.shape)}"
    elif per_channel_quant:
        scale_mode = _cabi.SCALE_VECTOR
        w1s = w1_scale.float().reshape(e, -1).contiguous()
        w2s = w2_scale.float().reshape(e, -1).contiguous()
        assert w1s.shape == (e, n) and w2s.shape == (e, k_out), "per-channel scales must be [E, N]"
    else:
        scale_mode = _cabi.SCALE_SCALAR  # one scale per expert, one per activation tensor
        w1s = w1_scale.float().reshape(-1).contiguous()
        w2s = w2_scale.float().reshape(-1).contiguous()
        assert w1s.numel() == e and w2s.numel() == e, "per-tensor weight scales must hold one value per expert"

    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if num_tokens == 0:
        return out
    tw = topk_weights if topk_weights.dtype in _cabi.DTYPE_CODE else topk_weights.float()
    tw = tw.contiguous()

    with _cabi.device_guard(hidden_states):
        for begin in range(0, num_tokens, _CHUNK_SIZE):
            end = min(begin + _CHUNK_SIZE, num_tokens)
            h = hidden_states[begin:end]
            ids = topk_ids[begin:end]
            w = tw[begin:end].reshape(-1)
            t = end - begin
            numel = t * top_k

            sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, _TILE_ROWS, global_num_experts, expert_map)
            rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS

            if scale_mode == _cabi.SCALE_BLOCK:
                if top_k > 1:
                    a1, a1s = _group_quant_once_then_gather(h, 128, sorted_ids, top_k, numel, post_pad, rows)
                else:
                    a1, a1s = _group_quant(h, 128, sorted_ids, top_k, numel, post_pad, rows)
            elif scale_mode == _cabi.SCALE_VECTOR:
                quant_rows = _per_token_quant_int8 if use_int8_w8a8 else _per_token_quant
                a1, a1s = quant_rows(h, sorted_ids, top_k, numel, post_pad, rows)
            else:
                a1, a1s = _per_tensor_quant(h, a1_scale, sorted_ids, top_k, numel, post_pad, rows)
            act = torch.empty((rows, inter), dtype=dtype, device=h.device)
            _grouped_gemm(act, a1, w1, a1s, w1s, None, sorted_ids, expert_ids, post_pad, numel,
                          scale_mode, fuse_silu=True, scatter=False, mul_weight=False)
            if scale_mode == _cabi.SCALE_BLOCK:
                a2, a2s = _group_quant(act, 128, None, 1, 0, post_pad, rows)
            elif scale_mode == _cabi.SCALE_VECTOR:
                a2, a2s = quant_rows(act, None, 1, 0, post_pad, rows)
            else:
                a2, a2s = _per_tensor_quant(act, a2_scale, None, 1, 0, post_pad, rows, amax_rows_dev=post_pad)
            routed = torch.empty((t, top_k, k_out), dtype=dtype, device=h.device)
            _grouped_gemm(routed, a2, w2, a2s, w2s, w, sorted_ids, expert_ids, post_pad, numel,
                          scale_mode, fuse_silu=False, scatter=True, mul_weight=True)
            moe_sum(routed, out[begin:end])
    return out


def _dtype_of(compute_type):
    if isinstance(compute_type, torch.dtype):
        return compute_type
    name = str(compute_type)
    for key, dt in (("bfloat16", torch.bfloat16), ("bf16", torch.bfloat16), ("float16", torch.float16),
                    ("fp16", torch.float16), ("float32", torch.float32), ("fp32", torch.float32)):
        if name.endswith(key):
            return dt
    raise ValueError(f"unsupported compute_type {compute_type!r}")


def invoke_fused_moe_triton_kernel(A, B, C, A_scale, B_scale, topk_weights, sorted_token_ids, expert_ids,
                                   num_tokens_post_padded, mul_routed_weight, top_k, config, compute_type,
                                   use_fp8_w8a8=False, use_int8_w8a8=False, use_int8_w8a16=False, use_int4_w4a16=False,
                                   per_channel_quant=False, block_shape=None, B_bias=None, FUSE_SILU=False,
                                   direct_sum=False, out_top_k=1) -> None:
    """One grouped expert GEMM over rows already sorted by ``moe_align_block_size``
    (reference: fused_moe.py:1602-1727; the name is kept, the kernel is the tcgen05 grouped GEMM).

    A [M, K] FP8 with A_scale (block [M, K/128], per-token [M, 1] or per-tensor [1]); B [E, N, K];
    row ``s`` of ``sorted_token_ids`` reads A[s // top_k] and writes C.view(-1, N_out)[s];
    ``config["BLOCK_SIZE_M"]`` is the block size the ids were aligned with.
    """
    assert topk_weights is not None or not mul_routed_weight
    assert topk_weights is None or topk_weights.stride(1) == 1
    assert sorted_token_ids is None or sorted_token_ids.stride(0) == 1
    if use_int8_w8a8 or use_int8_w8a16 or use_int4_w4a16:
        raise NotImplementedError("use_fp8_w8a8 and unquantised 16-bit operands are implemented here")
    if B_bias is not None or direct_sum:
        raise NotImplementedError("expert bias and direct_sum are not implemented")
    if not use_fp8_w8a8:
        # unquantised operands (the reference's plain tl.dot branch, fused_moe.py:1468): bf16 or fp16 A and B
        assert A.dtype == B.dtype and A.dtype in (torch.bfloat16, torch.float16), "16-bit operands of one type"
        _cabi.require_cuda(A, B, C, sorted_token_ids, expert_ids, num_tokens_post_padded)
        block_rows = int(config["BLOCK_SIZE_M"])
        e, n, k = B.shape
        m = A.shape[0]
        numel = m * top_k
        assert C.dtype == _dtype_of(compute_type), "C must have the compute dtype"
        c2 = C.view(-1, n // 2 if FUSE_SILU else n)
        rows = sorted_token_ids.numel() // block_rows * block_rows
        with _cabi.device_guard(A):
            a_sorted = torch.empty((rows, k), dtype=A.dtype, device=A.device)
            _cabi.check(_cabi.lib().fg_gather_rows_fp8(
                _cabi.ptr(A), None, _cabi.ptr(a_sorted), None, rows, 2 * k, 0, 2 * A.stride(0), 1,
                _cabi.ptr(sorted_token_ids), top_k, numel, _cabi.ptr(num_tokens_post_padded),
                _cabi.stream_ptr(A.device)))
            tw = None
            if mul_routed_weight:
                tw = topk_weights if topk_weights.dtype in _cabi.DTYPE_CODE else topk_weights.float()
                tw = tw.contiguous().reshape(-1)
            one_a = torch.ones(1, dtype=torch.float32, device=A.device)
            one_b = torch.ones(e, dtype=torch.float32, device=A.device)
            _grouped_gemm(c2, a_sorted, B, one_a, one_b, tw, sorted_token_ids, expert_ids, num_tokens_post_padded,
                          numel, _cabi.SCALE_SCALAR, fuse_silu=FUSE_SILU, scatter=True, mul_weight=mul_routed_weight,
                          block_rows=block_rows, a_scale_per_row=0)
        return
    assert B_scale is not None and A_scale is not None
    _cabi.require_cuda(A, B, C, A_scale, B_scale, sorted_token_ids, expert_ids, num_tokens_post_padded)
    block_rows = int(config["BLOCK_SIZE_M"])
    e, n, k = B.shape
    m = A.shape[0]
    numel = m * top_k
    out_dtype = _dtype_of(compute_type)
    assert C.dtype == out_dtype, "C must have the compute dtype"
    n_out = n // 2 if FUSE_SILU else n
    c2 = C.view(-1, n_out)
    rows = sorted_token_ids.numel() // block_rows * block_rows
    if block_shape is not None:
        assert list(block_shape) == [128, 128], "only 128x128 blocks are implemented"
        assert ceil_div(n, 128) == B_scale.size(-2) and ceil_div(k, 128) == B_scale.size(-1)
        scale_mode, per_row, s_cols = _cabi.SCALE_BLOCK, 1, k // 128
        w_s = B_scale.float().contiguous()
    elif per_channel_quant:
        scale_mode, per_row, s_cols = _cabi.SCALE_VECTOR, 1, 1
        w_s = B_scale.float().reshape(e, -1).contiguous()
    else:
        per_row = 1 if A_scale.numel() == m and m > 1 else 0
        scale_mode, s_cols = _cabi.SCALE_SCALAR, (1 if per_row else 0)
        w_s = B_scale.float().reshape(-1).contiguous()
    with _cabi.device_guard(A):
        a_sorted = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=A.device)
        if s_cols:
            a_s = A_scale.float().reshape(m, s_cols).contiguous()
            a_s_sorted = torch.empty((rows, s_cols), dtype=torch.float32, device=A.device)
        else:
            a_s, a_s_sorted = None, A_scale.float().reshape(-1)[:1].contiguous()
        _cabi.check(_cabi.lib().fg_gather_rows_fp8(
            _cabi.ptr(A), _cabi.ptr(a_s), _cabi.ptr(a_sorted), _cabi.ptr(a_s_sorted if s_cols else None), rows, k,
            s_cols, A.stride(0), max(s_cols, 1), _cabi.ptr(sorted_token_ids), top_k, numel,
            _cabi.ptr(num_tokens_post_padded), _cabi.stream_ptr(A.device)))
        tw = None
        if mul_routed_weight:
            tw = topk_weights if topk_weights.dtype in _cabi.DTYPE_CODE else topk_weights.float()
            tw = tw.contiguous().reshape(-1)
        _grouped_gemm(c2, a_sorted, B, a_s_sorted, w_s, tw, sorted_token_ids, expert_ids, num_tokens_post_padded,
                      numel, scale_mode, fuse_silu=FUSE_SILU, scatter=True, mul_weight=mul_routed_weight,
                      block_rows=block_rows, a_scale_per_row=per_row)


def dispatch_fused_moe_kernel(A, B, C, A_scale, B_scale, B_zp, topk_weights, sorted_token_ids, expert_ids,
                              num_tokens_post_padded, mul_routed_weight, top_k, config, compute_type, use_fp8_w8a8,
                              use_int8_w8a8, use_int8_w8a16, use_int4_w4a16, per_channel_quant, block_shape=None,
                              B_bias=None, FUSE_SILU=False, direct_sum=False, out_top_k=1) -> None:
    """Reference: fused_moe.py:1730-1818.  The zero-point (wna16 / GPTQ-AWQ) branch is not implemented."""
    if B_zp is not None:
        raise NotImplementedError("zero points (weight-only quantisation) are not implemented")
    invoke_fused_moe_triton_kernel(A, B, C, A_scale, B_scale, topk_weights, sorted_token_ids, expert_ids,
                                   num_tokens_post_padded, mul_routed_weight, top_k, config, compute_type,
                                   use_fp8_w8a8, use_int8_w8a8, use_int8_w8a16, use_int4_w4a16, per_channel_quant,
                                   block_shape, B_bias, FUSE_SILU=FUSE_SILU, direct_sum=direct_sum, out_top_k=out_top_k)


def inplace_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
) -> None:
    """``fused_experts_impl(..., inplace=True)``: the result replaces ``hidden_states``; returns
    None.  Positional order and defaults are the reference's (fused_moe.py:2188-2238), which a
    custom-op registration binds positionally."""
    fused_experts_impl(
        hidden_states, w1, w2, topk_weights, topk_ids, inplace=True, activation=activation,
        apply_router_weight_on_input=apply_router_weight_on_input, use_fp8_w8a8=use_fp8_w8a8,
        use_int8_w8a8=use_int8_w8a8, use_int8_w8a16=use_int8_w8a16, use_int4_w4a16=use_int4_w4a16,
        per_channel_quant=per_channel_quant, global_num_experts=global_num_experts, w1_scale=w1_scale,
        w2_scale=w2_scale, a1_scale=a1_scale, a2_scale=a2_scale, block_shape=block_shape, w1_bias=w1_bias,
        w2_bias=w2_bias)


def outplace_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list] = None,
    w1_bias: Optional[torch.Tensor] = None,
    w2_bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``fused_experts_impl(..., inplace=False)``: returns a new tensor (reference
    fused_moe.py:2241-2290, same positional order and defaults)."""
    return fused_experts_impl(
        hidden_states, w1, w2, topk_weights, topk_ids, inplace=False, activation=activation,
        apply_router_weight_on_input=apply_router_weight_on_input, use_fp8_w8a8=use_fp8_w8a8,
        use_int8_w8a8=use_int8_w8a8, use_int8_w8a16=use_int8_w8a16, use_int4_w4a16=use_int4_w4a16,
        per_channel_quant=per_channel_quant, global_num_experts=global_num_experts, w1_scale=w1_scale,
        w2_scale=w2_scale, a1_scale=a1_scale, a2_scale=a2_scale, block_shape=block_shape, w1_bias=w1_bias,
        w2_bias=w2_bias)
