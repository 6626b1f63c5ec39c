"""topk_softmax: softmax over the experts followed by top-k selection, one launch.

Mirrors src/flag_gems/fused/topk_softmax.py:84-137 of the reference (the function vLLM's
``_moe_C::topk_softmax`` is replaced with): same arguments, same in-place outputs, the same
``topk <= 32`` assertion and TypeError for an index dtype other than int32/int64/uint32.
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))

_INDEX_KIND = {torch.int32: 0, torch.uint32: 1, torch.int64: 2}


def topk_softmax(
    topk_weights: torch.Tensor,
    topk_indices: torch.Tensor,
    token_expert_indices: torch.Tensor,
    gating_output: torch.Tensor,
    renormalize: bool = False,
    expert_counts: torch.Tensor = None,
) -> None:
    """``expert_counts`` (int32 [num_experts], optional, not in the reference) receives the number
    of route slots per expert added to its current content."""
    logger.debug("GEMS TOPK SOFTMAX")
    num_tokens, num_experts = gating_output.shape
    topk = topk_weights.size(-1)
    assert topk <= 32
    if topk_indices.dtype not in _INDEX_KIND:
        raise TypeError("topk_indices must be int32/int64/uint32")
    _cabi.require_cuda(topk_weights, topk_indices, token_expert_indices, gating_output)
    assert topk_weights.dtype == torch.float32 and token_expert_indices.dtype == torch.int32
    assert topk_weights.shape == (num_tokens, topk) and topk_indices.shape == (num_tokens, topk)
    assert token_expert_indices.shape == (num_tokens, topk)
    assert topk_weights.is_contiguous() and topk_indices.is_contiguous() and token_expert_indices.is_contiguous()
    if gating_output.dtype not in _cabi.DTYPE_CODE:
        raise NotImplementedError(f"unsupported gating dtype {gating_output.dtype}")
    g = gating_output if gating_output.is_contiguous() else gating_output.contiguous()
    if expert_counts is not None:
        assert expert_counts.dtype == torch.int32 and expert_counts.numel() >= num_experts
        assert expert_counts.is_contiguous()
    with _cabi.device_guard(g):
        _cabi.check(
            _cabi.lib().fg_topk_softmax(
                _cabi.ptr(topk_weights), _cabi.ptr(topk_indices), _INDEX_KIND[topk_indices.dtype],
                _cabi.ptr(token_expert_indices), _cabi.ptr(g), _cabi.DTYPE_CODE[g.dtype], num_tokens, num_experts,
                topk, 1 if renormalize else 0, _cabi.ptr(expert_counts), _cabi.stream_ptr(g.device),
            )
        )
