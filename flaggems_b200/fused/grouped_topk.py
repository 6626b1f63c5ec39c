"""grouped_topk: group-limited top-k routing (DeepSeek-V3), one launch.

Mirrors src/flag_gems/fused/grouped_topk.py:245-355 of the reference (vLLM's
``_moe_C::grouped_topk``): same arguments, argument checks and error texts, same outputs
(fp32 weights and int32 expert indices, both [num_tokens, topk]).  The sigmoid of
``scoring_func == 1`` and the two reference kernels run as one kernel.
"""
import logging

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def grouped_topk(
    scores: torch.Tensor,
    n_group: int,
    topk_group: int,
    topk: int,
    renormalize: bool,
    routed_scaling_factor: float,
    bias: torch.Tensor,
    scoring_func: int = 0,
    expert_counts: torch.Tensor = None,
):
    """``expert_counts`` (int32 [num_experts], optional, not in the reference) receives the number
    of route slots per expert added to its current content."""
    logger.debug("GEMS GROUPED TOPK")
    if scores.ndim != 2:
        raise ValueError("scores must be a 2D Tensor")
    num_tokens, num_experts = scores.shape
    if num_experts % n_group != 0:
        raise ValueError("num_experts must be divisible by n_group")
    if n_group > 32:
        raise ValueError("n_group should be smaller than or equal to 32")
    if topk > 32:
        raise ValueError("topk should be smaller than or equal to 32 for now")
    if scoring_func not in (0, 1):
        raise ValueError("scoring_func must be 0 (none) or 1 (sigmoid)")
    if bias.dtype != scores.dtype:
        bias = bias.to(scores.dtype)
    if bias.ndim != 1:
        bias = bias.flatten()
    if len(bias) != num_experts:
        raise ValueError(f"bias length ({len(bias)}) must match num_experts ({num_experts})")
    if scores.dtype not in _cabi.DTYPE_CODE:
        raise ValueError(f"Unsupported dtype: {scores.dtype}")
    _cabi.require_cuda(scores, bias)
    if scores.stride(1) != 1:
        scores = scores.contiguous()
    bias = bias.contiguous()
    topk_values = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.float32)
    topk_indices = torch.empty((num_tokens, topk), device=scores.device, dtype=torch.int32)
    if expert_counts is not None:
        assert expert_counts.dtype == torch.int32 and expert_counts.numel() >= num_experts
        assert expert_counts.is_contiguous()
    with _cabi.device_guard(scores):
        _cabi.check(
            _cabi.lib().fg_grouped_topk(
                _cabi.ptr(topk_values), _cabi.ptr(topk_indices), _cabi.ptr(scores), _cabi.ptr(bias),
                _cabi.DTYPE_CODE[scores.dtype], num_tokens, num_experts, scores.stride(0) if num_tokens > 0 else num_experts,
                n_group, topk_group, topk, 1 if renormalize else 0, float(routed_scaling_factor), scoring_func,
                _cabi.ptr(expert_counts), _cabi.stream_ptr(scores.device),
            )
        )
    return topk_values, topk_indices
