"""moe_align_block_size: sort route slots by expert and pad every expert to a block.

Mirrors src/flag_gems/fused/moe_align_block_size.py:789-820 (allocating form) and
:520-664 (out-parameter form, which keeps the reference's ``_triton`` suffix although
it launches the single cluster kernel behind ``fg_moe_align_block_size``).
"""
import logging
from typing import Optional

import torch

from .. import _cabi

logger = logging.getLogger(__name__.replace("flaggems_b200", "flag_gems", 1))


def ceil_div(a, b):
    return (a + b - 1) // b


def round_up(x: int, y: int) -> int:
    return ((x + y - 1) // y) * y


def _launch(topk_ids, num_experts, block_size, sorted_token_ids, expert_ids, num_tokens_post_pad, expert_map):
    _cabi.require_cuda(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_pad, expert_map)
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise NotImplementedError(f"topk_ids must be int32 or int64, got {topk_ids.dtype}")
    for t in (sorted_token_ids, expert_ids, num_tokens_post_pad):
        assert t.dtype == torch.int32 and t.is_contiguous()
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    emap = None
    if expert_map is not None:
        emap = expert_map.to(torch.int32).contiguous()
    with _cabi.device_guard(topk_ids):
        _cabi.check(
            _cabi.lib().fg_moe_align_block_size(
                _cabi.ptr(ids), 1 if ids.dtype == torch.int64 else 0, ids.numel(), num_experts, block_size,
                _cabi.ptr(emap), 0 if emap is None else emap.numel(),
                _cabi.ptr(sorted_token_ids), sorted_token_ids.numel(),
                _cabi.ptr(expert_ids), expert_ids.numel(), _cabi.ptr(num_tokens_post_pad),
                _cabi.stream_ptr(topk_ids.device),
            )
        )


def moe_align_block_size_triton(
    topk_ids: torch.Tensor,
    num_experts: int,
    block_size: int,
    sorted_token_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_post_pad: torch.Tensor,
) -> None:
    logger.debug("GEMS MOE ALIGN BLOCK SIZE")
    _launch(topk_ids, num_experts, block_size, sorted_token_ids, expert_ids, num_tokens_post_pad, None)


def moe_align_block_size(
    topk_ids: torch.Tensor,
    block_size: int,
    num_experts: int,
    expert_map: Optional[torch.Tensor] = None,
    pad_sorted_ids: bool = False,
) -> "tuple[torch.Tensor, torch.Tensor, torch.Tensor]":
    logger.debug("GEMS MOE ALIGN BLOCK SIZE")
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_num_tokens_padded = round_up(max_num_tokens_padded, block_size)
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=topk_ids.device)
    max_num_m_blocks = ceil_div(max_num_tokens_padded, block_size)
    expert_ids = torch.empty((max_num_m_blocks,), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1), dtype=torch.int32, device=topk_ids.device)
    _launch(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad, expert_map)
    return sorted_ids, expert_ids, num_tokens_post_pad
