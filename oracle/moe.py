"""CPU oracle: fused-MoE building blocks and whole layers (test infrastructure only)."""
from typing import Optional, Tuple

import torch

from .gemm import block_scaled_mm
from .quant import per_tensor_quant_fp8, per_token_group_quant_fp8, per_token_quant_fp8, per_token_quant_int8


def moe_align_block_size(
    topk_ids: torch.Tensor,
    block_size: int,
    num_experts: int,
    expert_map: Optional[torch.Tensor] = None,
    pad_sorted_ids: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Counting sort of route slots by expert with per-expert padding to block_size.

    Follows the reference's stable-sort golden tests/test_moe_align_block_size.py:28-123
    for the ordering (route indices ascending inside each expert) and the kernel
    API src/flag_gems/fused/moe_align_block_size.py:789-820 for the buffer sizes
    (``max_pad = numel + E*(bs-1)``, ``cdiv(max_pad, bs)`` blocks) and for
    ``expert_map``: every entry of expert_ids, the trailing -1 ones included, is
    re-indexed as ``expert_map[expert_ids]`` (:817-818), so blocks of unmapped
    experts stay in place with id -1 and trailing blocks read expert_map[-1].
    """
    numel = topk_ids.numel()
    max_pad = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_pad = (max_pad + block_size - 1) // block_size * block_size
    n_blocks = (max_pad + block_size - 1) // block_size
    flat = topk_ids.reshape(-1).to(torch.int64)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    order = torch.sort(flat, stable=True).indices
    sorted_e = flat[order]
    first_of_e = torch.cumsum(counts, 0) - counts
    pos = torch.arange(numel) - first_of_e[sorted_e]
    sorted_ids = torch.full((max_pad,), numel, dtype=torch.int32)
    sorted_ids[starts[sorted_e] + pos] = order.to(torch.int32)
    expert_ids = torch.full((n_blocks,), -1, dtype=torch.int32)
    blocks_per_e = padded // block_size
    expert_ids[: int(blocks_per_e.sum())] = torch.repeat_interleave(
        torch.arange(num_experts, dtype=torch.int32), blocks_per_e
    )
    if expert_map is not None:
        expert_ids = expert_map[expert_ids.long()].to(torch.int32)
    total = torch.tensor([int(ends[-1]) if num_experts > 0 else 0], dtype=torch.int32)
    return sorted_ids, expert_ids, total


def silu_and_mul(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """out = dtype(x32 / (1 + exp(-x32)) * y32), one rounding.

    Follows src/flag_gems/fused/fused_moe.py:795-800 (== fused/silu_and_mul.py:26-31).
    """
    xf = x.float()
    return (xf / (1.0 + torch.exp(-xf)) * y.float()).to(torch.promote_types(x.dtype, y.dtype))


def moe_sum(inp: torch.Tensor) -> torch.Tensor:
    """[M, topk, K] -> [M, K], fp32 sum over topk in slot order, cast to input dtype.

    Follows src/flag_gems/fused/moe_sum.py:57-67.
    """
    acc = torch.zeros(inp.shape[0], inp.shape[2], dtype=torch.float32)
    for k in range(inp.shape[1]):
        acc += inp[:, k, :].float()
    return acc.to(inp.dtype)


def _silu_mul_f32(z: torch.Tensor, fuse_silu: bool, dtype: torch.dtype) -> torch.Tensor:
    d = z.shape[-1] // 2
    if not fuse_silu:
        z = z.to(dtype).float()
    g, u = z[..., :d], z[..., d:]
    return (g / (1.0 + torch.exp(-g)) * u).to(dtype)


def expert_rows_block_fp8(
    rows: torch.Tensor,
    w1_e: torch.Tensor,
    w2_e: torch.Tensor,
    s1_e: torch.Tensor,
    s2_e: torch.Tensor,
    weights: torch.Tensor,
    block: int = 128,
    fuse_silu: bool = True,
    return_intermediate: bool = False,
):
    """One expert of the block-FP8 layer applied to the rows routed to it: the loop body of
    ``fused_moe_block_fp8`` below (tests/test_fused_experts_impl.py:604-662 with the device
    path's fp32 router-weight multiply, src/flag_gems/fused/fused_moe.py:1485-1493).
    rows [R, H] bf16/fp16, weights [R]; returns [R, H_out] in the rows' dtype (and the
    activation [R, I] after SiLU*up when asked)."""
    hq, hs = per_token_group_quant_fp8(rows, block)
    z = block_scaled_mm(hq, w1_e, hs, s1_e, block, block, torch.float32)
    act = _silu_mul_f32(z, fuse_silu, rows.dtype)
    aq, asc = per_token_group_quant_fp8(act, block)
    r = block_scaled_mm(aq, w2_e, asc, s2_e, block, block, torch.float32)
    r = (r * weights.float().reshape(-1, 1)).to(rows.dtype)
    return (r, act) if return_intermediate else r


def expert_rows_per_channel_fp8(
    rows: torch.Tensor,
    w1_e: torch.Tensor,
    w2_e: torch.Tensor,
    s1_e: torch.Tensor,
    s2_e: torch.Tensor,
    weights: torch.Tensor,
    fuse_silu: bool = True,
) -> torch.Tensor:
    """One expert of the per-token x per-channel FP8 layer on the rows routed to it (loop body
    of ``fused_moe_per_channel_fp8`` below; same "parity unpinned" status)."""
    hq, hs = per_token_quant_fp8(rows)
    z = torch.mm(hq.float(), w1_e.float().t()) * hs * s1_e.float().reshape(1, -1)
    act = _silu_mul_f32(z, fuse_silu, rows.dtype)
    aq, asc = per_token_quant_fp8(act)
    r = torch.mm(aq.float(), w2_e.float().t()) * asc * s2_e.float().reshape(1, -1)
    return (r * weights.float().reshape(-1, 1)).to(rows.dtype)


def fused_moe_block_fp8(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    block: int = 128,
    fuse_silu: bool = True,
    expert_lo: int = 0,
    expert_hi: Optional[int] = None,
    addend: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Block-FP8 (128x128 weight blocks, 1x128 activation groups) MoE layer.

    Skeleton of tests/test_fused_experts_impl.py:604-662: group-quantise each
    routed row, block-scaled matmul with w1[e], SiLU(gate)*up, group-quantise,
    block-scaled matmul with w2[e], weight by the router weight, sum over top-k.
    Where the reference's device path is more specific than its golden the
    device path is followed: router weight multiplied in fp32 before the bf16
    cast (src/flag_gems/fused/fused_moe.py:1485-1493) and an fp32 top-k sum
    (fused/moe_sum.py:57-67); ``fuse_silu=True`` keeps gate/up in fp32 into the
    activation as the FUSE_SILU kernel branch does (:1346-1347), False rounds
    them to bf16 first as the golden and the unfused path do.
    Only experts in [expert_lo, expert_hi) contribute (expert-parallel shards);
    w1/w2 then hold just those experts.  ``addend`` [T, H] (the shared-expert output)
    joins the top-k sum in fp32 before the single cast to the output dtype.
    """
    t, h = hidden.shape
    topk = topk_ids.shape[1]
    e_hi = w1.shape[0] + expert_lo if expert_hi is None else expert_hi
    hq, hs = per_token_group_quant_fp8(hidden, block)
    out = torch.zeros(t, topk, w2.shape[1], dtype=torch.float32)
    for e in range(expert_lo, e_hi):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        le = e - expert_lo
        z = block_scaled_mm(hq[tok], w1[le], hs[tok], w1_scale[le], block, block, torch.float32)
        act = _silu_mul_f32(z, fuse_silu, hidden.dtype)
        aq, asc = per_token_group_quant_fp8(act, block)
        r = block_scaled_mm(aq, w2[le], asc, w2_scale[le], block, block, torch.float32)
        r = (r * topk_weights[tok, slot].float().unsqueeze(1)).to(hidden.dtype)
        out[tok, slot] = r.float()
    acc = moe_sum(out)
    if addend is not None:
        acc = acc + addend.float()
    return acc.to(hidden.dtype)


def fused_moe_per_channel_fp8(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    fuse_silu: bool = True,
) -> torch.Tensor:
    """Per-token activation x per-output-channel weight FP8 MoE layer.

    PARITY UNPINNED: the reference has no test of this FP8 combination.  Restated
    from the kernel source: dynamic per-token quant (fused_moe.py:673-684),
    ``acc * a_scale * b_scale`` (:1337-1341, :1478-1479), SiLU in fp32 (:1344),
    per-token re-quantisation, router weight in fp32 then cast (:1485-1493),
    fp32 top-k sum (fused/moe_sum.py:57-67).  The layout of the computation
    follows the int8 per-channel test tests/test_fused_experts_impl.py:765-835.
    w1_scale: [E, 2I] (or [E, 2I, 1]), w2_scale: [E, H] (or [E, H, 1]).
    """
    t, h = hidden.shape
    topk = topk_ids.shape[1]
    hq, hs = per_token_quant_fp8(hidden)
    out = torch.zeros(t, topk, w2.shape[1], dtype=torch.float32)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        s1 = w1_scale[e].float().reshape(1, -1)
        s2 = w2_scale[e].float().reshape(1, -1)
        z = torch.mm(hq[tok].float(), w1[e].float().t()) * hs[tok] * s1
        act = _silu_mul_f32(z, fuse_silu, hidden.dtype)
        aq, asc = per_token_quant_fp8(act)
        r = torch.mm(aq.float(), w2[e].float().t()) * asc * s2
        r = (r * topk_weights[tok, slot].float().unsqueeze(1)).to(hidden.dtype)
        out[tok, slot] = r.float()
    return moe_sum(out).to(hidden.dtype)


def fused_moe_per_channel_int8(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
) -> torch.Tensor:
    """INT8 w8a8 MoE layer with per-token activation and per-output-channel weight scales.

    Restated from the kernel path of src/flag_gems/fused/fused_moe.py: per-token int8 quantisation of
    the rows (:732-739), exact integer accumulation (``tl.dot`` of int8 operands into int32, :1318-1331),
    ``acc.to(float32) * a_scale * b_scale`` (:1337-1341, :1478-1479), fused SiLU in fp32 (:1344),
    per-token re-quantisation, router weight in fp32 then cast (:1485-1493), fp32 top-k sum.  The
    reference's test of this mode, tests/test_fused_experts_impl.py:765-835, compares with a per-row
    fake-quantised golden; tests/test_oracle_golden.py holds that golden's output as a fixture.
    The integer products are accumulated in float64 here, which is exact for these sizes.
    w1_scale: [E, 2I] (or [E, 2I, 1]), w2_scale: [E, H] (or [E, H, 1])."""
    t, h = hidden.shape
    topk = topk_ids.shape[1]
    hq, hs = per_token_quant_int8(hidden)
    out = torch.zeros(t, topk, w2.shape[1], dtype=torch.float32)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        s1 = w1_scale[e].float().reshape(1, -1)
        s2 = w2_scale[e].float().reshape(1, -1)
        z = torch.mm(hq[tok].double(), w1[e].double().t()).float() * hs[tok] * s1
        act = _silu_mul_f32(z, True, hidden.dtype)
        aq, asc = per_token_quant_int8(act)
        r = torch.mm(aq.double(), w2[e].double().t()).float() * asc * s2
        r = (r * topk_weights[tok, slot].float().unsqueeze(1)).to(hidden.dtype)
        out[tok, slot] = r.float()
    return moe_sum(out).to(hidden.dtype)


def fused_moe_16bit(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Unquantised (bf16 / fp16) MoE layer and the weight-only int8 / int4 forms.

    Restated from src/flag_gems/fused/fused_moe.py: integer weights (int4 values live in int8
    containers) are converted to the activation type (:1976-1983); products of 16-bit operands
    accumulate in fp32 (``tl.dot``, :1468); fused SiLU in fp32 (:1344) rounded to the activation
    type; router weight in fp32 then cast (:1485-1493); fp32 top-k sum.  One deliberate difference:
    the reference multiplies the converted weights by their per-channel scale in the activation
    type before the product (one more rounding of every weight); here, as in the device path, the
    exactly converted integers are multiplied and the fp32 scale is applied to the fp32 sums, which
    is what the reference's own golden for these modes computes
    (tests/test_fused_experts_impl.py:837-872, fp32 ``w_int * scale``).
    w1: [E, 2I, H], w2: [E, H, I]; w*_scale: None or [E, N] per output channel."""
    t, h = hidden.shape
    topk = topk_ids.shape[1]
    out = torch.zeros(t, topk, w2.shape[1], dtype=torch.float32)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        z = torch.mm(hidden[tok].float(), w1[e].to(hidden.dtype).float().t())
        if w1_scale is not None:
            z = z * w1_scale[e].float().reshape(1, -1)
        act = _silu_mul_f32(z, True, hidden.dtype)
        r = torch.mm(act.float(), w2[e].to(hidden.dtype).float().t())
        if w2_scale is not None:
            r = r * w2_scale[e].float().reshape(1, -1)
        r = (r * topk_weights[tok, slot].float().unsqueeze(1)).to(hidden.dtype)
        out[tok, slot] = r.float()
    return moe_sum(out).to(hidden.dtype)


def fused_moe_per_tensor_fp8(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Per-tensor FP8 MoE layer: one scale per expert weight, one per activation tensor.

    Restated from the kernel path of src/flag_gems/fused/fused_moe.py: per-tensor quantisation of
    the hidden states (:686-698, dynamic unless a1_scale is given), ``acc * a_scale * b_scale``
    (:1478-1479), fused SiLU in fp32 (:1344), per-tensor quantisation of the whole intermediate
    [T*topk, I], router weight in fp32 then cast (:1485-1493), fp32 top-k sum.  The reference's own
    test of this mode (tests/test_fused_experts_impl.py:375-461) compares against a per-row
    fake-quantised formulation with rtol 0.5; this restatement follows the device path instead.
    """
    t, h = hidden.shape
    topk = topk_ids.shape[1]
    inter = w2.shape[2]
    hq, hs = per_tensor_quant_fp8(hidden, a1_scale)
    act = torch.zeros(t, topk, inter, dtype=hidden.dtype)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        z = torch.mm(hq[tok].float(), w1[e].float().t()) * hs * w1_scale.reshape(-1)[e].float()
        act[tok, slot] = _silu_mul_f32(z, True, hidden.dtype)
    aq, a_s = per_tensor_quant_fp8(act.reshape(t * topk, inter), a2_scale)
    aq = aq.reshape(t, topk, inter)
    out = torch.zeros(t, topk, w2.shape[1], dtype=torch.float32)
    for e in range(w1.shape[0]):
        tok, slot = torch.nonzero(topk_ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        r = torch.mm(aq[tok, slot].float(), w2[e].float().t()) * a_s * w2_scale.reshape(-1)[e].float()
        r = (r * topk_weights[tok, slot].float().unsqueeze(1)).to(hidden.dtype)
        out[tok, slot] = r.float()
    return moe_sum(out).to(hidden.dtype)


def dense_block_fp8_mlp(
    hidden: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    block: int = 128,
) -> torch.Tensor:
    """Shared-expert MLP composed from the dense ops: group quant -> block mm
    (bf16) -> silu_and_mul -> group quant -> block mm (bf16).

    The reference has no shared-expert code; this is the composition of
    per_token_group_quant_fp8 / w8a8_block_fp8_matmul / silu_and_mul that a
    DeepSeek-V3 layer built on the reference would run for the shared expert.
    """
    hq, hs = per_token_group_quant_fp8(hidden, block)
    z = block_scaled_mm(hq, w1, hs, w1_scale, block, block, hidden.dtype)
    d = z.shape[-1] // 2
    act = silu_and_mul(z[:, :d], z[:, d:])
    aq, asc = per_token_group_quant_fp8(act, block)
    return block_scaled_mm(aq, w2, asc, w2_scale, block, block, hidden.dtype)
