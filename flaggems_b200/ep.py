"""Expert-parallel fused MoE layer (DeepSeek-V3 shape): tokens are data-parallel, experts are
block-partitioned over the ranks of one node, and routed rows travel by all-to-all.

The reference has no dispatch/combine code: its only multi-GPU hook is the ``expert_map`` /
``-1`` convention of ``fused_experts_impl`` (src/flag_gems/fused/fused_moe.py:1350-1364,
src/flag_gems/fused/moe_align_block_size.py:817-818), which assumes replicated tokens and an
external all-reduce.  This layer keeps the per-row arithmetic of that function (block-FP8
quantisation -> grouped GEMM1 with fused SiLU*up -> re-quantisation -> grouped GEMM2 with the
router weight applied in fp32 before the bf16 cast -> fp32 top-k sum in slot order), so a
row's result does not depend on the number of ranks.

Per step and rank:
  1. order the T_loc*topk route slots by destination rank (stable), count per destination;
  2. quantise the local tokens to FP8 (1x128 groups) straight into that send order;
  3. exchange counts, then FP8 rows + scales + (local expert id, router weight) by
     ``all_to_all_single`` (NCCL over NVLink; gloo in the CPU tests);
  4. received rows: moe_align over local expert ids, gather into expert-sorted padded order,
     GEMM1(+SiLU) / quant / GEMM2(x weight), results written back in arrival order;
  5. return the bf16 rows by the reverse all-to-all;
  6. home rank: fp32 sum over the top-k slots in slot order (+ the shared-expert output) and
     one bf16 cast.
The shared expert (a dense block-FP8 MLP applied to every local token) is composed from the
dense ops of this package and runs on a side stream while the dispatch is in flight.
"""
from typing import Optional

import torch
import torch.distributed as dist

from . import _cabi
from .fused.fused_moe import _TILE_ROWS, _group_quant, _grouped_gemm
from .fused.moe_align_block_size import moe_align_block_size
from .fused.silu_and_mul import silu_and_mul
from .ops.per_token_group_quant_fp8 import per_token_group_quant_fp8
from .ops.w8a8_block_fp8_matmul import w8a8_block_fp8_matmul


class CudaMoEOps:
    """Device work of the layer: every method launches kernels of the C-ABI library."""

    def __init__(self, w1, w2, w1_scale, w2_scale, shared=None):
        self.w1, self.w2 = w1, w2
        self.w1_scale = w1_scale.float().contiguous()
        self.w2_scale = w2_scale.float().contiguous()
        self.shared = shared
        self.num_local_experts = w1.shape[0]
        self.inter = w2.shape[2]
        self.hidden = w1.shape[2]

    def route_order(self, dest, world):
        """Route slots ordered by destination rank, ascending slot index inside a rank."""
        order, _, _ = moe_align_block_size(dest, 1, world)
        return order[: dest.numel()]

    def local_routed(self, hidden, topk_ids, weight, topk):
        """Single-rank form: all experts are local, rows go straight into expert-sorted order.
        Returns the routed results as [T*topk, H] in route-slot order."""
        t = hidden.shape[0]
        numel = t * topk
        sorted_ids, expert_ids, post_pad = moe_align_block_size(topk_ids, _TILE_ROWS, self.num_local_experts)
        rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
        a1, a1s = _group_quant(hidden, 128, sorted_ids, topk, numel, post_pad, rows)
        act = torch.empty((rows, self.inter), dtype=hidden.dtype, device=hidden.device)
        _grouped_gemm(act, a1, self.w1, a1s, self.w1_scale, None, sorted_ids, expert_ids, post_pad, numel,
                      _cabi.SCALE_BLOCK, fuse_silu=True, scatter=False, mul_weight=False)
        a2, a2s = _group_quant(act, 128, None, 1, 0, post_pad, rows)
        y = torch.empty((numel, self.w2.shape[1]), dtype=hidden.dtype, device=hidden.device)
        _grouped_gemm(y, a2, self.w2, a2s, self.w2_scale, weight, sorted_ids, expert_ids, post_pad, numel,
                      _cabi.SCALE_BLOCK, fuse_silu=False, scatter=True, mul_weight=True)
        return y

    def quant_gather(self, hidden, order, topk):
        numel = order.numel()
        return _group_quant(hidden, 128, order, topk, hidden.shape[0] * topk, None, numel)

    def expert_compute(self, xq, xs, local_expert, weight, out_dtype):
        """xq/xs: R received FP8 rows + scales, local_expert int32 [R], weight fp32 [R]."""
        r = xq.shape[0]
        y = torch.empty((r, self.w2.shape[1]), dtype=out_dtype, device=xq.device)
        if r == 0:
            return y
        sorted_ids, expert_ids, post_pad = moe_align_block_size(local_expert, _TILE_ROWS, self.num_local_experts)
        rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
        k = xq.shape[1]
        a1 = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=xq.device)
        a1s = torch.empty((rows, xs.shape[1]), dtype=torch.float32, device=xq.device)
        _cabi.check(
            _cabi.lib().fg_gather_rows_fp8(
                _cabi.ptr(xq), _cabi.ptr(xs), _cabi.ptr(a1), _cabi.ptr(a1s), rows, k, xs.shape[1],
                _cabi.ptr(sorted_ids), 1, r, _cabi.ptr(post_pad), _cabi.stream_ptr(xq.device),
            )
        )
        act = torch.empty((rows, self.inter), dtype=out_dtype, device=xq.device)
        _grouped_gemm(act, a1, self.w1, a1s, self.w1_scale, None, sorted_ids, expert_ids, post_pad, r,
                      _cabi.SCALE_BLOCK, fuse_silu=True, scatter=False, mul_weight=False)
        a2, a2s = _group_quant(act, 128, None, 1, 0, post_pad, rows)
        _grouped_gemm(y, a2, self.w2, a2s, self.w2_scale, weight, sorted_ids, expert_ids, post_pad, r,
                      _cabi.SCALE_BLOCK, fuse_silu=False, scatter=True, mul_weight=True)
        return y

    def shared_expert(self, hidden):
        if self.shared is None:
            return None
        w1, w2, s1, s2 = self.shared
        hq, hs = per_token_group_quant_fp8(hidden, 128)
        z = w8a8_block_fp8_matmul(hq, w1, hs, s1, [128, 128], hidden.dtype)
        d = z.shape[-1] // 2
        act = silu_and_mul(z[:, :d], z[:, d:])
        aq, a_s = per_token_group_quant_fp8(act, 128)
        return w8a8_block_fp8_matmul(aq, w2, a_s, s2, [128, 128], hidden.dtype)

    def combine(self, rows, inv, tokens, topk, addend):
        out = torch.empty((tokens, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        if tokens == 0:
            return out
        _cabi.check(
            _cabi.lib().fg_moe_sum_indexed(
                _cabi.ptr(rows), _cabi.ptr(out), tokens, topk, rows.shape[1], _cabi.DTYPE_CODE[rows.dtype],
                _cabi.ptr(inv), _cabi.ptr(addend), _cabi.stream_ptr(rows.device),
            )
        )
        return out

    def side_stream(self, device):
        return torch.cuda.Stream(device=device)


class ExpertParallelMoE:
    """One MoE layer whose ``num_experts`` routed experts are split evenly over ``world`` ranks.

    ``w1`` [E_loc, 2I, H] / ``w2`` [E_loc, H, I] hold this rank's experts (FP8 e4m3, 128x128 block
    scales ``w1_scale`` / ``w2_scale``); rank r owns global experts [r*E_loc, (r+1)*E_loc).
    ``shared`` = (w1 [2I_s, H], w2 [H, I_s], w1_scale, w2_scale) adds a dense expert applied to
    every token.  ``group`` is a torch.distributed process group (None: default group; a
    single-rank layer needs no process group at all).
    """

    def __init__(self, w1, w2, w1_scale, w2_scale, num_experts: int, rank: int = 0, world: int = 1,
                 group=None, shared=None, ops=None):
        assert num_experts % world == 0, "experts must divide evenly over the ranks"
        assert w1.shape[0] == num_experts // world, "w1 must hold exactly this rank's experts"
        self.num_experts, self.rank, self.world, self.group = num_experts, rank, world, group
        self.num_local_experts = num_experts // world
        self.ops = ops if ops is not None else CudaMoEOps(w1, w2, w1_scale, w2_scale, shared)
        self._side = None
        self.last_counts = None  # (send_counts, recv_counts) of the latest step, for reporting

    # -- collectives ---------------------------------------------------------------------
    def _all_to_all(self, send, send_counts, recv_counts):
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        return recv

    def _exchange_counts(self, send_counts_dev):
        recv_counts_dev = torch.empty_like(send_counts_dev)
        dist.all_to_all_single(recv_counts_dev, send_counts_dev, group=self.group)
        both = torch.stack([send_counts_dev, recv_counts_dev]).cpu()  # the step's one host sync
        return both[0].tolist(), both[1].tolist()

    # -- forward ---------------------------------------------------------------------------
    def forward(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        assert hidden.dim() == 2 and hidden.is_contiguous()
        assert topk_weights.shape == topk_ids.shape and topk_ids.shape[0] == hidden.shape[0]
        tokens, topk = topk_ids.shape
        numel = tokens * topk
        ops = self.ops
        flat_ids = topk_ids.reshape(-1)
        flat_w = topk_weights.reshape(-1).float()

        # The shared expert only needs the local tokens: overlap it with the dispatch.
        shared_out, side = None, None
        if getattr(ops, "shared", None) is not None:
            if hidden.is_cuda:
                if self._side is None:
                    self._side = ops.side_stream(hidden.device)
                side = self._side
                side.wait_stream(torch.cuda.current_stream(hidden.device))
                with torch.cuda.stream(side):
                    shared_out = ops.shared_expert(hidden)
            else:
                shared_out = ops.shared_expert(hidden)

        if self.world == 1:
            y = ops.local_routed(hidden, topk_ids, flat_w, topk)
            inv = None
        else:
            dest = (flat_ids // self.num_local_experts).to(torch.int32)
            order = ops.route_order(dest, self.world)
            send_counts_dev = torch.bincount(dest, minlength=self.world).to(torch.int64)
            send_counts, recv_counts = self._exchange_counts(send_counts_dev)
            self.last_counts = (send_counts, recv_counts)
            order_l = order.long()
            xq, xs = ops.quant_gather(hidden, order, topk)
            meta = torch.stack([(flat_ids[order_l] % self.num_local_experts).to(torch.int32),
                                flat_w[order_l].view(torch.int32)], dim=1).contiguous()
            xq_r = self._all_to_all(xq.view(torch.uint8), send_counts, recv_counts).view(torch.float8_e4m3fn)
            xs_r = self._all_to_all(xs, send_counts, recv_counts)
            meta_r = self._all_to_all(meta, send_counts, recv_counts)
            y_r = ops.expert_compute(xq_r, xs_r, meta_r[:, 0].contiguous(),
                                     meta_r[:, 1].contiguous().view(torch.float32), hidden.dtype)
            y = self._all_to_all(y_r, recv_counts, send_counts)
            inv = torch.empty(numel, dtype=torch.int32, device=hidden.device)
            inv[order_l] = torch.arange(numel, dtype=torch.int32, device=hidden.device)

        if side is not None:
            main = torch.cuda.current_stream(hidden.device)
            main.wait_stream(side)
            shared_out.record_stream(main)
        return ops.combine(y, inv, tokens, topk, shared_out)

    __call__ = forward
