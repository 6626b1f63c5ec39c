"""Expert-parallel fused MoE layer (DeepSeek-V3 shape): tokens are data-parallel, experts are
block-partitioned over the ranks of one node, and routed rows travel by all-to-all.

The reference has no dispatch/combine code: its only multi-GPU hook is the ``expert_map`` /
``-1`` convention of ``fused_experts_impl`` (src/flag_gems/fused/fused_moe.py:1350-1364,
src/flag_gems/fused/moe_align_block_size.py:817-818), which assumes replicated tokens and an
external all-reduce.  This layer keeps the per-row arithmetic of that function (block-FP8
quantisation -> grouped GEMM1 with fused SiLU*up -> re-quantisation -> grouped GEMM2 with the
router weight applied in fp32 before the bf16 cast -> fp32 top-k sum in slot order), so a
routed row's result does not depend on the number of ranks.  (The shared expert is a dense GEMM
over the rank's own tokens; its tile and split-K choice follows that token count, so its last
bit may.)

Per step and rank:
  1. order the T_loc*topk route slots by destination rank (stable), count per destination;
  2. quantise the local tokens to FP8 (1x128 groups) straight into that send order; the rows
     (FP8 payload + scales + local expert id, router weight, home slot, home rank) either go into
     this rank's region of the destination's receive buffer over NVLink peer memory from inside
     the quantisation kernel ("p2p"), or travel by ``all_to_all_single`` (NCCL; gloo in the CPU
     tests);
  3. counts reach the receivers by an all-gather that doubles as the "rows have landed" barrier;
  4. received rows: moe_align over local expert ids, gather into expert-sorted padded order,
     GEMM1(+SiLU) / quant / GEMM2(x weight); GEMM2's epilogue stores each result row into the home
     rank's combine buffer over peer memory (or rows return by the reverse all-to-all);
  5. home rank: fp32 sum over the top-k slots in slot order (+ the shared-expert output) and
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


def balanced_expert_placement(counts: torch.Tensor, world: int) -> torch.Tensor:
    """Static expert placement from routing statistics: returns ``slot`` with
    ``slot[logical_expert] = rank * E_loc + local_index`` such that every rank holds exactly
    E/world experts and the routed rows per rank are as even as a greedy longest-first
    assignment makes them.  With a skewed router (a few experts take most of the rows) the
    contiguous placement leaves one rank with several times the average load; the layer's
    step time is the slowest rank's.  The placement only renames experts: per-row arithmetic
    is untouched."""
    e = counts.numel()
    assert e % world == 0
    cap = e // world
    load = [0] * world
    used = [0] * world
    slot = torch.empty(e, dtype=torch.int64)
    for ex in torch.argsort(counts.cpu(), descending=True, stable=True).tolist():
        r = min((r for r in range(world) if used[r] < cap), key=lambda r: (load[r], r))
        slot[ex] = r * cap + used[r]
        used[r] += 1
        load[r] += int(counts[ex])
    return slot


def packed_row_bytes(hidden: int) -> int:
    """Bytes of one dispatch row: FP8 payload, 1x128 group scales, then int32 local expert, fp32
    router weight, int32 route slot at the home rank, int32 home rank; a multiple of 16."""
    return (hidden + 4 * (hidden // 128) + 16 + 15) // 16 * 16


class SymmetricBuffers:
    """``count`` device buffers of ``nbytes`` on every rank, each mapped into every other rank of
    the node through CUDA IPC.  ``ptrs[i][r]`` is the address, valid in this process, of buffer i
    of rank r.  Creation is collective over ``group``; so is :meth:`close`."""

    def __init__(self, nbytes, count, rank, world, group=None):
        import ctypes

        L = _cabi.lib()
        self.nbytes, self.count, self.rank, self.world, self.group = nbytes, count, rank, world, group
        self.local, handles = [], []
        for _ in range(count):
            ptr = ctypes.c_void_p()
            h = (ctypes.c_ubyte * 64)()
            _cabi.check(L.fg_symm_alloc(nbytes, ctypes.byref(ptr), h))
            self.local.append(ptr.value)
            handles.append(bytes(h))
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        self.ptrs, self._opened = [], []
        for i in range(count):
            row = []
            for r in range(world):
                if r == rank:
                    row.append(self.local[i])
                else:
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r][i])
                    _cabi.check(L.fg_symm_open(buf, ctypes.byref(ptr)))
                    row.append(ptr.value)
                    self._opened.append(ptr.value)
            self.ptrs.append(row)
        self.ptr_arrays = [(ctypes.c_void_p * world)(*row) for row in self.ptrs]
        dist.barrier(group=group)

    def close(self):
        """Collective: unmaps the peers' buffers, waits until every rank has done so, then frees
        this rank's buffers.  The caller has already made sure that no kernel that touches the
        buffers is in flight on any rank (device synchronise + barrier)."""
        L = _cabi.lib()
        for p in self._opened:
            L.fg_symm_close(p)
        self._opened = []
        if self.local:
            dist.barrier(group=self.group)
        for p in self.local:
            L.fg_symm_free(p)
        self.local, self.ptrs, self.ptr_arrays = [], [], []


class CudaMoEOps:
    """Device work of the layer: every method launches kernels of the C-ABI library.  Workspaces
    are cached between steps, so a steady-state step allocates only its outputs."""

    def __init__(self, w1, w2, w1_scale, w2_scale, shared=None):
        self.w1, self.w2 = w1, w2
        self.w1_scale = w1_scale.float().contiguous()
        self.w2_scale = w2_scale.float().contiguous()
        self.shared = shared
        self.num_local_experts = w1.shape[0]
        self.inter = w2.shape[2]
        self.hidden = w1.shape[2]
        self.row_bytes = packed_row_bytes(self.hidden)
        self._ws = None

    def _workspace(self, n_rows, device):
        need = _cabi.lib().fg_moe_routed_workspace_bytes(n_rows, self.num_local_experts, self.hidden, self.inter)
        if self._ws is None or self._ws.numel() < need or self._ws.device != device:
            self._ws = torch.empty(int(need * 1.25) + 256, dtype=torch.uint8, device=device)
        return self._ws

    def plan_and_pack(self, hidden, topk_ids, topk_w, world, rank):
        """Orders the route slots by destination rank (stable), counts rows per destination and
        writes the packed dispatch rows in that order.  Returns (packed [numel, row_bytes] uint8,
        counts int32 [world] on the device, inv int32 [numel]: row of each route slot)."""
        t, topk = topk_ids.shape
        numel = t * topk
        dev = hidden.device
        order = torch.empty(numel, dtype=torch.int32, device=dev)
        blocks = torch.empty(numel + 1, dtype=torch.int32, device=dev)
        meta = torch.empty(world + 1, dtype=torch.int32, device=dev)  # [0]: post_pad, [1:]: counts
        inv = torch.empty(numel, dtype=torch.int32, device=dev)
        packed = torch.empty((numel, self.row_bytes), dtype=torch.uint8, device=dev)
        L, st = _cabi.lib(), _cabi.stream_ptr(dev)
        ids64 = 1 if topk_ids.dtype == torch.int64 else 0
        _cabi.check(L.fg_moe_align_block_size_ex(
            _cabi.ptr(topk_ids), ids64, numel, world, 1, None, 0, _cabi.ptr(order), numel, _cabi.ptr(blocks),
            numel + 1, _cabi.ptr(meta), 1, self.num_local_experts, meta.data_ptr() + 4, None, st))
        _cabi.check(L.fg_ep_pack_rows_fp8(
            _cabi.ptr(hidden), _cabi.DTYPE_CODE[hidden.dtype], t, self.hidden, hidden.stride(0),
            _cabi.ptr(topk_ids), ids64, _cabi.ptr(topk_w), _cabi.DTYPE_CODE[topk_w.dtype], topk,
            self.num_local_experts, rank, _cabi.ptr(order), _cabi.ptr(packed), self.row_bytes, _cabi.ptr(inv), st))
        return packed, meta[1:], inv

    def route(self, topk_ids, world):
        """Route slots ordered by destination rank (stable) and rows per destination, on the device."""
        numel = topk_ids.numel()
        dev = topk_ids.device
        order = torch.empty(numel, dtype=torch.int32, device=dev)
        meta = torch.empty(world + 1, dtype=torch.int32, device=dev)
        _cabi.check(_cabi.lib().fg_moe_align_block_size_ex(
            _cabi.ptr(topk_ids), 1 if topk_ids.dtype == torch.int64 else 0, numel, world, 1, None, 0,
            _cabi.ptr(order), numel, None, 0, _cabi.ptr(meta), 1, self.num_local_experts,
            meta.data_ptr() + 4, None, _cabi.stream_ptr(dev)))
        return order, meta[1:]

    def pack_to_peers(self, hidden, topk_ids, topk_w, order, send_counts, world, rank, peer_rows, region_rows):
        """Quantises the local tokens and stores every packed row directly into this rank's region
        of its destination rank's receive buffer (``send_counts``: rows per destination, on the
        device; rows beyond a region are dropped by the kernel and reported in the status word)."""
        t, topk = topk_ids.shape
        dev = hidden.device
        # staging rows: every token is quantised once there, then copied to its top-k destinations
        stage = getattr(self, "_stage", None)
        if stage is None or stage.shape[0] < t or stage.device != dev:
            stage = torch.empty((max(t, 1), self.row_bytes), dtype=torch.uint8, device=dev)
            self._stage = stage
        _cabi.check(_cabi.lib().fg_ep_pack_rows_fp8_peer(
            _cabi.ptr(hidden), _cabi.DTYPE_CODE[hidden.dtype], t, self.hidden, hidden.stride(0),
            _cabi.ptr(topk_ids), 1 if topk_ids.dtype == torch.int64 else 0, _cabi.ptr(topk_w),
            _cabi.DTYPE_CODE[topk_w.dtype], topk, self.num_local_experts, rank, _cabi.ptr(order), _cabi.ptr(stage),
            self.row_bytes, None, _cabi.ptr(send_counts), peer_rows, world, region_rows, _cabi.stream_ptr(dev)))

    def experts_from_buffer(self, rows_ptr, world, region_rows, counts_matrix, rank, out_dtype, device, peer_out,
                            peer_rows):
        """Routed-expert pipeline on the rows that peers stored into this rank's receive buffer:
        region s of the buffer holds counts_matrix[s, rank] rows (read on the device); results go
        to the home ranks' combine buffers of ``peer_rows`` rows each."""
        capacity = world * region_rows
        ws = self._workspace(capacity, device)
        _cabi.check(_cabi.lib().fg_moe_routed_block_fp8_packed(
            None, rows_ptr, capacity, self.row_bytes, _cabi.ptr(self.w1), _cabi.ptr(self.w2),
            _cabi.ptr(self.w1_scale), _cabi.ptr(self.w2_scale), self.num_local_experts, self.hidden, self.inter,
            _cabi.ptr(ws), ws.numel(), _cabi.DTYPE_CODE[out_dtype], peer_out, len(peer_out), peer_rows, None,
            region_rows, counts_matrix.data_ptr() + 4 * rank, world, _cabi.stream_ptr(device)))

    def experts_packed(self, packed, out_dtype, peer_out=None, peer_rows=0):
        """Routed-expert pipeline on R received packed rows.  Without ``peer_out`` the result is
        returned as [R, H] in arrival order; with it (a ctypes array of one buffer address per
        rank, each buffer ``peer_rows`` rows) GEMM2 stores every row into its home rank's buffer
        and None is returned."""
        r = packed.shape[0]
        y = None
        if peer_out is None:
            y = torch.empty((r, self.w2.shape[1]), dtype=out_dtype, device=packed.device)
        if r == 0:
            return y
        ws = self._workspace(r, packed.device)
        _cabi.check(_cabi.lib().fg_moe_routed_block_fp8_packed(
            _cabi.ptr(y), _cabi.ptr(packed), r, self.row_bytes, _cabi.ptr(self.w1), _cabi.ptr(self.w2),
            _cabi.ptr(self.w1_scale), _cabi.ptr(self.w2_scale), self.num_local_experts, self.hidden, self.inter,
            _cabi.ptr(ws), ws.numel(), _cabi.DTYPE_CODE[out_dtype], peer_out,
            0 if peer_out is None else len(peer_out), peer_rows, None, 0, None, 0,
            _cabi.stream_ptr(packed.device)))
        return y

    def combine_slots(self, buf_ptr, tokens, topk, dtype, device, addend):
        """Top-k sum over a [tokens*topk, H] buffer given by address (rows in route-slot order)."""
        out = torch.empty((tokens, self.w2.shape[1]), dtype=dtype, device=device)
        if tokens:
            _cabi.check(_cabi.lib().fg_moe_sum_indexed(
                buf_ptr, _cabi.ptr(out), tokens, topk, self.w2.shape[1], _cabi.DTYPE_CODE[dtype], None,
                _cabi.ptr(addend), _cabi.stream_ptr(device)))
        return out

    def local_routed(self, hidden, topk_ids, topk_w):
        """Single-rank form: all experts are local.  Result [T*topk, H] in route-slot order."""
        t, topk = topk_ids.shape
        y = torch.empty((t * topk, self.w2.shape[1]), dtype=hidden.dtype, device=hidden.device)
        if t == 0:
            return y
        ws = self._workspace(t * topk, hidden.device)
        _cabi.check(_cabi.lib().fg_moe_routed_block_fp8_local(
            _cabi.ptr(y), _cabi.ptr(hidden), _cabi.DTYPE_CODE[hidden.dtype], _cabi.ptr(topk_ids),
            1 if topk_ids.dtype == torch.int64 else 0, _cabi.ptr(topk_w), _cabi.DTYPE_CODE[topk_w.dtype], t, topk,
            _cabi.ptr(self.w1), _cabi.ptr(self.w2), _cabi.ptr(self.w1_scale), _cabi.ptr(self.w2_scale),
            self.num_local_experts, self.hidden, self.inter, _cabi.ptr(ws), ws.numel(),
            _cabi.stream_ptr(hidden.device)))
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


TRANSPORTS = ("a2a", "p2p_combine", "p2p")


class ExpertParallelMoE:
    """One MoE layer whose ``num_experts`` routed experts are split evenly over ``world`` ranks.

    ``w1`` [E_loc, 2I, H] / ``w2`` [E_loc, H, I] hold this rank's experts (FP8 e4m3, 128x128 block
    scales ``w1_scale`` / ``w2_scale``); rank r owns global experts [r*E_loc, (r+1)*E_loc).
    ``shared`` = (w1 [2I_s, H], w2 [H, I_s], w1_scale, w2_scale) adds a dense expert applied to
    every token.  ``group`` is a torch.distributed process group (None: default group; a
    single-rank layer needs no process group at all).

    ``transport`` is fixed at construction and must be the same on every rank, so that all ranks
    issue the same collectives in every step whatever their token counts:
      "a2a"          rows and results travel by ``all_to_all_single`` (one host wait per step);
      "p2p_combine"  dispatch by all-to-all, combine fused into GEMM2 over peer memory;
      "p2p"          dispatch fused into the quantisation kernel as well: no host wait, two small
                     collectives per step (the count all-gather and one barrier).
    The peer-memory transports need ``max_slots_per_rank`` = the largest tokens * topk any rank will
    pass in one step; a step beyond it raises before anything is launched.  Call :meth:`close`
    (collective) before the process group is destroyed.
    """

    def __init__(self, w1, w2, w1_scale, w2_scale, num_experts: int, rank: int = 0, world: int = 1,
                 group=None, shared=None, ops=None, transport: str = "a2a", max_slots_per_rank: int = 0):
        assert num_experts % world == 0, "experts must divide evenly over the ranks"
        assert w1.shape[0] == num_experts // world, "w1 must hold exactly this rank's experts"
        assert transport in TRANSPORTS, f"transport must be one of {TRANSPORTS}"
        assert 0 <= rank < world
        self.num_experts, self.rank, self.world, self.group = num_experts, rank, world, group
        self.num_local_experts = num_experts // world
        self.ops = ops if ops is not None else CudaMoEOps(w1, w2, w1_scale, w2_scale, shared)
        self._side = None
        self.last_counts = None  # (send_counts, recv_counts) of the latest all-to-all step, for reporting
        self.trace = None  # set to a list to collect (phase name, CUDA event) marks of a step
        if world == 1 or ops is not None:
            transport = "a2a"  # one rank exchanges nothing; the CPU stand-ins have no peer memory
        self.transport = transport
        self.max_slots = int(max_slots_per_rank)
        self._symm = self._recv = None
        self._graph = None
        if world > 1 and dist.get_world_size(group) != world:
            raise ValueError(f"the process group has {dist.get_world_size(group)} ranks, the layer was "
                             f"built for {world}")
        if transport != "a2a":
            assert self.max_slots > 0, "the peer-memory transports need max_slots_per_rank"
            hidden_size = w1.shape[2]
            # Combine buffer: one bf16/fp16 row per route slot of this rank, written by the ranks
            # that hold the slot's expert (GEMM2's epilogue) and read by the top-k sum here.
            self._symm = SymmetricBuffers(self.max_slots * hidden_size * 2, 1, rank, world, group)
            self._flag = torch.zeros(1, dtype=torch.float32, device=w1.device)
        if transport == "p2p":
            # Receive buffer: `world` regions of max_slots rows; source rank s writes only region s,
            # so nobody needs anybody's counts before sending.  One buffer is enough: a peer's next
            # step cannot store into it before this rank has entered the collective that follows
            # its own reads (every step is ordered on one stream per rank), see forward().
            self._recv = SymmetricBuffers(world * self.max_slots * self.ops.row_bytes, 1, rank, world, group)
            self._counts_matrix = torch.zeros(world * world, dtype=torch.int32, device=w1.device)

    def _mark(self, name, device):
        if self.trace is not None and device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(device))
            self.trace.append((name, ev))

    # -- collectives ---------------------------------------------------------------------
    def _all_to_all(self, send, send_counts, recv_counts):
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        return recv

    def _exchange_counts(self, send_counts_dev):
        recv_counts_dev = torch.empty_like(send_counts_dev)
        dist.all_to_all_single(recv_counts_dev, send_counts_dev, group=self.group)
        both = torch.stack([send_counts_dev, recv_counts_dev]).cpu()  # the step's one host wait
        return both[0].tolist(), both[1].tolist()

    # -- forward ---------------------------------------------------------------------------
    def forward(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        assert hidden.dim() == 2 and hidden.is_contiguous()
        assert topk_weights.shape == topk_ids.shape and topk_ids.shape[0] == hidden.shape[0]
        tokens, topk = topk_ids.shape
        ops = self.ops
        dev = hidden.device
        # Everything that can refuse the step does so here, before the first launch or collective.
        if self.transport != "a2a":
            if tokens * topk > self.max_slots:
                raise ValueError(f"{tokens} tokens x top-{topk} = {tokens * topk} route slots exceed "
                                 f"max_slots_per_rank = {self.max_slots}")
            if hidden.dtype not in (torch.bfloat16, torch.float16):
                raise TypeError("the peer-memory transports carry bf16 or fp16 rows")
        topk_ids = topk_ids.contiguous()
        topk_weights = topk_weights.contiguous()
        if topk_weights.dtype not in _cabi.DTYPE_CODE:
            topk_weights = topk_weights.float()

        # The shared expert only needs the local tokens: overlap it with the dispatch.
        shared_out, side = None, None
        if getattr(ops, "shared", None) is not None:
            if hidden.is_cuda:
                if self._side is None:
                    self._side = ops.side_stream(dev)
                side = self._side
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    shared_out = ops.shared_expert(hidden)
            else:
                shared_out = ops.shared_expert(hidden)

        def join_shared():
            if side is not None:
                main = torch.cuda.current_stream(dev)
                main.wait_stream(side)
                shared_out.record_stream(main)

        self._mark("start", dev)
        if self.world == 1:
            y = ops.local_routed(hidden, topk_ids, topk_weights)
            self._mark("experts", dev)
            join_shared()
            out = ops.combine(y, None, tokens, topk, shared_out)
            self._mark("sum", dev)
            return out

        if self.transport == "p2p":
            # Device-driven step: no host wait, no payload through NCCL.  Ordering between ranks
            # comes from the two collectives, which sit on the same stream as the kernels:
            #  * the count all-gather completes on a rank only after every rank has launched it,
            #    i.e. after every rank's pack kernel (and its peer stores) has finished;
            #  * the barrier completes only after every rank's GEMM2 (and its peer stores) has.
            # The same two facts protect the single receive / combine buffers across steps: a
            # peer's pack of step k+1 follows its barrier of step k, which needs this rank to have
            # queued that barrier behind its own reads of step k; a peer's GEMM2 of step k+1
            # follows its all-gather of step k+1, which this rank queues behind its top-k sum of step k.
            order, counts_dev = ops.route(topk_ids, self.world)
            self._mark("route", dev)
            ops.pack_to_peers(hidden, topk_ids, topk_weights, order, counts_dev, self.world, self.rank,
                              self._recv.ptr_arrays[0], self.max_slots)
            self._mark("pack+dispatch", dev)
            dist.all_gather_into_tensor(self._counts_matrix, counts_dev.contiguous(), group=self.group)
            self._mark("counts", dev)
            ops.experts_from_buffer(self._recv.local[0], self.world, self.max_slots, self._counts_matrix, self.rank,
                                    hidden.dtype, dev, self._symm.ptr_arrays[0], self.max_slots)
            self._mark("experts+combine", dev)
            dist.all_reduce(self._flag, group=self.group)  # every rank's GEMM2 has finished
            self._mark("barrier", dev)
            join_shared()
            out = ops.combine_slots(self._symm.local[0], tokens, topk, hidden.dtype, dev, shared_out)
            self._mark("sum", dev)
            return out

        packed, counts_dev, inv = ops.plan_and_pack(hidden, topk_ids, topk_weights, self.world, self.rank)
        self._mark("route+pack", dev)
        send_counts, recv_counts = self._exchange_counts(counts_dev)
        self.last_counts = (send_counts, recv_counts)
        self._mark("counts", dev)
        packed_r = self._all_to_all(packed, send_counts, recv_counts)
        self._mark("dispatch", dev)
        if self.transport == "p2p_combine":
            ops.experts_packed(packed_r, hidden.dtype, self._symm.ptr_arrays[0], self.max_slots)
            self._mark("experts+combine", dev)
            # every rank's GEMM2 has finished once this stream-ordered collective completes
            dist.all_reduce(self._flag, group=self.group)
            self._mark("barrier", dev)
            join_shared()
            out = ops.combine_slots(self._symm.local[0], tokens, topk, hidden.dtype, dev, shared_out)
        else:
            y_r = ops.experts_packed(packed_r, hidden.dtype)
            self._mark("experts", dev)
            y = self._all_to_all(y_r, recv_counts, send_counts)
            self._mark("combine_a2a", dev)
            join_shared()
            out = ops.combine(y, inv, tokens, topk, shared_out)
        self._mark("sum", dev)
        return out

    __call__ = forward

    # -- CUDA-graph replay -------------------------------------------------------------------
    def capture(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> None:
        """Record the whole step (every kernel of this rank, the side-stream fork for the shared
        expert and, with several ranks, the stream-ordered count all-gather and barrier) into one
        CUDA graph, so that a step costs the host one launch whatever the host is busy with.

        The three tensors become the step's static inputs: write new values into them (``copy_``)
        and call :meth:`replay`.  With several ranks every rank must call ``capture`` and
        ``replay`` the same number of times, and :meth:`close` (or :meth:`release_graphs`) before
        the process group is destroyed.  Only the "p2p" transport can be recorded (the all-to-all
        variants wait on the host for their counts)."""
        assert hidden.is_cuda, "graphs are a CUDA feature"
        dev = hidden.device
        assert self.world == 1 or self.transport == "p2p", "only the device-driven step can be recorded"
        self.trace = None
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):  # warm up off the default stream: lazy initialisation, allocator pools
            for _ in range(2):
                self.forward(hidden, topk_weights, topk_ids)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        launches0 = _cabi.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            out = self.forward(hidden, topk_weights, topk_ids)
        self._graph, self._graph_out = g, out
        self.kernels_per_replay = _cabi.launch_count() - launches0
        self._graph_inputs = (hidden, topk_weights, topk_ids)

    def release_graphs(self) -> None:
        """Destroy the recorded graph.  With several ranks this must happen before the process
        group is destroyed: the graph holds NCCL kernels."""
        if self._graph is not None:
            torch.cuda.synchronize()
            self._graph, self._graph_out, self._graph_inputs = None, None, None
            torch.cuda.synchronize()

    def replay(self) -> torch.Tensor:
        """One step from the recorded graph; returns the graph's static output tensor (overwritten
        by the next replay)."""
        self._graph.replay()
        return self._graph_out

    def close(self) -> None:
        """Collective, ordered teardown: graphs released, device idle, all ranks past their last
        step, peer mappings closed on every rank, and only then the shared buffers freed.  After
        it the process group may be destroyed."""
        self.release_graphs()
        if self._symm is None and self._recv is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for b in (self._recv, self._symm):
            if b is not None:
                b.close()
        self._symm = self._recv = None
