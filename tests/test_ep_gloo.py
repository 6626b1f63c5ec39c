"""Expert-parallel layer: host logic (routing order, counts, all-to-all, inverse permutation,
combine) on 2 CPU ranks over gloo.  The device work is swapped for CPU-oracle stand-ins here;
the result must equal the single-rank oracle of the whole layer bit for bit."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FP8 = torch.float8_e4m3fn


class OracleOps:
    """Test double for CudaMoEOps: same methods and the same packed row format, computed by the
    CPU oracle."""

    def __init__(self, w1, w2, s1, s2, shared=None):
        from flaggems_b200.ep import packed_row_bytes

        self.w1, self.w2, self.s1, self.s2, self.shared = w1, w2, s1, s2, shared
        self.hidden = w1.shape[2]
        self.e_loc = w1.shape[0]
        self.row_bytes = packed_row_bytes(self.hidden)

    def plan_and_pack(self, hidden, topk_ids, topk_w, world, rank):
        import oracle

        t, topk = topk_ids.shape
        numel = t * topk
        flat = topk_ids.reshape(-1)
        dest = flat // self.e_loc
        order = torch.sort(dest, stable=True).indices
        counts = torch.bincount(dest, minlength=world).to(torch.int32)
        q, s = oracle.per_token_group_quant_fp8(hidden[order // topk], 128)
        h = self.hidden
        packed = torch.zeros(numel, self.row_bytes, dtype=torch.uint8)
        packed[:, :h] = q.view(torch.uint8)
        packed[:, h:h + 4 * (h // 128)] = s.contiguous().view(torch.uint8).reshape(numel, -1)
        off = h + 4 * (h // 128)
        packed[:, off:off + 4] = (flat[order] % self.e_loc).to(torch.int32).view(torch.uint8).reshape(numel, 4)
        packed[:, off + 4:off + 8] = topk_w.reshape(-1).float()[order].view(torch.uint8).reshape(numel, 4)
        packed[:, off + 8:off + 12] = order.to(torch.int32).view(torch.uint8).reshape(numel, 4)
        packed[:, off + 12:off + 16] = torch.full((numel,), rank, dtype=torch.int32).view(torch.uint8).reshape(numel, 4)
        inv = torch.empty(numel, dtype=torch.int32)
        inv[order] = torch.arange(numel, dtype=torch.int32)
        return packed, counts, inv

    def _unpack(self, packed):
        h = self.hidden
        off = h + 4 * (h // 128)
        xq = packed[:, :h].contiguous().view(FP8)
        xs = packed[:, h:off].contiguous().view(torch.float32)
        le = packed[:, off:off + 4].contiguous().view(torch.int32).reshape(-1)
        wt = packed[:, off + 4:off + 8].contiguous().view(torch.float32).reshape(-1)
        return xq, xs, le, wt

    def experts_packed(self, packed, dtype):
        return self._experts(*self._unpack(packed), dtype)

    def local_routed(self, hidden, topk_ids, topk_w):
        import oracle

        topk = topk_ids.shape[1]
        xq, xs = oracle.per_token_group_quant_fp8(hidden[torch.arange(topk_ids.numel()) // topk], 128)
        return self._experts(xq, xs, topk_ids.reshape(-1).int(), topk_w.reshape(-1).float(), hidden.dtype)

    def _experts(self, xq, xs, le, wt, dtype):
        import oracle
        from oracle.moe import _silu_mul_f32

        y = torch.zeros(xq.shape[0], self.w2.shape[1], dtype=dtype)
        for e in range(self.w1.shape[0]):
            rows = torch.nonzero(le == e).flatten()
            if rows.numel() == 0:
                continue
            z = oracle.block_scaled_mm(xq[rows], self.w1[e], xs[rows], self.s1[e], out_dtype=torch.float32)
            act = _silu_mul_f32(z, True, dtype)
            aq, a_s = oracle.per_token_group_quant_fp8(act, 128)
            r = oracle.block_scaled_mm(aq, self.w2[e], a_s, self.s2[e], out_dtype=torch.float32)
            y[rows] = (r * wt[rows].unsqueeze(1)).to(dtype)
        return y

    def shared_expert(self, hidden):
        import oracle

        return None if self.shared is None else oracle.dense_block_fp8_mlp(hidden, *self.shared)

    def combine(self, rows, inv, tokens, topk, addend):
        idx = torch.arange(tokens * topk) if inv is None else inv.long()
        acc = torch.zeros(tokens, rows.shape[1])
        for k in range(topk):
            acc += rows[idx.view(tokens, topk)[:, k]].float()
        if addend is not None:
            acc += addend.float()
        return acc.to(rows.dtype)


def make_case(seed=0, t=48, h=256, i=128, e=8, topk=3, with_shared=True):
    import oracle

    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1 = torch.empty(e, 2 * i, h, dtype=FP8)
    w2 = torch.empty(e, h, i, dtype=FP8)
    s1 = torch.empty(e, 2 * i // 128, h // 128)
    s2 = torch.empty(e, h // 128, i // 128)
    for x in range(e):
        w1[x], s1[x] = oracle.quantize_weight_block(torch.randn(2 * i, h, generator=g) * 0.05)
        w2[x], s2[x] = oracle.quantize_weight_block(torch.randn(h, i, generator=g) * 0.05)
    shared = None
    if with_shared:
        a, sa = oracle.quantize_weight_block(torch.randn(2 * i, h, generator=g) * 0.05)
        b, sb = oracle.quantize_weight_block(torch.randn(h, i, generator=g) * 0.05)
        shared = (a, b, sa, sb)
    # skewed router so that ranks receive different amounts
    p = torch.arange(1, e + 1).float() ** -1.1
    score = torch.log(p / p.sum()) - torch.log(-torch.log(torch.rand(t, e, generator=g).clamp_min(1e-9)))
    sc, ti = torch.topk(score, topk)
    tw = torch.softmax(sc, -1).bfloat16()
    return hidden, w1, w2, s1, s2, tw, ti, shared


def expected(case):
    import oracle

    hidden, w1, w2, s1, s2, tw, ti, shared = case
    add = None if shared is None else oracle.dense_block_fp8_mlp(hidden, *shared)
    return oracle.fused_moe_block_fp8(hidden, w1, w2, s1, s2, tw, ti, addend=add)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flaggems_b200.ep import ExpertParallelMoE

        case = make_case()
        hidden, w1, w2, s1, s2, tw, ti, shared = case
        e, t = w1.shape[0], hidden.shape[0]
        el, tl = e // world, t // world
        lo = rank * el
        ops = OracleOps(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], shared)
        layer = ExpertParallelMoE(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], e, rank, world,
                                  ops=ops)
        sl = slice(rank * tl, (rank + 1) * tl)
        out = layer(hidden[sl].contiguous(), tw[sl].contiguous(), ti[sl].contiguous())
        ref = expected(case)[sl]
        send, recv = layer.last_counts
        q.put((rank, bool(torch.equal(out, ref)), float((out.float() - ref.float()).abs().max()), send, recv))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(300)
def test_two_rank_layer_equals_single_rank_oracle():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    res.sort()
    for rank, equal, err, send, recv in res:
        assert equal, f"rank {rank}: max abs err {err}"
        assert sum(send) == 24 * 3
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0
    assert res[0][3][1] == res[1][4][0] and res[1][3][0] == res[0][4][1]


def test_single_rank_layer_with_oracle_ops():
    from flaggems_b200.ep import ExpertParallelMoE

    case = make_case(seed=3, t=20, e=4, topk=2)
    hidden, w1, w2, s1, s2, tw, ti, shared = case
    layer = ExpertParallelMoE(w1, w2, s1, s2, 4, ops=OracleOps(w1, w2, s1, s2, shared))
    assert torch.equal(layer(hidden, tw, ti), expected(case))


# ---- unequal token counts, refusals and host-side failures ---------------------------------------
def _uneven_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flaggems_b200.ep import ExpertParallelMoE

        case = make_case(seed=11)
        hidden, w1, w2, s1, s2, tw, ti, shared = case
        e = w1.shape[0]
        el = e // world
        lo = rank * el
        ops = OracleOps(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], shared)
        layer = ExpertParallelMoE(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], e, rank, world,
                                  ops=ops)
        sl = slice(0, 30) if rank == 0 else slice(30, 48)  # 30 and 18 tokens
        paths = []
        for _ in range(2):
            out = layer(hidden[sl].contiguous(), tw[sl].contiguous(), ti[sl].contiguous())
            paths.append(layer.transport)
        ref = expected(case)[sl]
        q.put((rank, bool(torch.equal(out, ref)), paths))
        layer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_unequal_token_counts_take_the_same_path_on_every_rank():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_uneven_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0, "a rank did not exit cleanly after close()"
    assert res[0][2] == res[1][2], "ranks chose different transports"
    assert all(r[1] for r in res)


def _failing_worker(rank, world, port, q, mode):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from flaggems_b200.ep import ExpertParallelMoE

    case = make_case(seed=12)
    hidden, w1, w2, s1, s2, tw, ti, shared = case
    e = w1.shape[0]
    el = e // world
    lo = rank * el
    ops = OracleOps(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], shared)
    try:
        if mode == "world_mismatch":
            ExpertParallelMoE(w1[:2], w2[:2], s1[:2], s2[:2], e, rank, 4, ops=ops)
            q.put((rank, "no error"))
            return
        layer = ExpertParallelMoE(w1[lo:lo + el], w2[lo:lo + el], s1[lo:lo + el], s2[lo:lo + el], e, rank, world,
                                  ops=ops)
        sl = slice(rank * 24, (rank + 1) * 24)
        if mode == "rank_raises" and rank == 1:
            raise RuntimeError("rank 1 fails before the step")
        if mode == "wrong_counts" and rank == 1:
            # this rank announces counts that do not add up to the rows it sends
            real = layer._exchange_counts

            def lying(send_counts_dev):
                send, recv = real(send_counts_dev)
                send[0] += 3
                return send, recv

            layer._exchange_counts = lying
        layer(hidden[sl].contiguous(), tw[sl].contiguous(), ti[sl].contiguous())
        q.put((rank, "no error"))
    except Exception as exc:  # noqa: BLE001 - the test asserts on what each rank saw
        q.put((rank, type(exc).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


@pytest.mark.timeout(120)
@pytest.mark.parametrize("mode", ["world_mismatch", "rank_raises", "wrong_counts"])
def test_host_side_failures_end_in_exceptions_not_hangs(mode):
    """Failures made on the host (never on a device): a layer built for another world size, a rank
    that raises before the step, a rank whose announced counts are wrong.  Every rank must come
    back with an exception within the process group's (shortened) timeout."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank hung after the failure")
    if mode == "world_mismatch":
        assert res == {0: "ValueError", 1: "ValueError"}
    elif mode == "rank_raises":
        assert res[1] == "RuntimeError" and res[0] != "no error"
    else:
        assert res[0] != "no error" or res[1] != "no error"


def test_step_beyond_capacity_is_refused_before_any_collective():
    """With a peer-memory transport a step with more route slots than max_slots_per_rank raises at
    once; no process group exists here, so reaching any collective would fail differently."""
    from flaggems_b200.ep import ExpertParallelMoE

    case = make_case(seed=3, t=20, e=4, topk=2)
    hidden, w1, w2, s1, s2, tw, ti, shared = case
    layer = ExpertParallelMoE(w1, w2, s1, s2, 4, ops=OracleOps(w1, w2, s1, s2, shared))
    layer.world, layer.transport, layer.max_slots = 2, "p2p", 39
    with pytest.raises(ValueError, match="exceed max_slots_per_rank"):
        layer(hidden, tw, ti)
    layer.max_slots = 40
    with pytest.raises(TypeError, match="bf16 or fp16"):
        layer(hidden.float(), tw, ti)
