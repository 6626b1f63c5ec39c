"""Expert-parallel layer on real GPUs (NCCL): every rank's output must equal the single-GPU layer
on the same tokens bit for bit, and the single-GPU layer must match the CPU oracle."""
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

from tests.test_ep_gloo import expected, make_case  # noqa: E402

pytestmark = pytest.mark.gpu


def _layer_single(case, dev, sl=slice(None)):
    """The single-rank layer (all experts local) on the tokens `sl` of the case.  A routed row's
    bits do not depend on which other rows are in the step; the shared expert is a dense GEMM whose
    tile / split-K choice follows the number of local tokens, so a rank's reference is the
    single-rank layer on that rank's own tokens."""
    from flaggems_b200.ep import ExpertParallelMoE

    hidden, w1, w2, s1, s2, tw, ti, shared = case
    layer = ExpertParallelMoE(w1.to(dev), w2.to(dev), s1.to(dev), s2.to(dev), w1.shape[0],
                              shared=tuple(t.to(dev) for t in shared))
    return layer(hidden[sl].contiguous().to(dev), tw[sl].contiguous().to(dev), ti[sl].contiguous().to(dev))


def test_single_gpu_layer_matches_oracle():
    case = make_case(seed=5, t=160, h=512, i=256, e=16, topk=4)
    out = _layer_single(case, torch.device("cuda", 0))
    ref = expected(case).float()
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=max(1e-2, 1e-2 * float(ref.abs().max())))
    frac = float(((out.cpu().float() - ref).abs() <= 1e-2 + 1e-2 * ref.abs()).float().mean())
    assert frac >= 0.999, f"only {frac:.5f} of the elements are within rtol 1e-2 / atol 1e-2"


def test_single_gpu_graph_replay_equals_eager():
    """The step recorded into a CUDA graph gives the eager step's bits, also after new inputs have
    been written into the static input tensors."""
    from flaggems_b200 import _cabi
    from flaggems_b200.ep import ExpertParallelMoE

    dev = torch.device("cuda", 0)
    case = make_case(seed=7, t=96, h=512, i=256, e=16, topk=4)
    hidden, w1, w2, s1, s2, tw, ti, shared = case
    layer = ExpertParallelMoE(w1.to(dev), w2.to(dev), s1.to(dev), s2.to(dev), w1.shape[0],
                              shared=tuple(t.to(dev) for t in shared))
    h, w, i = hidden.to(dev), tw.to(dev), ti.to(dev)
    eager = layer(h, w, i).clone()
    layer.capture(h, w, i)
    assert layer.kernels_per_replay > 0
    assert torch.equal(layer.replay(), eager)
    assert torch.equal(layer.replay(), eager)
    case2 = make_case(seed=8, t=96, h=512, i=256, e=16, topk=4)
    h.copy_(case2[0].to(dev))
    w.copy_(case2[5].to(dev))
    i.copy_(case2[6].to(dev))
    replayed = layer.replay().clone()
    assert torch.equal(replayed, layer(h, w, i))
    assert _cabi.device_status() == 0


def _worker(rank, world, port, q):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a short timeout: ranks whose collectives do not match give up within a minute
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    layers = []
    try:
        from flaggems_b200 import _cabi
        from flaggems_b200.ep import ExpertParallelMoE

        case = make_case(seed=5, t=160, h=512, i=256, e=16, topk=4)
        hidden, w1, w2, s1, s2, tw, ti, shared = case
        e, t = w1.shape[0], hidden.shape[0]
        el, tl = e // world, t // world
        lo = rank * el
        sl = slice(rank * tl, (rank + 1) * tl)
        single = _layer_single(case, dev, sl)
        equal, repeat, graph_ok, err = True, True, True, 0.0
        n_slots = tl * ti.shape[1]
        h, w, i = hidden[sl].to(dev), tw[sl].to(dev), ti[sl].to(dev)
        for transport in ("a2a", "p2p_combine", "p2p"):
            layer = ExpertParallelMoE(w1[lo:lo + el].to(dev), w2[lo:lo + el].to(dev), s1[lo:lo + el].to(dev),
                                      s2[lo:lo + el].to(dev), e, rank, world,
                                      shared=tuple(x.to(dev) for x in shared), transport=transport,
                                      max_slots_per_rank=n_slots + 8)
            layers.append(layer)
            outs = [layer(h, w, i) for _ in range(3)]
            equal = equal and bool(torch.equal(outs[0], single))
            repeat = repeat and bool(torch.equal(outs[0], outs[1])) and bool(torch.equal(outs[0], outs[2]))
            err = max(err, float((outs[0].float() - single.float()).abs().max()))
            if transport == "p2p":
                # the recorded step (kernels, all-gather and barrier in one CUDA graph) gives the same bits
                layer.capture(h, w, i)
                for _ in range(3):
                    graph_ok = graph_ok and bool(torch.equal(layer.replay(), single))
            torch.cuda.synchronize()
            dist.barrier()
        q.put((rank, equal, repeat, graph_ok, err, _cabi.device_status()))
    finally:
        for layer in layers:
            layer.close()
        dist.destroy_process_group()


@pytest.mark.timeout(400)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_equals_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = sorted(q.get(timeout=240) for _ in range(world))
        for p in procs:
            p.join(90)
            assert p.exitcode == 0, "a rank did not exit cleanly after close() + destroy_process_group()"
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    for rank, equal, repeat, graph_ok, err, status in res:
        assert status == 0
        assert repeat, f"rank {rank}: two runs differ"
        assert equal, f"rank {rank}: differs from the single-GPU layer, max abs err {err}"
        assert graph_ok, f"rank {rank}: graph replay differs from the single-GPU layer"


def _emulated_ranks(case, world, dev, corrupt=None):
    """The device-driven ("p2p") step of `world` ranks run one after the other on ONE GPU: the
    "peer" receive and combine buffers are ordinary tensors of this device, so every kernel of the
    exchange (region dispatch from the quantisation kernel, region-aware align, peer scatter from
    GEMM2, slot-order sum) runs exactly as it does across GPUs; only NCCL's part (moving the count
    rows, ordering the ranks) is done by this loop.  No kernel here waits on another."""
    import ctypes

    from flaggems_b200.ep import CudaMoEOps

    hidden, w1, w2, s1, s2, tw, ti, shared = case
    e, t, topk = w1.shape[0], hidden.shape[0], ti.shape[1]
    el, tl = e // world, t // world
    region = tl * topk
    ops = [CudaMoEOps(w1[r * el:(r + 1) * el].to(dev), w2[r * el:(r + 1) * el].to(dev),
                      s1[r * el:(r + 1) * el].to(dev), s2[r * el:(r + 1) * el].to(dev),
                      tuple(x.to(dev) for x in shared)) for r in range(world)]
    row_bytes = ops[0].row_bytes
    recv = [torch.full((world * region, row_bytes), 0xAB, dtype=torch.uint8, device=dev) for _ in range(world)]
    comb = [torch.full((region, hidden.shape[1]), float("nan"), dtype=hidden.dtype, device=dev) for _ in range(world)]
    recv_ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in recv])
    comb_ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in comb])
    counts = torch.zeros(world, world, dtype=torch.int32, device=dev)
    shards = []
    for r in range(world):
        sl = slice(r * tl, (r + 1) * tl)
        h, w, i = hidden[sl].to(dev), tw[sl].to(dev).contiguous(), ti[sl].to(dev).contiguous()
        shards.append((h, w, i))
        order, c = ops[r].route(i, world)
        counts[r] = c
        send_counts = c.contiguous()
        if corrupt is not None:
            send_counts = corrupt(r, send_counts)
        ops[r].pack_to_peers(h, i, w, order, send_counts, world, r, recv_ptrs, region)
    for r in range(world):
        ops[r].experts_from_buffer(recv[r].data_ptr(), world, region, counts.reshape(-1), r, hidden.dtype, dev,
                                   comb_ptrs, region)
    outs = []
    for r in range(world):
        h = shards[r][0]
        outs.append(ops[r].combine_slots(comb[r].data_ptr(), tl, topk, hidden.dtype, dev, ops[r].shared_expert(h)))
    torch.cuda.synchronize()
    return torch.cat(outs)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_equal_single_gpu(world):
    from flaggems_b200 import _cabi

    dev = torch.device("cuda", 0)
    case = make_case(seed=5, t=160, h=512, i=256, e=16, topk=4)
    tl = 160 // world
    single = torch.cat([_layer_single(case, dev, slice(r * tl, (r + 1) * tl)) for r in range(world)])
    out = _emulated_ranks(case, world, dev)
    assert _cabi.device_status() == 0
    assert torch.equal(out, single)
    # and the routed rows alone do not depend on the sharding at all
    whole = _layer_single(case, dev)
    torch.testing.assert_close(out.float(), whole.float(), rtol=0, atol=2.0 ** -6)


def test_rows_outside_their_region_are_dropped_and_reported():
    """A rank whose device-side counts promise fewer rows than it packs (a wrong count row) must not
    store the surplus anywhere: the kernel drops those rows and sets status code 2."""
    from flaggems_b200 import _cabi

    dev = torch.device("cuda", 0)
    case = make_case(seed=6, t=64, h=256, i=128, e=8, topk=2)
    assert _cabi.device_status() == 0

    def halve(rank, send_counts):
        return send_counts // 2 if rank == 1 else send_counts

    _emulated_ranks(case, 2, dev, corrupt=halve)
    with pytest.raises(_cabi.FlagGemsB200Error, match="code 2"):
        _cabi.device_status()
    assert _cabi.device_status() == 0  # read-and-clear; the context is still usable
    out = _emulated_ranks(case, 2, dev)
    assert torch.equal(out, torch.cat([_layer_single(case, dev, slice(0, 32)), _layer_single(case, dev, slice(32, 64))]))


def test_combine_rows_outside_the_home_buffer_are_dropped_and_reported():
    """GEMM2's peer scatter checks the (slot, home rank) trailer of every row against the number of
    peers and the rows a combine buffer holds."""
    import ctypes

    from flaggems_b200 import _cabi
    from flaggems_b200.ep import CudaMoEOps

    dev = torch.device("cuda", 0)
    hidden, w1, w2, s1, s2, tw, ti, shared = make_case(seed=9, t=32, h=256, i=128, e=4, topk=2, with_shared=False)
    ops = CudaMoEOps(w1.to(dev), w2.to(dev), s1.to(dev), s2.to(dev))
    packed, _, _ = ops.plan_and_pack(hidden.to(dev), ti.to(dev), tw.to(dev), 1, 0)
    n = packed.shape[0]
    small = torch.zeros(n // 2, hidden.shape[1], dtype=hidden.dtype, device=dev)  # holds half of the slots
    guard = small.clone()
    ptrs = (ctypes.c_void_p * 1)(small.data_ptr())
    assert _cabi.device_status() == 0
    ops.experts_packed(packed, hidden.dtype, ptrs, n // 2)
    with pytest.raises(_cabi.FlagGemsB200Error, match="code 2"):
        _cabi.device_status()
    assert bool((small != guard).any())  # rows inside the buffer were written


def test_bounded_wait_runs_out_and_reports():
    """A wait on a barrier that nothing completes gives up after its limit, the kernel returns, the
    status word names the site and later launches work."""
    from flaggems_b200 import _cabi

    assert _cabi.device_status() == 0
    _cabi.check(_cabi.lib().fg_selftest_bounded_wait(1_000_000, 77, _cabi.stream_ptr(torch.device("cuda", 0))))
    with pytest.raises(_cabi.FlagGemsB200Error) as info:
        _cabi.device_status()
    assert "code 1" in str(info.value) and "site 77" in str(info.value)
    assert _cabi.device_status() == 0
    x = torch.randn(4, 256, device="cuda").bfloat16()
    import flag_gems

    q, s = flag_gems.per_token_group_quant_fp8(x, 128)
    assert q.shape == x.shape and s.shape == (4, 2)


def test_dispatch_staged_equals_per_slot_quantisation():
    """The two forms of the dispatch kernel entry put the same bytes into the receive buffers: quantising
    every token once into staging rows and copying them out, or quantising per route slot while sending."""
    import ctypes

    from flaggems_b200 import _cabi
    from flaggems_b200.ep import CudaMoEOps

    dev = torch.device("cuda", 0)
    hidden, w1, w2, s1, s2, tw, ti, shared = make_case(seed=9, t=96, h=512, i=256, e=16, topk=4)
    world, rank = 4, 1
    ops = CudaMoEOps(w1[:4].to(dev), w2[:4].to(dev), s1[:4].to(dev), s2[:4].to(dev), None)
    h, w, i = hidden.to(dev), tw.to(dev).contiguous(), ti.to(dev).contiguous()
    t, topk = i.shape
    region = t * topk
    order, counts = ops.route(i, world)
    counts = counts.contiguous()
    bufs = []
    for staged in (True, False):
        recv = [torch.full((world * region, ops.row_bytes), 0xAB, dtype=torch.uint8, device=dev) for _ in range(world)]
        ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in recv])
        if staged:
            ops.pack_to_peers(h, i, w, order, counts, world, rank, ptrs, region)
        else:
            _cabi.check(_cabi.lib().fg_ep_pack_rows_fp8_peer(
                _cabi.ptr(h), _cabi.DTYPE_CODE[h.dtype], t, ops.hidden, h.stride(0), _cabi.ptr(i),
                1 if i.dtype == torch.int64 else 0, _cabi.ptr(w), _cabi.DTYPE_CODE[w.dtype], topk, ops.num_local_experts,
                rank, _cabi.ptr(order), None, ops.row_bytes, None, _cabi.ptr(counts), ptrs, world, region,
                _cabi.stream_ptr(dev)))
        torch.cuda.synchronize()
        bufs.append([b.cpu() for b in recv])
    assert _cabi.device_status() == 0
    c = counts.cpu().tolist()
    assert sum(c) == region
    for d in range(world):
        lo = rank * region
        assert torch.equal(bufs[0][d][lo:lo + c[d]], bufs[1][d][lo:lo + c[d]])
        # nothing outside this rank's region, or beyond its count, was touched
        assert bool((bufs[0][d][:lo] == 0xAB).all()) and bool((bufs[0][d][lo + c[d]:] == 0xAB).all())
