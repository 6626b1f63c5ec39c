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


def _layer_single(case, dev):
    from flaggems_b200.ep import ExpertParallelMoE

    hidden, w1, w2, s1, s2, tw, ti, shared = case
    layer = ExpertParallelMoE(w1.to(dev), w2.to(dev), s1.to(dev), s2.to(dev), w1.shape[0],
                              shared=tuple(t.to(dev) for t in shared))
    return layer(hidden.to(dev), tw.to(dev), ti.to(dev))


def test_single_gpu_layer_matches_oracle():
    case = make_case(seed=5, t=160, h=512, i=256, e=16, topk=4)
    out = _layer_single(case, torch.device("cuda", 0))
    ref = expected(case).float()
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=max(1e-2, 1e-2 * float(ref.abs().max())))


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
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flaggems_b200 import _cabi
        from flaggems_b200.ep import ExpertParallelMoE

        case = make_case(seed=5, t=160, h=512, i=256, e=16, topk=4)
        hidden, w1, w2, s1, s2, tw, ti, shared = case
        e, t = w1.shape[0], hidden.shape[0]
        el, tl = e // world, t // world
        lo = rank * el
        sl = slice(rank * tl, (rank + 1) * tl)
        single = _layer_single(case, dev)[sl]
        equal, repeat, err = True, True, 0.0
        # all-to-all both ways; combine fused into GEMM2 over peer memory; dispatch fused as well
        # (3 steps each, so both halves of the double buffers are used)
        n_slots = tl * ti.shape[1]
        for p2p_rows, recv_rows in ((0, 0), (n_slots, 0), (n_slots, world * n_slots)):
            layer = ExpertParallelMoE(w1[lo:lo + el].to(dev), w2[lo:lo + el].to(dev), s1[lo:lo + el].to(dev),
                                      s2[lo:lo + el].to(dev), e, rank, world,
                                      shared=tuple(x.to(dev) for x in shared), p2p_combine_rows=p2p_rows,
                                      p2p_dispatch_rows=recv_rows)
            outs = [layer(hidden[sl].to(dev), tw[sl].to(dev), ti[sl].to(dev)) for _ in range(3)]
            equal = equal and bool(torch.equal(outs[0], single))
            repeat = repeat and bool(torch.equal(outs[0], outs[1])) and bool(torch.equal(outs[0], outs[2]))
            err = max(err, float((outs[0].float() - single.float()).abs().max()))
            torch.cuda.synchronize()
            dist.barrier()
        q.put((rank, equal, repeat, err, _cabi.device_status()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
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
    res = sorted(q.get(timeout=500) for _ in range(world))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, equal, repeat, err, status in res:
        assert status == 0
        assert repeat, f"rank {rank}: two runs differ"
        assert equal, f"rank {rank}: differs from the single-GPU layer, max abs err {err}"
