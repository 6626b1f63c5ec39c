"""GPU parity: moe_align_block_size (exact), silu_and_mul, moe_sum vs the CPU oracle."""
import os

import pytest
import torch

import flag_gems
import oracle
from tests._isolated import check_isolated
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu


def _check_align(ids, bs, e, expert_map=None, pad=False):
    so, eo, no = flag_gems.moe_align_block_size(ids.cuda(), bs, e,
                                                None if expert_map is None else expert_map.cuda(), pad)
    sr, er, nr = oracle.moe_align_block_size(ids, bs, e, expert_map, pad)
    assert so.dtype == eo.dtype == no.dtype == torch.int32
    assert torch.equal(no.cpu(), nr), (no, nr)
    assert torch.equal(eo.cpu(), er)
    assert torch.equal(so.cpu(), sr)


@pytest.mark.parametrize("e", [10, 128, 250, 512])
@pytest.mark.parametrize("bs", [16, 32, 64])
@pytest.mark.parametrize("shape", [(1024, 10), (6152, 10), (11575, 10), (16384, 10)])
def test_moe_align_reference_grid(e, bs, shape):
    """Grid of tests/test_moe_align_block_size.py:216 (E x block x (tokens, topk))."""
    g = torch.Generator().manual_seed(e * 1000 + bs + shape[0])
    ids = torch.randint(0, e, shape, generator=g, dtype=torch.int32)
    _check_align(ids, bs, e)


def test_moe_align_known_answers_and_golden(golden_dir):
    _check_align(torch.tensor([[1, 3]], dtype=torch.int32), 8, 8)
    _check_align(torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]], dtype=torch.int32), 8, 8)
    for c in torch.load(os.path.join(golden_dir, "moe_align.pt")):
        so, eo, no = flag_gems.moe_align_block_size(c["topk_ids"].cuda(), c["block_size"], c["num_experts"])
        n = c["expert_ids"].numel()
        assert torch.equal(so.cpu(), c["sorted_ids"])
        assert torch.equal(eo.cpu()[:n], c["expert_ids"])
        assert torch.equal(no.cpu(), c["num_post_pad"])


def test_moe_align_baseline_configs():
    """configs[3]: T=4096, top-2, 8 experts, block 64; configs[4]: T=8192, top-8, 256 experts."""
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(4096, 8, generator=g)
    ids = torch.topk(torch.softmax(logits, -1), 2).indices
    _check_align(ids, 64, 8)                      # int64 ids, as torch.topk returns them
    _check_align(ids.int(), 64, 8)
    _check_align(ids, 128, 8)
    p = torch.arange(1, 257).float() ** -1.1
    p = p[torch.randperm(256, generator=g)]
    u = torch.rand(8192, 256, generator=g).clamp_min(1e-9)
    score = torch.log(p / p.sum()) - torch.log(-torch.log(u))
    ids = torch.topk(score, 8).indices
    _check_align(ids, 64, 256)
    _check_align(ids, 128, 256)


def test_moe_align_edges():
    _check_align(torch.zeros(0, 2, dtype=torch.int32), 16, 8)
    _check_align(torch.full((777, 3), 5, dtype=torch.int32), 64, 16)  # one hot expert
    _check_align(torch.arange(1024, dtype=torch.int32).reshape(1024, 1), 1, 1024)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 64, (32768, 8), generator=g)
    _check_align(ids, 128, 64)                     # 262144 slots: the full 8-CTA cluster
    _check_align(ids, 64, 64, pad=True)
    emap = torch.full((64,), -1, dtype=torch.int32)
    emap[16:32] = torch.arange(16, dtype=torch.int32)
    _check_align(ids[:1000], 32, 64, expert_map=emap)


def test_moe_align_out_param_and_vllm_op():
    g = torch.Generator().manual_seed(8)
    ids = torch.randint(0, 60, (513, 6), generator=g, dtype=torch.int32)
    sr, er, nr = oracle.moe_align_block_size(ids, 32, 60)
    so = torch.empty_like(sr, device="cuda")
    eo = torch.empty_like(er, device="cuda")
    no = torch.empty(1, dtype=torch.int32, device="cuda")
    flag_gems.moe_align_block_size_triton(ids.cuda(), 60, 32, so, eo, no)
    assert torch.equal(so.cpu(), sr) and torch.equal(eo.cpu(), er) and torch.equal(no.cpu(), nr)


def test_moe_align_short_buffers_for_decode_batches():
    """Fewer route slots than experts: at most numel experts are non-empty, so buffers of
    numel * block_size entries (what a caller sizes for decode batches) are enough."""
    ids = torch.tensor([[3, 17], [40, 3]], dtype=torch.int32)
    numel, bs, e = 4, 16, 64
    so = torch.full((numel * bs,), -7, dtype=torch.int32, device="cuda")
    eo = torch.full((numel,), -7, dtype=torch.int32, device="cuda")
    no = torch.empty(1, dtype=torch.int32, device="cuda")
    flag_gems.moe_align_block_size_triton(ids.cuda(), e, bs, so, eo, no)
    sr, er, nr = oracle.moe_align_block_size(ids, bs, e)
    assert int(no) == int(nr) == 48
    assert torch.equal(so.cpu()[:48], sr[:48]) and torch.equal(eo.cpu()[:3], er[:3])
    assert bool((so.cpu()[48:] == numel).all()) and int(eo.cpu()[3]) == -1
    with pytest.raises(AssertionError):
        flag_gems.moe_align_block_size_triton(ids.cuda(), e, bs, so[:40], eo, no)


def test_vllm_moe_ops_defined_by_patch_empty_vllm():
    """torch.ops._moe_C.* as patch_empty_vllm() defines them, in a process of their own."""
    check_isolated('''
import torch, flag_gems, oracle
flag_gems.patch_empty_vllm()
g = torch.Generator().manual_seed(8)
ids = torch.randint(0, 60, (513, 6), generator=g, dtype=torch.int32)
sr, er, nr = oracle.moe_align_block_size(ids, 32, 60)
so = torch.full_like(sr, -7, device="cuda"); eo = torch.full_like(er, -7, device="cuda")
no = torch.empty(1, dtype=torch.int32, device="cuda")
torch.ops._moe_C.moe_align_block_size(ids.cuda(), 60, 32, so, eo, no)
assert torch.equal(so.cpu(), sr) and torch.equal(eo.cpu(), er) and torch.equal(no.cpu(), nr)
x = torch.randn(33, 2, 4096).bfloat16()
out = torch.empty(33, 4096, dtype=torch.bfloat16, device="cuda")
torch.ops._moe_C.moe_sum(x.cuda(), out)
assert torch.equal(out.cpu(), oracle.moe_sum(x))
gate = torch.randn(64, 32)
w = torch.empty(64, 4, device="cuda"); i = torch.empty(64, 4, dtype=torch.int32, device="cuda")
src = torch.empty(64, 4, dtype=torch.int32, device="cuda")
torch.ops._moe_C.topk_softmax(w, i, src, gate.cuda(), True)
rw, ri, rs = oracle.topk_softmax(gate, 4, True, torch.int64)
assert torch.equal(i.cpu().long(), ri) and torch.allclose(w.cpu(), rw, atol=1e-5)
v, gi = torch.ops._moe_C.grouped_topk(gate.cuda(), 4, 2, 4, True, 1.0, torch.zeros(32, device="cuda"), 0)
rv, rgi = oracle.grouped_topk(gate, 4, 2, 4, True, 1.0, torch.zeros(32), 0)
assert torch.equal(gi.cpu(), rgi) and torch.allclose(v.cpu(), rv, atol=1e-5)
''')


def test_moe_align_deterministic():
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 256, (8192, 8), generator=g).cuda()
    a = flag_gems.moe_align_block_size(ids, 64, 256)
    b = flag_gems.moe_align_block_size(ids, 64, 256)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_silu_and_mul(dt):
    torch.manual_seed(10)
    z = (torch.randn(257, 2 * 1408) * 3).to(dt)
    x, y = z[:, :1408], z[:, 1408:]
    ref = oracle.silu_and_mul(x, y)
    zc = z.cuda()
    out = flag_gems.silu_and_mul(zc[:, :1408], zc[:, 1408:])
    tol = dict(rtol=1e-2, atol=1e-2) if dt != torch.float32 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol)
    o2 = torch.empty(257, 1408, dtype=dt, device="cuda")
    flag_gems.silu_and_mul_out(zc[:, :1408], zc[:, 1408:], o2)
    assert torch.equal(o2, out)


@pytest.mark.parametrize("shape", [(1, 1, 128), (33, 2, 4096), (64, 8, 7168), (7, 6, 1024)])
def test_moe_sum(shape):
    torch.manual_seed(11)
    x = torch.randn(*shape).bfloat16()
    out = torch.empty(shape[0], shape[2], dtype=torch.bfloat16, device="cuda")
    flag_gems.moe_sum(x.cuda(), out)
    assert torch.equal(out.cpu(), oracle.moe_sum(x))


def test_no_device_errors_recorded():
    assert _cabi.device_status() == 0
