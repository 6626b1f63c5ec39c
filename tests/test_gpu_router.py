"""Router kernels (topk_softmax, grouped_topk) on the GPU against the CPU oracle, on the reference's
own test grids (tests/test_topk_softmax.py:44-62, tests/test_grouped_topk.py:28-48,128-137), and
against vLLM's CUDA ops (the reference tests' criterion) when those load."""
import pytest
import torch

import flag_gems
import oracle
from flaggems_b200 import _cabi
from tests._isolated import check_isolated, require_vllm_ops

pytestmark = pytest.mark.gpu


def _check_selection(scores_cpu, got_idx, ref_idx, tie_eps=0.0):
    """Same experts in the same order, except where the oracle's own scores of the two candidates
    are within tie_eps (an fp32 rounding of exp or of the sigmoid may order such a pair either way)."""
    got_idx, ref_idx = got_idx.cpu().long(), ref_idx.cpu().long()
    bad = got_idx != ref_idx
    if bool(bad.any()):
        r, c = torch.nonzero(bad, as_tuple=True)
        a = scores_cpu[r, got_idx[r, c]]
        b = scores_cpu[r, ref_idx[r, c]]
        assert bool(((a - b).abs() <= tie_eps * b.abs().clamp(min=1e-30)).all()), "selected experts differ"
    # never the same expert twice in a row
    srt = got_idx.sort(dim=1)[0]
    assert bool((srt[:, 1:] != srt[:, :-1]).all()) or got_idx.shape[1] == 1


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64, torch.uint32])
@pytest.mark.parametrize("t,e,k", [(1, 4, 2), (4, 8, 2), (8, 16, 4), (32, 64, 8), (128, 128, 16), (500, 255, 30),
                                   (512, 256, 32), (1024, 512, 32), (77, 1000, 7)])
@pytest.mark.parametrize("input_dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("renormalize", [False, True])
def test_topk_softmax(t, e, k, input_dtype, index_dtype, renormalize):
    torch.manual_seed(42)
    gating = torch.randn(t, e, dtype=torch.float32).to(input_dtype)
    w = torch.empty(t, k, dtype=torch.float32, device="cuda")
    idx = torch.empty(t, k, dtype=index_dtype, device="cuda")
    src = torch.empty(t, k, dtype=torch.int32, device="cuda")
    counts = torch.zeros(e, dtype=torch.int32, device="cuda")
    flag_gems.topk_softmax(w, idx, src, gating.cuda(), renormalize, expert_counts=counts)
    rw, ri, rs = oracle.topk_softmax(gating, k, renormalize, torch.int64)
    probs = torch.softmax(gating.float(), -1)
    _check_selection(probs, idx.cpu().to(torch.int64), ri, tie_eps=1e-6)
    torch.testing.assert_close(w.cpu(), rw, atol=1e-5, rtol=0)
    assert torch.equal(src.cpu(), rs)
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.cpu().to(torch.int64).reshape(-1), minlength=e))
    if renormalize:
        torch.testing.assert_close(w.sum(-1).cpu(), torch.ones(t), atol=1e-5, rtol=0)


def test_topk_softmax_ties_and_errors():
    x = torch.zeros(2, 8, device="cuda")
    x[1, 5] = 1.0
    w = torch.empty(2, 3, device="cuda")
    idx = torch.empty(2, 3, dtype=torch.int32, device="cuda")
    src = torch.empty(2, 3, dtype=torch.int32, device="cuda")
    flag_gems.topk_softmax(w, idx, src, x)
    assert idx.cpu().tolist() == [[0, 1, 2], [5, 0, 1]]
    with pytest.raises(TypeError):
        flag_gems.topk_softmax(w, idx.to(torch.int16), src, x)
    with pytest.raises(AssertionError):
        flag_gems.topk_softmax(torch.empty(2, 33, device="cuda"), torch.empty(2, 33, dtype=torch.int32, device="cuda"),
                               torch.empty(2, 33, dtype=torch.int32, device="cuda"), torch.zeros(2, 64, device="cuda"))


def test_topk_softmax_equals_vllm_op():
    """The reference's own criterion (tests/test_topk_softmax.py): vLLM's CUDA op, run in a fresh
    process that imports vLLM's extension and registers nothing of this package's."""
    require_vllm_ops("_moe_C.topk_softmax")
    check_isolated('''
import torch
from vllm import _custom_ops as ops
import flag_gems
torch.manual_seed(42)
for (t, e, k) in [(32, 64, 8), (512, 256, 32), (500, 255, 30)]:
    for renorm in (False, True):
        g = torch.randn(t, e, device="cuda")
        vw = torch.empty(t, k, device="cuda")
        vi = torch.empty(t, k, dtype=torch.int32, device="cuda")
        vs = torch.empty(t, k, dtype=torch.int32, device="cuda")
        ops.topk_softmax(vw, vi, vs, g, renorm)
        w = torch.empty_like(vw); idx = torch.empty_like(vi); src = torch.empty_like(vs)
        flag_gems.topk_softmax(w, idx, src, g, renorm)
        assert torch.allclose(w, vw, atol=1e-5)
        assert torch.equal(idx, vi) and torch.equal(src, vs)
''')


GT_GRID = [(n, e, g, k, k) for n in (1, 3, 8) for e in (8, 16) for g in (2, 4) for k in (1, 2)]
GT_GRID += [(32, 64, 8, 8, 2), (64, 64, 8, 8, 2), (200, 256, 8, 8, 4), (33, 384, 32, 6, 3), (5, 1024, 8, 32, 4)]


def _tolerance(dtype, scoring_func, renormalize):
    # tests/test_grouped_topk.py:58-70
    if dtype == torch.bfloat16:
        return 5e-3, 1e-3
    if dtype == torch.float16:
        return (1e-3, 1e-4) if scoring_func == 1 else (5e-3, 1e-3)
    return (5e-4, 1e-4) if renormalize else (1e-5, 1e-5)


@pytest.mark.parametrize("t,e,n_group,topk,topk_group", GT_GRID)
@pytest.mark.parametrize("renormalize", [True, False])
@pytest.mark.parametrize("scoring_func", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_grouped_topk(t, e, n_group, topk, topk_group, renormalize, scoring_func, dtype):
    if e % n_group != 0 or topk > topk_group * (e // n_group):
        pytest.skip("not a valid routing configuration")
    torch.manual_seed(45)
    scores = torch.randn(t, e).to(dtype)
    bias = torch.randn(e).to(dtype)
    counts = torch.zeros(e, dtype=torch.int32, device="cuda")
    v, i = flag_gems.grouped_topk(scores.cuda(), n_group, topk_group, topk, renormalize, 2.5, bias.cuda(),
                                  scoring_func, expert_counts=counts)
    rv, ri = oracle.grouped_topk(scores, n_group, topk_group, topk, renormalize, 2.5, bias, scoring_func)
    assert v.dtype == torch.float32 and i.dtype == torch.int32 and v.shape == (t, topk)
    if scoring_func == 1:
        # expf on the GPU and the host's vector exp are a rounding apart, so a sigmoid may land on the
        # other side of a rounding boundary of `dtype`: candidates within one unit of `dtype` may swap
        eps = {torch.float32: 1e-6, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]
        sel = (torch.sigmoid(scores.float()).to(dtype) + bias[None, :]).float()
        _check_selection(sel, i, ri, tie_eps=eps)
        same = (i.cpu() == ri).all(dim=1)
    else:
        assert torch.equal(i.cpu(), ri)
        same = torch.ones(t, dtype=torch.bool)
    atol, rtol = _tolerance(dtype, scoring_func, renormalize)
    torch.testing.assert_close(v.cpu()[same], rv[same], atol=atol, rtol=rtol)
    assert torch.equal(counts.cpu().long(), torch.bincount(i.cpu().long().reshape(-1), minlength=e))


def test_grouped_topk_edges_and_errors():
    bias = torch.zeros(8, device="cuda")
    scores = torch.full((2, 8), float("-inf"), device="cuda")
    v, i = flag_gems.grouped_topk(scores, 2, 1, 2, True, 1.0, bias)
    assert torch.equal(v.cpu(), torch.full((2, 2), 0.5)) and i.cpu().tolist() == [[0, 1], [0, 1]]
    v, i = flag_gems.grouped_topk(torch.ones(1, 8, device="cuda"), 2, 1, 2, False, 1.0, bias)
    assert i.cpu().tolist() == [[0, 1]]
    s = torch.tensor([[4.0, 1.0, 0.0, 0.0, 3.0, 3.0, 0.0, 0.0]], device="cuda")
    v, i = flag_gems.grouped_topk(s, 2, 1, 1, False, 1.0, bias)
    assert i.cpu().tolist() == [[4]] and v.cpu().tolist() == [[3.0]]
    # a strided view of a wider tensor
    wide = torch.randn(16, 128, device="cuda")
    v1, i1 = flag_gems.grouped_topk(wide[:, :64], 8, 2, 4, True, 1.0, torch.zeros(64, device="cuda"))
    v2, i2 = flag_gems.grouped_topk(wide[:, :64].contiguous(), 8, 2, 4, True, 1.0, torch.zeros(64, device="cuda"))
    assert torch.equal(v1, v2) and torch.equal(i1, i2)
    with pytest.raises(ValueError, match="divisible"):
        flag_gems.grouped_topk(torch.zeros(1, 9, device="cuda"), 2, 1, 1, False, 1.0, torch.zeros(9, device="cuda"))
    with pytest.raises(ValueError, match="n_group"):
        flag_gems.grouped_topk(torch.zeros(1, 64, device="cuda"), 64, 1, 1, False, 1.0, torch.zeros(64, device="cuda"))
    with pytest.raises(ValueError, match="bias length"):
        flag_gems.grouped_topk(torch.zeros(1, 8, device="cuda"), 2, 1, 1, False, 1.0, torch.zeros(4, device="cuda"))
    with pytest.raises(ValueError, match="2D"):
        flag_gems.grouped_topk(torch.zeros(8, device="cuda"), 2, 1, 1, False, 1.0, bias)


def test_grouped_topk_against_vllm_op():
    """vLLM's CUDA grouped_topk in a fresh process.  fp32: same experts up to fp32 near-ties.  bf16:
    the installed vLLM keeps group scores and the sigmoid in fp32 where the reference (followed
    here, and by the oracle) rounds both to bf16 (grouped_topk.py:73-76, :291-294); near-tied groups
    then differ, so only most rows can agree."""
    require_vllm_ops("_moe_C.topk_softmax", "_moe_C.grouped_topk")
    check_isolated('''
import torch
from vllm import _custom_ops as ops
import flag_gems
TOL = {(torch.bfloat16, 0): (5e-3, 1e-3), (torch.bfloat16, 1): (5e-3, 1e-3)}
torch.manual_seed(0)
for dtype in (torch.float32, torch.bfloat16):
    for scoring in (0, 1):
        for renorm in (True, False):
            scores = torch.randn(64, 64, device="cuda").to(dtype)
            b = torch.randn(64, device="cuda").to(dtype)
            rw, ri = ops.grouped_topk(scores.clone(), 8, 2, 8, renorm, 1.0, b, scoring)
            w, i = flag_gems.grouped_topk(scores.clone(), 8, 2, 8, renorm, 1.0, b, scoring)
            same = (i.long() == ri.long()).all(dim=1)
            need = 62 if dtype == torch.float32 else 40
            assert int(same.sum()) >= need, (dtype, scoring, renorm, int(same.sum()))
            if dtype == torch.float32:
                atol, rtol = (5e-4, 1e-4) if renorm else (1e-5, 1e-5)
            else:
                atol, rtol = 5e-3, 1e-3
            torch.testing.assert_close(w[same], rw.float()[same], atol=atol, rtol=rtol)
''')


def test_apply_gems_patches_to_vllm_overrides_the_compiled_ops():
    """apply_gems_patches_to_vllm() on top of vLLM's own extension: afterwards the vLLM op names
    run this package's kernels (the launch counter moves) and give the oracle's results."""
    require_vllm_ops("_moe_C.topk_softmax", "_C.cutlass_scaled_mm")
    check_isolated('''
import torch
import vllm._custom_ops
import flag_gems, oracle
from flaggems_b200 import _cabi
flag_gems.apply_gems_patches_to_vllm(verbose=False)
def call(op, *args):
    # the installed vLLM may declare trailing arguments the reference's schemas do not have
    extra = []
    for a in op.default._schema.arguments[len(args):]:
        if a.has_default_value():
            break
        t = str(a.type)
        extra.append(None if t.startswith("Optional") else False if t == "bool" else 0)
    return op(*args, *extra)
n0 = _cabi.launch_count()
x = torch.randn(33, 2, 1024).bfloat16()
out = torch.empty(33, 1024, dtype=torch.bfloat16, device="cuda")
call(torch.ops._moe_C.moe_sum, x.cuda(), out)
assert torch.equal(out.cpu(), oracle.moe_sum(x))
g = torch.Generator().manual_seed(8)
ids = torch.randint(0, 60, (513, 6), generator=g, dtype=torch.int32)
sr, er, nr = oracle.moe_align_block_size(ids, 32, 60)
so = torch.full_like(sr, -7, device="cuda"); eo = torch.full_like(er, -7, device="cuda")
no = torch.empty(1, dtype=torch.int32, device="cuda")
call(torch.ops._moe_C.moe_align_block_size, ids.cuda(), 60, 32, so, eo, no)
assert torch.equal(so.cpu(), sr) and torch.equal(eo.cpu(), er) and torch.equal(no.cpu(), nr)
a = torch.randn(64, 512).bfloat16()
q = torch.empty(64, 512, dtype=torch.float8_e4m3fn, device="cuda")
s = torch.empty(64, 4, dtype=torch.float32, device="cuda")
call(torch.ops._C.per_token_group_fp8_quant, a.cuda(), q, s, 128, 1e-10, -448.0, 448.0, False)
qr, sr2 = oracle.per_token_group_quant_fp8(a, 128)
assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8)) and torch.equal(s.cpu(), sr2)
assert _cabi.launch_count() - n0 >= 3
''')


def test_router_full_size_properties():
    """DeepSeek-V3 routing shape (8192 tokens, 256 experts, 8 groups, 4 chosen, top-8): every row
    picks 8 distinct experts from at most 4 groups, weights renormalise to the scaling factor, the
    histogram adds up; a sampled block of rows equals the oracle."""
    torch.manual_seed(3)
    t, e = 8192, 256
    scores = torch.randn(t, e, device="cuda")
    bias = torch.randn(e, device="cuda") * 0.1
    counts = torch.zeros(e, dtype=torch.int32, device="cuda")
    v, i = flag_gems.grouped_topk(scores, 8, 4, 8, True, 2.5, bias, 1, expert_counts=counts)
    srt = i.sort(dim=1)[0]
    assert bool((srt[:, 1:] != srt[:, :-1]).all())
    groups = (i // 32).long()
    n_groups_used = torch.zeros(t, 8, device="cuda").scatter_(1, groups, 1.0).sum(1)
    assert bool((n_groups_used <= 4).all())
    torch.testing.assert_close(v.sum(1), torch.full((t,), 2.5, device="cuda"), atol=1e-4, rtol=0)
    assert int(counts.sum()) == t * 8
    rv, ri = oracle.grouped_topk(scores[1000:1064].cpu(), 8, 4, 8, True, 2.5, bias.cpu(), 1)
    sel = torch.sigmoid(scores[1000:1064].cpu()) + bias.cpu()[None, :]
    _check_selection(sel, i[1000:1064], ri, tie_eps=1e-6)
    w = torch.empty(t, 8, device="cuda")
    idx = torch.empty(t, 8, dtype=torch.int64, device="cuda")
    src = torch.empty(t, 8, dtype=torch.int32, device="cuda")
    flag_gems.topk_softmax(w, idx, src, scores, True)
    ref_w, ref_i = torch.topk(torch.softmax(scores, -1), 8)
    assert torch.equal(idx, ref_i)
    torch.testing.assert_close(w, ref_w / ref_w.sum(-1, keepdim=True), atol=1e-5, rtol=0)


def test_no_device_errors_recorded():
    assert _cabi.device_status() == 0
