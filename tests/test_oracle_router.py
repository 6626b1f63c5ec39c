"""CPU checks of the router oracles against independent torch formulas (no GPU)."""
import pytest
import torch

import oracle


@pytest.mark.parametrize("t,e,k", [(1, 4, 2), (8, 16, 4), (32, 64, 8), (50, 255, 30)])
@pytest.mark.parametrize("renorm", [False, True])
def test_topk_softmax_oracle_matches_torch_topk(t, e, k, renorm):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(t, e, generator=g)
    w, idx, src = oracle.topk_softmax(x, k, renorm, torch.int64)
    ref_w, ref_i = torch.topk(torch.softmax(x, -1), k)
    if renorm:
        ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert torch.equal(idx, ref_i)
    torch.testing.assert_close(w, ref_w, atol=1e-6, rtol=1e-5)
    assert torch.equal(src, (torch.arange(k)[None, :] * t + torch.arange(t)[:, None]).int())
    if renorm:
        torch.testing.assert_close(w.sum(-1), torch.ones(t), atol=1e-5, rtol=0)


def test_topk_softmax_oracle_ties_go_to_the_lower_index():
    x = torch.zeros(2, 8)
    x[1, 5] = 1.0
    w, idx, _ = oracle.topk_softmax(x, 3)
    assert idx[0].tolist() == [0, 1, 2]
    assert idx[1].tolist() == [5, 0, 1]


def _grouped_topk_torch(scores, n_group, topk_group, topk, renormalize, scaling, bias, scoring_func):
    """The usual torch formulation of bias-corrected group-limited routing (no ties assumed)."""
    s = torch.sigmoid(scores.float()).to(scores.dtype) if scoring_func == 1 else scores
    t, e = s.shape
    sb = (s + bias[None, :]).float()
    group_scores = sb.view(t, n_group, -1).topk(2, dim=-1)[0].sum(-1).to(scores.dtype).float()
    group_idx = torch.topk(group_scores, topk_group, dim=-1)[1]
    mask = torch.zeros_like(group_scores).scatter_(1, group_idx, 1).bool()
    mask = mask.repeat_interleave(e // n_group, dim=1)
    masked = sb.masked_fill(~mask, float("-inf"))
    ids = torch.topk(masked, topk, dim=-1)[1]
    w = s.float().gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling, ids.int()


@pytest.mark.parametrize("t,e,n_group,topk_group,topk", [(3, 8, 2, 1, 1), (8, 16, 4, 2, 2), (32, 64, 8, 2, 8),
                                                         (16, 256, 8, 4, 8)])
@pytest.mark.parametrize("renorm", [False, True])
@pytest.mark.parametrize("scoring", [0, 1])
def test_grouped_topk_oracle_matches_torch_formula(t, e, n_group, topk_group, topk, renorm, scoring):
    g = torch.Generator().manual_seed(45)
    scores = torch.randn(t, e, generator=g)
    bias = torch.randn(e, generator=g)
    v, i = oracle.grouped_topk(scores, n_group, topk_group, topk, renorm, 2.5, bias, scoring)
    rv, ri = _grouped_topk_torch(scores, n_group, topk_group, topk, renorm, 2.5, bias, scoring)
    assert torch.equal(i, ri)
    torch.testing.assert_close(v, rv, atol=1e-6, rtol=1e-5)


def test_grouped_topk_oracle_edge_cases():
    scores = torch.full((2, 8), float("-inf"))
    bias = torch.zeros(8)
    v, i = oracle.grouped_topk(scores, 2, 1, 2, True, 1.0, bias)
    assert torch.equal(v, torch.full((2, 2), 0.5)) and i.tolist() == [[0, 1], [0, 1]]
    # equal group scores: the lower group wins; equal experts: the lower index wins
    scores = torch.ones(1, 8)
    v, i = oracle.grouped_topk(scores, 2, 1, 2, False, 1.0, bias)
    assert i.tolist() == [[0, 1]]
    # a maximum that occurs twice counts twice in the group score (group 1: 3+3 beats group 0: 4+1)
    scores = torch.tensor([[4.0, 1.0, 0.0, 0.0, 3.0, 3.0, 0.0, 0.0]])
    v, i = oracle.grouped_topk(scores, 2, 1, 1, False, 1.0, bias)
    assert i.tolist() == [[4]]
    with pytest.raises(ValueError, match="divisible"):
        oracle.grouped_topk(torch.zeros(1, 9), 2, 1, 1, False, 1.0, torch.zeros(9))
    with pytest.raises(ValueError, match="bias length"):
        oracle.grouped_topk(torch.zeros(1, 8), 2, 1, 1, False, 1.0, torch.zeros(4))
    with pytest.raises(ValueError, match="scoring_func"):
        oracle.grouped_topk(torch.zeros(1, 8), 2, 1, 1, False, 1.0, torch.zeros(8), 2)


def test_router_host_api_checks_arguments_before_touching_a_device():
    """The host wrappers keep the reference's argument checks and error classes, and refuse CPU
    tensors instead of falling back."""
    import flag_gems

    with pytest.raises(ValueError, match="2D"):
        flag_gems.grouped_topk(torch.zeros(8), 2, 1, 1, False, 1.0, torch.zeros(8))
    with pytest.raises(ValueError, match="divisible"):
        flag_gems.grouped_topk(torch.zeros(1, 9), 2, 1, 1, False, 1.0, torch.zeros(9))
    with pytest.raises(ValueError, match="n_group"):
        flag_gems.grouped_topk(torch.zeros(1, 64), 64, 1, 1, False, 1.0, torch.zeros(64))
    with pytest.raises(ValueError, match="topk should be"):
        flag_gems.grouped_topk(torch.zeros(1, 64), 2, 1, 33, False, 1.0, torch.zeros(64))
    with pytest.raises(ValueError, match="scoring_func"):
        flag_gems.grouped_topk(torch.zeros(1, 8), 2, 1, 1, False, 1.0, torch.zeros(8), 3)
    with pytest.raises(ValueError, match="bias length"):
        flag_gems.grouped_topk(torch.zeros(1, 8), 2, 1, 1, False, 1.0, torch.zeros(4))
    with pytest.raises(ValueError, match="Unsupported dtype"):
        flag_gems.grouped_topk(torch.zeros(1, 8, dtype=torch.float64), 2, 1, 1, False, 1.0, torch.zeros(8))
    with pytest.raises(Exception, match="(?i)cuda"):
        flag_gems.grouped_topk(torch.zeros(1, 8), 2, 1, 1, False, 1.0, torch.zeros(8))
    w, i, s = torch.empty(2, 2), torch.empty(2, 2, dtype=torch.int16), torch.empty(2, 2, dtype=torch.int32)
    with pytest.raises(TypeError):
        flag_gems.topk_softmax(w, i, s, torch.zeros(2, 8))
    with pytest.raises(AssertionError):
        flag_gems.topk_softmax(torch.empty(2, 33), torch.empty(2, 33, dtype=torch.int32),
                               torch.empty(2, 33, dtype=torch.int32), torch.zeros(2, 64))
    with pytest.raises(Exception, match="(?i)cuda"):
        flag_gems.topk_softmax(w, i.int(), s, torch.zeros(2, 8))
