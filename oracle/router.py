"""CPU oracle: the router kernels that feed the fused MoE path (test infrastructure only).

PARITY UNPINNED by reference goldens: the reference's tests for these two functions
(tests/test_topk_softmax.py, tests/test_grouped_topk.py) hold no CPU golden and no fixed vectors;
they compare against vLLM's CUDA ops at run time.  The restatements below follow the reference's
Triton kernels line by line, and the GPU tests additionally compare the CUDA kernels with vLLM's
ops (the reference's own criterion) when vLLM's compiled ops load on the box.
"""
from typing import Tuple

import torch


def topk_softmax(gating_output: torch.Tensor, topk: int, renormalize: bool = False,
                 index_dtype: torch.dtype = torch.int32) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Softmax over the experts, then k rounds of arg-max with masking.

    Follows src/flag_gems/fused/topk_softmax.py:41-81:
      probs = exp(x - rowmax) / (sum(exp(x - rowmax)) + 1e-8) in fp32              (:54-56)
      round ki: the largest remaining prob and its (lowest) index; the entry becomes -inf (:59-74)
      token_expert_indices[r, ki] = ki * num_rows + r                              (:64-68)
      renormalize: weights / (sum of the k weights + 1e-8)                         (:76-81)
    Returns (topk_weights fp32 [T,k], topk_indices [T,k], token_expert_indices int32 [T,k]).
    """
    assert topk <= 32
    t, e = gating_output.shape
    x = gating_output.float()
    ex = torch.exp(x - x.amax(dim=1, keepdim=True))
    probs = ex / (ex.sum(dim=1, keepdim=True) + 1e-8)
    w = torch.empty(t, topk, dtype=torch.float32)
    idx = torch.empty(t, topk, dtype=torch.int64)
    rows = torch.arange(t)
    for ki in range(topk):
        m = probs.amax(dim=1)
        # lowest index among the maxima
        arg = torch.where(probs == m[:, None], torch.arange(e)[None, :], e).amin(dim=1)
        w[:, ki] = m
        idx[:, ki] = arg
        probs[rows, arg] = -float("inf")
    if renormalize:
        w = w / (w.sum(dim=1, keepdim=True) + 1e-8)
    src = (torch.arange(topk)[None, :] * t + rows[:, None]).to(torch.int32)
    return w, idx.to(index_dtype), src


def grouped_topk(scores: torch.Tensor, n_group: int, topk_group: int, topk: int, renormalize: bool,
                 routed_scaling_factor: float, bias: torch.Tensor, scoring_func: int = 0
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-limited top-k routing (DeepSeek-V3 style).

    Follows src/flag_gems/fused/grouped_topk.py:
      argument checks                                                              (:256-278)
      scoring_func 1: scores = sigmoid(scores.float()).to(dtype)                   (:291-294)
      group score = (max1 + max2).to(dtype) over (scores + bias) computed in the input dtype and
        widened to fp32; max2 = max1 when the maximum occurs more than once        (:24-76)
      non-finite (NaN, +inf) group scores count as -inf; if every group is -inf the token gets
        weights 1/topk and indices 0..topk-1                                       (:117-125, :221-227)
      the topk_group best groups, ties to the lower group index                    (:127-158)
      k rounds of arg-max over (scores + bias) of the experts in the chosen groups, ties to the
        lowest expert index; the weight is the score WITHOUT bias                  (:160-208)
      weights *= routed_scaling_factor / (sum + 1e-20) when renormalize, else
        *= routed_scaling_factor                                                   (:210-216)
    Returns (topk_values fp32 [T,k], topk_indices int32 [T,k]).
    """
    if scores.ndim != 2:
        raise ValueError("scores must be a 2D Tensor")
    t, e = scores.shape
    if e % n_group != 0:
        raise ValueError("num_experts must be divisible by n_group")
    if n_group > 32:
        raise ValueError("n_group should be smaller than or equal to 32")
    if topk > 32:
        raise ValueError("topk should be smaller than or equal to 32 for now")
    if scoring_func not in (0, 1):
        raise ValueError("scoring_func must be 0 (none) or 1 (sigmoid)")
    if bias.dtype != scores.dtype:
        bias = bias.to(scores.dtype)
    bias = bias.flatten()
    if len(bias) != e:
        raise ValueError(f"bias length ({len(bias)}) must match num_experts ({e})")
    epg = e // n_group
    dt = scores.dtype
    sp = torch.sigmoid(scores.float()).to(dt) if scoring_func == 1 else scores
    neg_inf = -float("inf")
    xb = (sp + bias[None, :]).float()  # the add happens in the input dtype
    vals = torch.empty(t, topk, dtype=torch.float32)
    idxs = torch.empty(t, topk, dtype=torch.int32)
    for r in range(t):
        g = xb[r].reshape(n_group, epg)
        max1 = g.amax(dim=1)
        cnt = (g == max1[:, None]).sum(dim=1)
        g2 = torch.where((g == max1[:, None]) & (cnt == 1)[:, None], torch.tensor(neg_inf), g)
        max2 = g2.amax(dim=1)
        gs = (max1 + max2).to(dt).float()
        finite = (gs == gs) & (gs != float("inf"))
        gs = torch.where(finite, gs, torch.tensor(neg_inf))
        if float(gs.max()) == neg_inf:
            vals[r] = 1.0 / topk
            idxs[r] = torch.arange(topk, dtype=torch.int32)
            continue
        # topk_group best groups, ties to the lower index: stable sort on descending score
        order = sorted(range(n_group), key=lambda j: (-float(gs[j]), j))
        chosen = torch.zeros(n_group, dtype=torch.bool)
        chosen[order[:topk_group]] = True
        sel = chosen.repeat_interleave(epg)
        score = torch.where(sel, xb[r], torch.tensor(neg_inf)).clone()
        out_v = torch.zeros(topk, dtype=torch.float32)
        out_i = torch.zeros(topk, dtype=torch.int32)
        for i in range(topk):
            m = score.max()
            k = int(torch.nonzero(score == m)[0])
            out_v[i] = sp[r, k].float()
            out_i[i] = k
            score[k] = neg_inf
        scale = routed_scaling_factor / (out_v.sum() + 1e-20) if renormalize else routed_scaling_factor
        vals[r] = out_v * scale
        idxs[r] = out_i
    return vals, idxs
