"""GPU parity: the fused MoE layer (grouped tcgen05 GEMMs) vs the CPU oracle."""
import os

import pytest
import torch

import flag_gems
import oracle
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _router(t, e, topk, g):
    logits = torch.randn(t, e, generator=g)
    tw, ti = torch.topk(torch.softmax(logits, -1), topk)
    return (tw / tw.sum(-1, keepdim=True)).bfloat16(), ti


def _close(got, ref, rel=1e-2):
    got, ref = got.cpu().float(), ref.float()
    torch.testing.assert_close(got, ref, rtol=1e-2, atol=max(1e-2, rel * float(ref.abs().max())))


@pytest.mark.parametrize("t,h,i,e,topk", [(64, 256, 128, 8, 2), (333, 512, 256, 8, 2), (16, 1024, 384, 4, 1),
                                          (1, 256, 128, 8, 2), (512, 4096, 1024, 8, 2)])
def test_fused_moe_per_channel(t, h, i, e, topk):
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1, s1 = oracle.quantize_weight_per_channel(torch.randn(e, 2 * i, h, generator=g) * 0.02)
    w2, s2 = oracle.quantize_weight_per_channel(torch.randn(e, h, i, generator=g) * 0.02)
    tw, ti = _router(t, e, topk, g)
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                       use_fp8_w8a8=True, per_channel_quant=True,
                                       w1_scale=s1.cuda(), w2_scale=s2.cuda())
    ref = oracle.fused_moe_per_channel_fp8(hidden, w1, w2, s1, s2, tw, ti)
    assert out.shape == hidden.shape and out.dtype == hidden.dtype
    _close(out, ref)


@pytest.mark.parametrize("t,h,i,e,topk", [(64, 256, 128, 8, 2), (200, 512, 256, 16, 4), (32, 7168, 2048, 8, 8),
                                          (129, 1024, 128, 64, 6)])
def test_fused_moe_block_fp8(t, h, i, e, topk):
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1 = torch.empty(e, 2 * i, h, dtype=FP8)
    w2 = torch.empty(e, h, i, dtype=FP8)
    s1 = torch.empty(e, 2 * i // 128, h // 128)
    s2 = torch.empty(e, h // 128, i // 128)
    for x in range(e):
        w1[x], s1[x] = oracle.quantize_weight_block(torch.randn(2 * i, h, generator=g) * 0.02)
        w2[x], s2[x] = oracle.quantize_weight_block(torch.randn(h, i, generator=g) * 0.02)
    tw, ti = _router(t, e, topk, g)
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                       use_fp8_w8a8=True, w1_scale=s1.cuda(), w2_scale=s2.cuda(),
                                       block_shape=[128, 128])
    ref = oracle.fused_moe_block_fp8(hidden, w1, w2, s1, s2, tw, ti)
    _close(out, ref)


def test_fused_moe_block_fp8_golden(golden_dir):
    """Against the output of the reference's own golden (tests/test_fused_experts_impl.py:604-662),
    with that test's tolerance."""
    c = torch.load(os.path.join(golden_dir, "fused_moe_block_fp8.pt"))
    out = flag_gems.fused_experts_impl(c["hidden"].cuda(), c["w1"].view(FP8).cuda(), c["w2"].view(FP8).cuda(),
                                       c["topk_weights"].cuda(), c["topk_ids"].cuda(), use_fp8_w8a8=True,
                                       w1_scale=c["w1_scale"].cuda(), w2_scale=c["w2_scale"].cuda(),
                                       block_shape=[128, 128])
    ref = c["out"].float()
    torch.testing.assert_close(out.cpu().float(), ref, rtol=0.2, atol=max(0.05, 0.05 * float(ref.abs().max())))


def test_fused_moe_expert_map_and_inplace():
    """The reference's expert-parallel convention: non-local experts map to -1 and contribute zeros;
    the two halves add up to the full layer."""
    g = torch.Generator().manual_seed(2)
    t, h, i, e, topk = 96, 512, 256, 8, 2
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1, s1 = oracle.quantize_weight_per_channel(torch.randn(e, 2 * i, h, generator=g) * 0.02)
    w2, s2 = oracle.quantize_weight_per_channel(torch.randn(e, h, i, generator=g) * 0.02)
    tw, ti = _router(t, e, topk, g)
    kw = dict(use_fp8_w8a8=True, per_channel_quant=True)
    full = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                        w1_scale=s1.cuda(), w2_scale=s2.cuda(), **kw)
    parts = []
    for lo in (0, 4):
        emap = torch.full((e,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        parts.append(flag_gems.fused_experts_impl(
            hidden.cuda(), w1[lo:lo + 4].cuda(), w2[lo:lo + 4].cuda(), tw.cuda(), ti.cuda(),
            global_num_experts=e, expert_map=emap.cuda(), w1_scale=s1[lo:lo + 4].cuda(),
            w2_scale=s2[lo:lo + 4].cuda(), **kw))
    torch.testing.assert_close((parts[0].float() + parts[1].float()).cpu(), full.float().cpu(), rtol=2e-2, atol=2e-2)
    hc = hidden.cuda().clone()
    flag_gems.inplace_fused_experts(hc, w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                    w1_scale=s1.cuda(), w2_scale=s2.cuda(), **kw)
    assert torch.equal(hc, full)


def test_no_device_errors_recorded():
    assert _cabi.device_status() == 0
