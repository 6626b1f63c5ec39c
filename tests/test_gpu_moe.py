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


def _close(got, ref, rel=1e-2, strict_frac=0.999):
    """Two bounds.  Every element: rtol 1e-2 with atol relative to the output range (rows are
    rounded to bf16 before the fp32 top-k sum, as in the reference, so one bf16 ulp of the
    largest addend can survive cancellation in a small sum).  And the bound the path is specified
    with, rtol 1e-2 + atol 1e-2 per element, must hold for at least `strict_frac` of the elements."""
    got, ref = got.cpu().float(), ref.float()
    torch.testing.assert_close(got, ref, rtol=1e-2, atol=max(1e-2, rel * float(ref.abs().max())))
    frac = float(((got - ref).abs() <= 1e-2 + 1e-2 * ref.abs()).float().mean())
    assert frac >= strict_frac, f"only {frac:.5f} of the elements are within rtol 1e-2 / atol 1e-2"


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


@pytest.mark.parametrize("static", [False, True])
def test_fused_moe_per_tensor(static):
    g = torch.Generator().manual_seed(3)
    t, h, i, e, topk = 100, 512, 256, 8, 2
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * 20).clamp(-448, 448).to(FP8)
    w2 = (torch.randn(e, h, i, generator=g) * 20).clamp(-448, 448).to(FP8)
    s1 = torch.rand(e, generator=g) * 1e-3 + 5e-4
    s2 = torch.rand(e, generator=g) * 1e-3 + 5e-4
    tw, ti = _router(t, e, topk, g)
    a1 = torch.tensor([0.011]) if static else None
    a2 = torch.tensor([0.004]) if static else None
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                                       w1_scale=s1.cuda(), w2_scale=s2.cuda(),
                                       a1_scale=None if a1 is None else a1.cuda(),
                                       a2_scale=None if a2 is None else a2.cuda())
    ref = oracle.fused_moe_per_tensor_fp8(hidden, w1, w2, s1, s2, tw, ti, a1, a2)
    # a value that sits on an FP8 rounding boundary of the shared intermediate scale may flip:
    # allow 2 % of the output range on top of rtol 1e-2
    _close(out, ref, rel=2e-2, strict_frac=0.99)


@pytest.mark.parametrize("block_m", [16, 64, 128])
@pytest.mark.parametrize("mode", ["block", "channel", "tensor"])
def test_dispatch_fused_moe_kernel(block_m, mode):
    """One grouped GEMM through the reference's launch-level API, ids aligned with several block sizes."""
    g = torch.Generator().manual_seed(4)
    t, k, n, e, topk = 77, 512, 384, 8, 2
    a = torch.randn(t, k, generator=g).bfloat16()
    w = torch.randn(e, n, k, generator=g) * 0.05
    tw, ti = _router(t, e, topk, g)
    if mode == "block":
        aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
        wq = torch.empty(e, n, k, dtype=FP8)
        ws = torch.empty(e, n // 128, k // 128)
        for x in range(e):
            wq[x], ws[x] = oracle.quantize_weight_block(w[x])
    elif mode == "channel":
        aq, a_s = oracle.per_token_quant_fp8(a)
        wq, ws = oracle.quantize_weight_per_channel(w)
    else:
        aq, a_s = oracle.per_tensor_quant_fp8(a)
        wq = (w / 0.001).clamp(-448, 448).to(FP8)
        ws = torch.full((e,), 0.001)
    sorted_ids, expert_ids, post_pad = flag_gems.moe_align_block_size(ti.cuda(), block_m, e)
    c = torch.full((t, topk, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    flag_gems.dispatch_fused_moe_kernel(
        aq.cuda(), wq.cuda(), c, a_s.cuda(), ws.cuda(), None, tw.cuda(), sorted_ids, expert_ids, post_pad,
        True, topk, {"BLOCK_SIZE_M": block_m}, torch.bfloat16, True, False, False, False, mode == "channel",
        block_shape=[128, 128] if mode == "block" else None)
    ref = torch.zeros(t, topk, n)
    for x in range(e):
        tok, slot = torch.nonzero(ti == x, as_tuple=True)
        if tok.numel() == 0:
            continue
        if mode == "block":
            r = oracle.block_scaled_mm(aq[tok], wq[x], a_s[tok], ws[x], out_dtype=torch.float32)
        elif mode == "channel":
            r = torch.mm(aq[tok].float(), wq[x].float().t()) * a_s[tok] * ws[x].reshape(1, -1)
        else:
            r = torch.mm(aq[tok].float(), wq[x].float().t()) * a_s * ws[x]
        ref[tok, slot] = (r * tw[tok, slot].float().unsqueeze(1)).bfloat16().float()
    assert not torch.isnan(c.float()).any()
    _close(c, ref)


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


# ---- int8 w8a8 ------------------------------------------------------------------------------
def _int8_channel_weights(e, n, k, g, scale):
    w = torch.randn(e, n, k, generator=g) * scale
    s = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / 127.0
    return (w / s).round().clamp(-128, 127).to(torch.int8), s.squeeze(-1)


def test_per_token_quant_int8_bit_exact():
    from flaggems_b200.fused.fused_moe import _int8_quantize

    g = torch.Generator().manual_seed(40)
    for (m, k, dt) in [(1, 128, torch.bfloat16), (77, 4096, torch.bfloat16), (33, 1000, torch.float16),
                       (5, 7168, torch.float32)]:
        x = (torch.randn(m, k, generator=g) * 3).to(dt)
        x[0, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 3.5, 1e-3, 0.0]).to(dt)  # halves round to even
        q, s = _int8_quantize(x.cuda(), None, True)
        qr, sr = oracle.per_token_quant_int8(x)
        assert q.dtype == torch.int8 and s.shape == (m, 1)
        assert torch.equal(s.cpu(), sr) and torch.equal(q.cpu(), qr)
    q, s = _int8_quantize(torch.zeros(3, 256, dtype=torch.bfloat16, device="cuda"), None, True)
    assert int(q.abs().max()) == 0 and float(s.max()) == pytest.approx(1e-10 / 127.0)


@pytest.mark.parametrize("t,h,i,e,topk", [(1, 128, 256, 8, 2), (16, 256, 512, 8, 2), (32, 128, 256, 8, 4),
                                          (333, 1024, 512, 8, 2), (512, 4096, 1024, 8, 2)])
def test_fused_moe_int8_per_channel(t, h, i, e, topk):
    """Shapes of FUSED_MOE_QUANT_CONFIGS (tests/test_fused_experts_impl.py:64-80) and two larger ones."""
    g = torch.Generator().manual_seed(41)
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1, s1 = _int8_channel_weights(e, 2 * i, h, g, 1.0 / h ** 0.5)
    w2, s2 = _int8_channel_weights(e, h, i, g, 1.0 / i ** 0.5)
    tw, ti = _router(t, e, topk, g)
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), use_int8_w8a8=True,
                                       per_channel_quant=True, w1_scale=s1.cuda(), w2_scale=s2.cuda())
    ref = oracle.fused_moe_per_channel_int8(hidden, w1, w2, s1, s2, tw, ti)
    assert out.shape == hidden.shape and out.dtype == hidden.dtype
    _close(out, ref)


def test_fused_moe_int8_golden(golden_dir):
    """The reference's int8 golden at its own tolerance (tests/test_fused_experts_impl.py:831-835)."""
    for c in torch.load(os.path.join(golden_dir, "fused_moe_fake_quant_int8.pt")):
        out = flag_gems.fused_experts_impl(c["hidden"].cuda(), c["w1"].cuda(), c["w2"].cuda(), c["topk_weights"].cuda(),
                                           c["topk_ids"].cuda(), use_int8_w8a8=True, per_channel_quant=True,
                                           w1_scale=c["w1_scale"].cuda(), w2_scale=c["w2_scale"].cuda())
        ref = c["out"].float()
        torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-1, atol=max(5e-2, float(ref.abs().max()) * 2e-2))
    with pytest.raises(NotImplementedError):
        flag_gems.fused_experts_impl(c["hidden"].cuda(), c["w1"].cuda(), c["w2"].cuda(), c["topk_weights"].cuda(),
                                     c["topk_ids"].cuda(), use_int8_w8a8=True, w1_scale=c["w1_scale"].cuda(),
                                     w2_scale=c["w2_scale"].cuda())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("t,h,i,e,topk", [(33, 256, 128, 8, 2), (200, 1024, 512, 16, 4), (512, 4096, 1024, 8, 2),
                                          (1, 512, 256, 4, 1)])
def test_fused_moe_unquantised_16bit(t, h, i, e, topk, dtype):
    """The default path of fused_experts_impl (no quantisation flags): 16-bit tcgen05 grouped GEMMs."""
    g = torch.Generator().manual_seed(21)
    hidden = torch.randn(t, h, generator=g).to(dtype)
    w1 = (torch.randn(e, 2 * i, h, generator=g) * h ** -0.5).to(dtype)
    w2 = (torch.randn(e, h, i, generator=g) * i ** -0.5).to(dtype)
    tw, ti = _router(t, e, topk, g)
    tw = tw.to(dtype)
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda())
    ref = oracle.fused_moe_16bit(hidden, w1, w2, tw, ti)
    assert out.shape == hidden.shape and out.dtype == dtype
    _close(out, ref)
    assert _cabi.device_status() == 0


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("t,e,h,i,topk", [(1, 8, 128, 256, 2), (4, 8, 128, 256, 2), (16, 8, 256, 512, 2),
                                          (32, 8, 128, 256, 2), (64, 8, 512, 1024, 2)])
def test_fused_moe_weight_only(t, e, h, i, topk, bits):
    """Recipe of tests/test_fused_experts_impl.py:880-1030 (int8 w8a16, and int4 values in int8 containers):
    per-channel symmetric weights, bf16 activations.  Against the oracle at the path's own tolerance and
    against the reference test's fp32 golden at the reference test's tolerance."""
    g = torch.Generator().manual_seed(0)
    dtype = torch.bfloat16
    hidden = torch.randn(t, h, generator=g).to(dtype)
    qmax, qmin = (127, -128) if bits == 8 else (7, -8)
    def quant(w):
        sc = w.abs().amax(-1, keepdim=True).clamp(min=1e-10) / qmax
        return (w / sc).round().clamp(qmin, qmax).to(torch.int8), sc.squeeze(-1)
    w1, s1 = quant(torch.randn(e, 2 * i, h, generator=g) * h ** -0.5)
    w2, s2 = quant(torch.randn(e, h, i, generator=g) * i ** -0.5)
    tw, ti = _router(t, e, topk, g)
    kw = dict(use_int8_w8a16=True) if bits == 8 else dict(use_int4_w4a16=True)
    out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                       per_channel_quant=True, w1_scale=s1.cuda(), w2_scale=s2.cuda(), **kw)
    _close(out, oracle.fused_moe_16bit(hidden, w1, w2, tw, ti, s1, s2))
    # the reference test's golden: everything in fp32, rows weighted and rounded, summed in the output type
    gold = torch.zeros(t, h, dtype=dtype)
    for m in range(t):
        for j in range(topk):
            ex = int(ti[m, j])
            z = hidden[m].float() @ (w1[ex].float() * s1[ex].unsqueeze(-1)).t()
            gate, up = z[:i], z[i:]
            r = ((gate * torch.sigmoid(gate)) * up) @ (w2[ex].float() * s2[ex].unsqueeze(-1)).t()
            gold[m] += (tw[m, j].float() * r).to(dtype)
    rtol, atol_rel = (2e-1, 2e-2) if bits == 8 else (3e-1, 5e-2)
    torch.testing.assert_close(out.cpu(), gold, rtol=rtol, atol=max(5e-2, float(gold.abs().max()) * atol_rel))
    assert _cabi.device_status() == 0


def test_fused_moe_weight_only_golden(golden_dir):
    """The committed outputs of the reference's weight-only golden, at the reference tests' tolerances."""
    for c in torch.load(os.path.join(golden_dir, "fused_moe_weight_only.pt")):
        kw = dict(use_int8_w8a16=True) if c["bits"] == 8 else dict(use_int4_w4a16=True)
        out = flag_gems.fused_experts_impl(c["hidden"].cuda(), c["w1"].cuda(), c["w2"].cuda(), c["topk_weights"].cuda(),
                                           c["topk_ids"].cuda(), per_channel_quant=True, w1_scale=c["w1_scale"].cuda(),
                                           w2_scale=c["w2_scale"].cuda(), **kw)
        ref = c["out"].float()
        rtol, rel = (2e-1, 2e-2) if c["bits"] == 8 else (3e-1, 5e-2)
        torch.testing.assert_close(out.cpu().float(), ref, rtol=rtol, atol=max(5e-2, ref.abs().max().item() * rel))


@pytest.mark.parametrize("block_m", [16, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dispatch_fused_moe_kernel_unquantised(block_m, dtype):
    """The launch-level API with 16-bit operands and no quantisation flags (the reference's plain branch)."""
    g = torch.Generator().manual_seed(5)
    t, k, n, e, topk = 77, 520, 384, 8, 2
    a = torch.randn(t, k, generator=g).to(dtype)
    w = (torch.randn(e, n, k, generator=g) * 0.05).to(dtype)
    tw, ti = _router(t, e, topk, g)
    sorted_ids, expert_ids, post_pad = flag_gems.moe_align_block_size(ti.cuda(), block_m, e)
    c = torch.full((t, topk, n), float("nan"), dtype=dtype, device="cuda")
    flag_gems.dispatch_fused_moe_kernel(
        a.cuda(), w.cuda(), c, None, None, None, tw.cuda(), sorted_ids, expert_ids, post_pad,
        True, topk, {"BLOCK_SIZE_M": block_m}, dtype, False, False, False, False, False)
    ref = torch.zeros(t, topk, n)
    for x in range(e):
        tok, slot = torch.nonzero(ti == x, as_tuple=True)
        if tok.numel():
            r = torch.mm(a[tok].float(), w[x].float().t())
            ref[tok, slot] = (r * tw[tok, slot].float().unsqueeze(1)).to(dtype).float()
    assert not torch.isnan(c.float()).any()
    _close(c, ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("mode", ["block", "channel"])
def test_fused_moe_fp8_other_activation_types(mode, dtype):
    """The reference accepts fp16 and fp32 hidden states as well (fused_moe.py:1879); intermediates and the
    output then have that type."""
    g = torch.Generator().manual_seed(17)
    t, h, i, e, topk = 96, 512, 256, 8, 2
    hidden = torch.randn(t, h, generator=g).to(dtype)
    tw, ti = _router(t, e, topk, g)
    tw = tw.to(dtype)
    if mode == "block":
        w1 = torch.empty(e, 2 * i, h, dtype=FP8)
        w2 = torch.empty(e, h, i, dtype=FP8)
        s1 = torch.empty(e, 2 * i // 128, h // 128)
        s2 = torch.empty(e, h // 128, i // 128)
        for x in range(e):
            w1[x], s1[x] = oracle.quantize_weight_block(torch.randn(2 * i, h, generator=g) * 0.02)
            w2[x], s2[x] = oracle.quantize_weight_block(torch.randn(h, i, generator=g) * 0.02)
        out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                           use_fp8_w8a8=True, w1_scale=s1.cuda(), w2_scale=s2.cuda(),
                                           block_shape=[128, 128])
        ref = oracle.fused_moe_block_fp8(hidden, w1, w2, s1, s2, tw, ti)
    else:
        w1, s1 = oracle.quantize_weight_per_channel(torch.randn(e, 2 * i, h, generator=g) * 0.02)
        w2, s2 = oracle.quantize_weight_per_channel(torch.randn(e, h, i, generator=g) * 0.02)
        out = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(),
                                           use_fp8_w8a8=True, per_channel_quant=True,
                                           w1_scale=s1.cuda(), w2_scale=s2.cuda())
        ref = oracle.fused_moe_per_channel_fp8(hidden, w1, w2, s1, s2, tw, ti)
    assert out.dtype == dtype
    _close(out, ref)
    assert _cabi.device_status() == 0


def test_fused_moe_16bit_expert_map_inplace_and_empty():
    """The unquantised path under the reference's expert-parallel convention (non-local experts map to -1 and
    contribute zeros; the halves add up), in place, through outplace_fused_experts, and with no tokens."""
    g = torch.Generator().manual_seed(23)
    t, h, i, e, topk = 96, 512, 256, 8, 2
    hidden = torch.randn(t, h, generator=g).bfloat16()
    w1 = (torch.randn(e, 2 * i, h, generator=g) * h ** -0.5).bfloat16()
    w2 = (torch.randn(e, h, i, generator=g) * i ** -0.5).bfloat16()
    tw, ti = _router(t, e, topk, g)
    full = flag_gems.fused_experts_impl(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda())
    parts = []
    for lo in (0, 4):
        emap = torch.full((e,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        parts.append(flag_gems.fused_experts_impl(hidden.cuda(), w1[lo:lo + 4].cuda(), w2[lo:lo + 4].cuda(), tw.cuda(),
                                                  ti.cuda(), global_num_experts=e, expert_map=emap.cuda()))
    torch.testing.assert_close((parts[0].float() + parts[1].float()).cpu(), full.float().cpu(), rtol=2e-2, atol=2e-2)
    hc = hidden.cuda().clone()
    flag_gems.inplace_fused_experts(hc, w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda())
    assert torch.equal(hc, full)
    assert torch.equal(flag_gems.outplace_fused_experts(hidden.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda()), full)
    empty = flag_gems.fused_experts_impl(hidden[:0].cuda(), w1.cuda(), w2.cuda(), tw[:0].cuda(), ti[:0].cuda())
    assert empty.shape == (0, h)
    assert _cabi.device_status() == 0
