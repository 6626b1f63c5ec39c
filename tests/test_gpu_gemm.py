"""GPU parity: scaled FP8 GEMMs (tcgen05) vs the CPU fp32 oracle, rtol/atol 1e-2."""
import os

import pytest
import torch

import flag_gems
import oracle
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
TOL = dict(rtol=1e-2, atol=1e-2)


def _close(got, want, **tol):
    tol = tol or TOL
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol)


def _llama_like(m, n, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = torch.randn(n, k, generator=g) * 0.02
    wq, sw = oracle.quantize_weight_per_channel(w)
    aq, sa = oracle.per_token_quant_fp8(a)
    return aq, sa, wq, sw, g


@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (16, 512, 4096), (128, 4096, 4096), (256, 4096, 4096),
                                   (1024, 6144, 4096), (33, 208, 496), (83, 7744, 3888), (129, 144, 144),
                                   (512, 4096, 14336),
                                   # decode-sized M: the narrow tiles that keep every SM streaming weights
                                   (1, 4096, 4096), (16, 6144, 4096), (32, 28672, 4096), (33, 4096, 4096),
                                   (128, 4096, 14336), (8, 4096, 14336)])
@pytest.mark.parametrize("bias", [False, True])
def test_cutlass_scaled_mm_per_token_per_channel(m, n, k, bias):
    aq, sa, wq, sw, g = _llama_like(m, n, k)
    b = torch.randn(n, generator=g).bfloat16() if bias else None
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    wq_c = wq.cuda()
    flag_gems.cutlass_scaled_mm(c, aq.cuda(), wq_c.t(), sa.cuda().view(-1), sw.cuda(),
                                None if b is None else b.cuda())
    ref = oracle.scaled_mm(aq, wq.t(), sa, sw, b)
    if b is None:
        _close(c, ref)
    else:
        # The bias is added after rounding to bf16, so one bf16 ulp of the pre-bias value
        # (2^-8 relative) survives a cancelling bias: allow for it on top of rtol/atol 1e-2.
        pre = oracle.scaled_mm(aq, wq.t(), sa, sw, None).float().abs()
        err = (c.cpu().float() - ref.float()).abs()
        assert bool((err <= 1e-2 + 1e-2 * ref.float().abs() + pre * 2.0 ** -7).all()), float(err.max())


@pytest.mark.parametrize("pa,pb", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_cutlass_scaled_mm_scale_kinds(pa, pb, out_dtype):
    m, n, k = 192, 384, 512
    g = torch.Generator().manual_seed(1)
    a = torch.randn(m, k, generator=g).clamp(-448, 448).to(FP8)
    w = torch.randn(n, k, generator=g).clamp(-448, 448).to(FP8)
    sa = torch.rand(m if pa else 1, generator=g) * 0.02 + 0.01
    sb = torch.rand(n if pb else 1, generator=g) * 0.02 + 0.01
    c = torch.empty(m, n, dtype=out_dtype, device="cuda")
    flag_gems.cutlass_scaled_mm(c, a.cuda(), w.cuda().t(), sa.cuda(), sb.cuda())
    _close(c, oracle.scaled_mm(a, w.t(), sa, sb, None, out_dtype))


def test_cutlass_scaled_mm_baseline_config0():
    """configs[0]: act_quant(A[256,4096], block=K) feeding W[4096,4096] per-channel."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn(256, 4096, generator=g).bfloat16()
    w = torch.randn(4096, 4096, generator=g) * 0.02
    wq, sw = oracle.quantize_weight_per_channel(w)
    aq, sa = flag_gems.act_quant_triton(a.cuda(), 4096)
    aq_r, sa_r = oracle.act_quant(a, 4096)
    assert torch.equal(aq.cpu().view(torch.uint8), aq_r.view(torch.uint8))
    c = torch.empty(256, 4096, dtype=torch.bfloat16, device="cuda")
    flag_gems.cutlass_scaled_mm(c, aq, wq.cuda().t(), sa.view(-1), sw.cuda(), None)
    _close(c, oracle.scaled_mm(aq_r, wq.t(), sa_r, sw))


def test_scaled_mm_golden_fixtures(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "scaled_mm.pt")):
        a = c["a"].view(FP8)
        w = c["b_nk"].view(FP8)
        m, n = a.shape[0], w.shape[0]
        out = torch.empty(m, n, dtype=torch.float32, device="cuda")
        flag_gems.cutlass_scaled_mm(out, a.cuda(), w.cuda().t(), c["sa"].reshape(-1).cuda(),
                                    c["sb"].reshape(-1).cuda())
        ref = c["c_f32_nobias"]
        _close(out, ref, rtol=1e-3, atol=1e-3 * float(ref.abs().max()))


def test_scaled_mm_asserts():
    a = torch.zeros(16, 128, dtype=FP8, device="cuda")
    w = torch.zeros(32, 128, dtype=FP8, device="cuda")
    s = torch.ones(1, device="cuda")
    c = torch.empty(16, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):
        flag_gems.cutlass_scaled_mm(c, a, w.t().contiguous(), s, s)  # b not column-major
    with pytest.raises(AssertionError):
        flag_gems.cutlass_scaled_mm(c, a, torch.zeros(64, 32, dtype=FP8, device="cuda").t().t(), s, s)
    with pytest.raises(AssertionError):
        flag_gems.cutlass_scaled_mm(c, a, w.t(), s.double(), s)


@pytest.mark.parametrize("m,n,k", [(16, 16, 16), (17, 31, 32), (64, 48, 80)])
@pytest.mark.parametrize("mode", ["scalar", "rowwise_1d", "rowwise_2d"])
@pytest.mark.parametrize("out_dtype,use_bias", [(torch.bfloat16, False), (torch.float16, True), (torch.float32, True)])
def test_aten_scaled_mm(m, n, k, mode, out_dtype, use_bias):
    """Shapes, scale modes and tolerance of tests/test_scaled_mm.py:144 (fp8 rows)."""
    g = torch.Generator().manual_seed(2)
    mat1 = (torch.randn(m, k, generator=g) * 0.25).to(FP8)
    mat2 = (torch.randn(k, n, generator=g) * 0.25).to(FP8)
    if mode == "scalar":
        sa, sb = torch.tensor([0.75]), torch.tensor([1.25])
    else:
        sa, sb = torch.linspace(0.75, 1.25, m), torch.linspace(1.25, 0.75, n)
        if mode == "rowwise_2d":
            sa, sb = sa.reshape(m, 1), sb.reshape(1, n)
    bias = (torch.randn(n, generator=g) * 0.25).to(out_dtype) if use_bias else None
    ref = oracle.scaled_mm(mat1, mat2, sa, sb, bias, out_dtype, bias_after_round=False)
    with flag_gems.use_gems():
        res = torch._scaled_mm(mat1.cuda(), mat2.cuda(), sa.cuda(), sb.cuda(),
                               bias=None if bias is None else bias.cuda(),
                               scale_result=torch.tensor([2.0], device="cuda"),
                               out_dtype=out_dtype, use_fast_accum=True)
    assert res.dtype == out_dtype
    _close(res, ref)
    out = torch.empty(m, n, dtype=out_dtype, device="cuda")
    with flag_gems.use_gems():
        ret = torch.ops.aten._scaled_mm.out(mat1.cuda(), mat2.cuda(), sa.cuda(), sb.cuda(),
                                            bias=None if bias is None else bias.cuda(), out_dtype=out_dtype,
                                            out=out)
    assert ret.data_ptr() == out.data_ptr()
    _close(out, ref)


@pytest.mark.parametrize("m,n,k", [(16, 16, 16), (17, 31, 32), (64, 48, 80), (300, 520, 256), (4, 4096, 1024)])
@pytest.mark.parametrize("mode", ["scalar", "rowwise_2d"])
@pytest.mark.parametrize("use_bias", [False, True])
def test_aten_scaled_mm_default_out_dtype_is_fp8(m, n, k, mode, use_bias):
    """torch._scaled_mm(a, b, sa, sb) without out_dtype: the result has the operands' dtype
    (src/flag_gems/ops/scaled_mm.py:214-220).  FP8 bytes must equal the oracle's wherever the fp32
    value is not within accumulation-order distance of a rounding boundary: at most a few
    elements may differ, and then by one FP8 step."""
    g = torch.Generator().manual_seed(12)
    mat1 = (torch.randn(m, k, generator=g) * 0.5).to(FP8)
    mat2 = (torch.randn(k, n, generator=g) * 0.5).to(FP8)
    if mode == "scalar":
        sa, sb = torch.tensor([0.75]), torch.tensor([40.0])  # large enough for some values to saturate
    else:
        sa, sb = torch.linspace(0.75, 1.25, m).reshape(m, 1), torch.linspace(30.0, 50.0, n).reshape(1, n)
    bias = (torch.randn(n, generator=g) * 4).bfloat16() if use_bias else None
    ref = oracle.scaled_mm(mat1, mat2, sa, sb, bias, FP8, bias_after_round=False)
    with flag_gems.use_gems():
        res = torch._scaled_mm(mat1.cuda(), mat2.cuda(), sa.cuda(), sb.cuda(),
                               bias=None if bias is None else bias.cuda())
        out = torch.empty(m, n, dtype=FP8, device="cuda")
        torch.ops.aten._scaled_mm.out(mat1.cuda(), mat2.cuda(), sa.cuda(), sb.cuda(),
                                      bias=None if bias is None else bias.cuda(), out=out)
    assert res.dtype == FP8 and res.shape == (m, n)
    assert torch.equal(res.view(torch.uint8), out.view(torch.uint8))
    got, want = res.cpu().float(), ref.float()
    assert bool(torch.isfinite(got).all()) and float(got.abs().max()) <= 448.0
    if mode == "scalar" and m * n >= 100000:
        assert float(want.abs().max()) == 448.0, "the case is meant to exercise saturation"
    differ = got != want
    assert float(differ.float().mean()) <= 2e-3
    # a differing element is one FP8 step away: relative distance at most 2^-3
    assert bool(((got - want).abs()[differ] <= 0.126 * want.abs()[differ].clamp(min=2.0 ** -6)).all())


# ---- block-scaled ------------------------------------------------------------------------

def _block_case(m, n, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = torch.randn(n, k, generator=g) * 0.02
    aq, a_s = oracle.per_token_group_quant_fp8(a, 128)
    wq, w_s = oracle.quantize_weight_block(w, 128)
    return aq, a_s, wq, w_s


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (64, 128, 128), (256, 256, 256), (83, 7752, 3840),
                                   (1, 2112, 7168), (64, 4096, 7168), (512, 2112, 7168), (300, 1536, 1024),
                                   (16, 4096, 7168), (128, 2112, 7168), (1, 24576, 7168), (40, 18432, 7168),
                                   # wide enough for the 192-column tile (scale blocks straddle its halves)
                                   (2048, 2112, 1024), (1100, 4096, 512), (1536, 1408, 384)])
def test_w8a8_block_fp8_matmul(m, n, k):
    aq, a_s, wq, w_s = _block_case(m, n, k)
    out = flag_gems.w8a8_block_fp8_matmul(aq.cuda(), wq.cuda(), a_s.cuda(), w_s.cuda(), [128, 128])
    assert out.dtype == torch.bfloat16 and out.shape == (m, n)
    _close(out, oracle.block_scaled_mm(aq, wq, a_s, w_s))


def test_w8a8_block_reference_test_recipe():
    """Recipe of tests/test_w8a8_block_fp8_matmul.py: randn->fp8 operands, scales 0.01*rand+0.005,
    fp16 output, rtol 1e-3 / atol 1e-4*K (fp16 rounding aside)."""
    g = torch.Generator().manual_seed(3)
    for (m, n, k) in [(128, 256, 512), (84, 7168, 3840)]:
        a = torch.randn(m, k, generator=g).clamp(-448, 448).to(FP8)
        b = torch.randn(n, k, generator=g).clamp(-448, 448).to(FP8)
        a_s = 0.01 * torch.rand(m, k // 128, generator=g) + 0.005
        b_s = 0.01 * torch.rand((n + 127) // 128, k // 128, generator=g) + 0.005
        out = flag_gems.w8a8_block_fp8_matmul(a.cuda(), b.cuda(), a_s.cuda(), b_s.cuda(), [128, 128], torch.float16)
        ref = oracle.block_scaled_mm(a, b, a_s, b_s, out_dtype=torch.float32)
        _close(out, ref, rtol=2e-3, atol=1e-4 * k)


def test_block_scaled_golden_and_negative_scales(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "block_scaled_mm.pt")):
        a, b = c["a"].view(FP8), c["b"].view(FP8)
        out = flag_gems.w8a8_block_fp8_matmul(a.cuda(), b.cuda(), c["a_s"].cuda(), c["b_s"].cuda(), [128, 128],
                                              torch.float32)
        _close(out, c["c"], rtol=1e-3, atol=1e-3 * float(c["c"].abs().max()))
    g = torch.Generator().manual_seed(4)
    a = torch.randn(40, 256, generator=g).clamp(-448, 448).to(FP8)
    b = torch.randn(384, 256, generator=g).clamp(-448, 448).to(FP8)
    a_s = torch.randn(40, 2, generator=g) * 0.01      # the reference's MoE test draws signed scales
    b_s = torch.randn(3, 2, generator=g) * 0.01
    out = flag_gems.w8a8_block_fp8_matmul(a.cuda(), b.cuda(), a_s.cuda(), b_s.cuda(), [128, 128], torch.float32)
    ref = oracle.block_scaled_mm(a, b, a_s, b_s, out_dtype=torch.float32)
    _close(out, ref, rtol=1e-3, atol=1e-3 * float(ref.abs().max()))


def test_fp8_matmul_and_blockwise_cutlass_form():
    aq, a_s, wq, w_s = _block_case(200, 1024, 2048, seed=5)
    ref = oracle.block_scaled_mm(aq, wq, a_s, w_s)
    out = flag_gems.fp8_matmul(aq.cuda(), a_s.cuda(), wq.cuda(), w_s.cuda())
    _close(out, ref)
    c = torch.empty(200, 1024, dtype=torch.bfloat16, device="cuda")
    flag_gems.cutlass_scaled_mm(c, aq.cuda(), wq.cuda().t(), a_s.cuda(), w_s.cuda().t().contiguous())
    _close(c, ref)


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 256), (3900, 4112, 272), (8192, 2304, 144)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_scaled_mm_cta_pair_tiles(m, n, k, out_dtype):
    """Shapes with at least three waves of 256 x 256 tiles take the two-CTA (cta_group::2)
    kernel: every row and column, ragged edges and a bias included, against the oracle."""
    aq, sa, wq, sw, g = _llama_like(m, n, k, seed=11)
    b = torch.randn(n, generator=g).to(out_dtype)
    c = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    flag_gems.cutlass_scaled_mm(c, aq.cuda(), wq.cuda().t(), sa.cuda().view(-1), sw.cuda(), b.cuda())
    ref = oracle.scaled_mm(aq, wq.t(), sa, sw, b, out_dtype=out_dtype)
    pre = oracle.scaled_mm(aq, wq.t(), sa, sw, None, out_dtype=out_dtype).float().abs()
    err = (c.cpu().float() - ref.float()).abs()
    assert bool((err <= 1e-2 + 1e-2 * ref.float().abs() + pre * 2.0 ** -7).all()), float(err.max())
    assert _cabi.device_status() == 0


def test_gemm_full_size_linearity():
    """configs[1]/[2] sizes without a CPU oracle pass: doubling every scale doubles the output
    exactly (powers of two commute with every rounding), and a sampled block of rows/columns
    matches the oracle."""
    g = torch.Generator().manual_seed(6)
    m, n, k = 4096, 4096, 7168
    aq = torch.randn(m, k, generator=g).clamp(-448, 448).to(FP8).cuda()
    wq = torch.randn(n, k, generator=g).clamp(-448, 448).to(FP8).cuda()
    a_s = (torch.rand(m, k // 128, generator=g) * 1e-2 + 1e-3).cuda()
    w_s = (torch.rand(n // 128, k // 128, generator=g) * 1e-2 + 1e-3).cuda()
    o1 = flag_gems.w8a8_block_fp8_matmul(aq, wq, a_s, w_s, [128, 128])
    o2 = flag_gems.w8a8_block_fp8_matmul(aq, wq, a_s * 2, w_s, [128, 128])
    assert torch.equal(o2.float(), o1.float() * 2)
    rows = torch.arange(1000, 1064)
    ref = oracle.block_scaled_mm(aq[rows].cpu(), wq[512:768].cpu(), a_s[rows].cpu(), w_s[4:6].cpu())
    _close(o1[rows][:, 512:768], ref)
    sa = (torch.rand(m, generator=g) * 1e-2 + 1e-3).cuda()
    sb = (torch.rand(n, generator=g) * 1e-2 + 1e-3).cuda()
    c1 = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    c2 = torch.empty_like(c1)
    flag_gems.cutlass_scaled_mm(c1, aq, wq.t(), sa, sb)
    flag_gems.cutlass_scaled_mm(c2, aq, wq.t(), sa * 2, sb)
    assert torch.equal(c2.float(), c1.float() * 2)
    ref = oracle.scaled_mm(aq[rows].cpu(), wq[512:768].cpu().t(), sa[rows].cpu(), sb[512:768].cpu())
    _close(c1[rows][:, 512:768], ref)


def test_no_device_errors_recorded():
    assert _cabi.device_status() == 0


# ---- aten _scaled_grouped_mm ---------------------------------------------------------------
def _grouped_case(case, g, groups=3, m=5, n=16, k=32):
    def mk(*shape):
        return (torch.randn(*shape, generator=g) * 0.25).to(FP8)

    if case == "m_varying":
        sizes = [2, 3, 4] if groups == 3 else [int(x) for x in torch.randint(0, 3 * m, (groups,), generator=g)]
        total = sum(sizes)
        offs = torch.tensor(sizes, dtype=torch.int32).cumsum(0).to(torch.int32)
        return mk(total, k), mk(groups, n, k).transpose(1, 2), torch.linspace(0.75, 1.25, total), \
            torch.linspace(1.25, 0.75, groups * n).reshape(groups, n), offs
    if case == "batch":
        return mk(groups, m, k), mk(groups, n, k).transpose(1, 2), torch.linspace(0.75, 1.25, groups * m).reshape(groups, m), \
            torch.linspace(1.25, 0.75, groups * n).reshape(groups, n), None
    if case == "k_varying":
        offs = torch.tensor([8, 20, k], dtype=torch.int32)
        return mk(m, k), mk(n, k).t(), torch.linspace(0.75, 1.25, 3 * m), torch.linspace(1.25, 0.75, 3 * n), offs
    offs = torch.tensor([8, 20, 32], dtype=torch.int32)
    return mk(groups, m, k), mk(32, k).t(), torch.linspace(0.75, 1.25, groups * m).reshape(groups, m), \
        torch.linspace(1.25, 0.75, 32), offs


@pytest.mark.parametrize("case", ["m_varying", "batch", "k_varying", "n_varying"])
@pytest.mark.parametrize("use_bias", [False, True])
@pytest.mark.parametrize("out_dtype", [None, torch.float32])
def test_aten_scaled_grouped_mm(case, use_bias, out_dtype):
    """The four operand forms, shapes, scales and bias kinds of tests/test_scaled_grouped_mm.py:60-127, through
    torch._scaled_grouped_mm under use_gems(); rtol/atol 1e-2 against the fp32 oracle (the reference's own
    FP8 tolerance there is rtol 0.5 / atol 0.25)."""
    g = torch.Generator().manual_seed(21)
    a, b, sa, sb, offs = _grouped_case(case, g)
    n = b.shape[-1]
    bias = None
    if use_bias:
        bias = torch.randn(3, n, generator=g) if case in ("batch", "k_varying") else torch.randn(n, generator=g)
    target = out_dtype or torch.bfloat16
    ref = oracle.scaled_grouped_mm(a, b, sa, sb, offs, bias, target)
    dev = lambda t: None if t is None else t.cuda()  # noqa: E731
    with flag_gems.use_gems():
        res = torch._scaled_grouped_mm(dev(a), dev(b), dev(sa), dev(sb), offs=dev(offs), bias=dev(bias),
                                       out_dtype=out_dtype, use_fast_accum=True)
    assert res.dtype == target and res.shape == ref.shape
    _close(res, ref)


@pytest.mark.parametrize("groups,m_avg,n,k", [(8, 300, 512, 1024), (64, 40, 2048, 7168), (5, 1, 256, 128)])
def test_scaled_grouped_mm_ragged_groups(groups, m_avg, n, k):
    """Groups of very different sizes, some empty, rows left over after the last group end untouched."""
    g = torch.Generator().manual_seed(22)
    sizes = torch.randint(0, 2 * m_avg + 1, (groups,), generator=g)
    sizes[1] = 0
    total = int(sizes.sum()) + 3  # three rows past the last group end
    offs = sizes.cumsum(0).to(torch.int32)
    a = (torch.randn(total, k, generator=g) * 0.5).to(FP8)
    w = (torch.randn(groups, n, k, generator=g) * 0.5).to(FP8)
    sa, sb = torch.rand(total, generator=g) + 0.5, torch.rand(groups, n, generator=g) * 0.02
    bias = torch.randn(groups, n, generator=g)
    out = flag_gems.scaled_grouped_mm(a.cuda(), w.cuda().transpose(1, 2), sa.cuda(), sb.cuda(), offs.cuda(), bias.cuda())
    used = int(offs[-1])
    ref = oracle.scaled_grouped_mm(a[:used], w.transpose(1, 2), sa[:used], sb, offs, bias)
    _close(out[:used], ref)
    assert _cabi.device_status() == 0


# ---- batched block-scaled products ------------------------------------------------------------
@pytest.mark.parametrize("b,m,n,k", [(4, 37, 256, 512), (2, 300, 384, 1024), (16, 8, 128, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_w8a8_block_fp8_bmm(b, m, n, k, out_dtype):
    g = torch.Generator().manual_seed(31)
    x = torch.randn(b, m, k, generator=g).bfloat16()
    xq, xs = oracle.per_token_group_quant_fp8(x, 128)
    yq = torch.empty(b, n, k, dtype=FP8)
    ys = torch.empty(b, n // 128, k // 128)
    for i in range(b):
        yq[i], ys[i] = oracle.quantize_weight_block(torch.randn(n, k, generator=g) * 0.05)
    z = flag_gems.w8a8_block_fp8_bmm(xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), [128, 128], output_dtype=out_dtype)
    assert z.shape == (b, m, n) and z.dtype == out_dtype
    for i in range(b):
        _close(z[i], oracle.block_scaled_mm(xq[i], yq[i], xs[i], ys[i], out_dtype=out_dtype))
    z2 = torch.full((b, m, n), 7.0, dtype=out_dtype, device="cuda")
    ret = flag_gems.w8a8_block_fp8_bmm(xq.cuda(), yq.cuda(), xs.cuda(), ys.cuda(), z=z2, output_dtype=out_dtype)
    assert ret.data_ptr() == z2.data_ptr() and torch.equal(z2, z)


def test_fp8_einsum_bhr_hdr_bhd():
    """DeepSeek-style absorbed projection: out[b,h,d] = sum_r x[b,h,r] y[h,d,r], permuted views, no copies."""
    g = torch.Generator().manual_seed(32)
    b, h, r, d = 48, 8, 512, 256
    x = torch.randn(b, h, r, generator=g).bfloat16()
    xq, xs = oracle.per_token_group_quant_fp8(x, 128)
    yq = torch.empty(h, d, r, dtype=FP8)
    ys = torch.empty(h, d // 128, r // 128)
    for i in range(h):
        yq[i], ys[i] = oracle.quantize_weight_block(torch.randn(d, r, generator=g) * 0.05)
    z = flag_gems.fp8_einsum("bhr,hdr->bhd", xq.cuda(), xs.cuda(), yq.cuda(), ys.cuda())
    assert z.shape == (b, h, d) and z.dtype == torch.bfloat16 and z.is_contiguous()
    for i in range(h):
        _close(z[:, i], oracle.block_scaled_mm(xq[:, i].contiguous(), yq[i], xs[:, i].contiguous(), ys[i]))
    with pytest.raises(AssertionError):
        flag_gems.fp8_einsum("bhr,hrd->bhd", xq.cuda(), xs.cuda(), yq.cuda(), ys.cuda())
