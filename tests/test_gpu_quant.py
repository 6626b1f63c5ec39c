"""GPU parity: FP8 quantisation kernels vs the CPU oracle, bit for bit (bytes and scales)."""
import os

import pytest
import torch

import flag_gems
import oracle
from tests._isolated import check_isolated
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu
U8 = torch.uint8


def _bits(t):
    return t.contiguous().view(torch.int32)


def _assert_bytes_equal(got, want):
    got = got.cpu().view(U8)
    want = want.view(U8)
    nbad = int((got != want).sum())
    assert nbad == 0, f"{nbad} of {want.numel()} FP8 bytes differ"


@pytest.mark.parametrize("m", [1, 40, 164, 3454])
@pytest.mark.parametrize("n", [128, 896, 2048, 8192])
@pytest.mark.parametrize("block", [64, 128])
@pytest.mark.parametrize("fmt", [None, "ue8m0"])
def test_act_quant_reference_shapes(m, n, block, fmt):
    """Shape grid of the reference's own test (tests/test_act_quant.py:33-36), seed 0."""
    torch.manual_seed(0)
    x = torch.randn(m, n).bfloat16()
    y, s = flag_gems.act_quant_triton(x.cuda(), block, fmt)
    yr, sr = oracle.act_quant(x, block, fmt)
    assert y.dtype == torch.float8_e4m3fn and s.dtype == torch.float32 and s.shape == (m, n // block)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(y, yr)


def test_act_quant_baseline_config_and_per_token_block():
    """First benchmark configuration: A bf16 [256, 4096], group 128; and block_size = K (per-token scales)."""
    torch.manual_seed(0)
    x = torch.randn(256, 4096).bfloat16()
    for block in (128, 4096, 512, 1024):
        y, s = flag_gems.act_quant_triton(x.cuda(), block)
        yr, sr = oracle.act_quant(x, block)
        assert torch.equal(_bits(s.cpu()), _bits(sr)), block
        _assert_bytes_equal(y, yr)


def test_act_quant_golden_fixtures(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "act_quant.pt")):
        y, s = flag_gems.act_quant_triton(c["x"].cuda(), c["block_size"], c["scale_fmt"])
        assert torch.equal(_bits(s.cpu()), _bits(c["s"]))
        _assert_bytes_equal(y, c["y"])


def test_act_quant_edge_values():
    x = torch.zeros(3, 256).bfloat16()
    x[1, :] = 1e-6
    x[2, 0] = 3e38
    x[2, 1] = -448.0
    y, s = flag_gems.act_quant_triton(x.cuda(), 128)
    yr, sr = oracle.act_quant(x, 128)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(y, yr)
    e = torch.empty(0, 128).bfloat16().cuda()
    y, s = flag_gems.act_quant_triton(e, 128)
    assert y.shape == (0, 128) and s.shape == (0, 1)


def test_act_quant_3d_and_large():
    torch.manual_seed(1)
    x = torch.randn(4, 33, 512).bfloat16()
    y, s = flag_gems.act_quant_triton(x.cuda(), 128)
    yr, sr = oracle.act_quant(x, 128)
    assert y.shape == x.shape and s.shape == (4, 33, 4)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(y, yr)
    x = (torch.randn(12027, 2048) * 3).bfloat16()
    y, s = flag_gems.act_quant_triton(x.cuda(), 128)
    yr, sr = oracle.act_quant(x, 128)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(y, yr)


@pytest.mark.parametrize("tokens", [7, 83, 2048])
@pytest.mark.parametrize("d", [512, 4096, 5120, 13824])
@pytest.mark.parametrize("group", [64, 128, 256, 512])
def test_group_quant_reference_shapes(tokens, d, group):
    """Shape grid of tests/test_per_token_group_quant_fp8.py (accuracy_utils FP8_QUANT_SHAPES)."""
    torch.manual_seed(0)
    x = torch.rand(tokens, d).bfloat16()
    for ue8m0 in (False, True):
        q, s = flag_gems.per_token_group_quant_fp8(x.cuda(), group, scale_ue8m0=ue8m0)
        qr, sr = oracle.per_token_group_quant_fp8(x, group, scale_ue8m0=ue8m0)
        assert torch.equal(_bits(s.cpu()), _bits(sr))
        _assert_bytes_equal(q, qr)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_group_quant_dtypes_layouts(dt):
    torch.manual_seed(2)
    x = (torch.randn(65, 1536) * 2).to(dt)
    q, s = flag_gems.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True)
    qr, sr = oracle.per_token_group_quant_fp8(x, 128, column_major_scales=True)
    assert s.shape == sr.shape and s.stride() == sr.stride()
    assert torch.equal(_bits(s.cpu().contiguous()), _bits(sr.contiguous()))
    _assert_bytes_equal(q, qr)
    # non power-of-two-friendly group (generic kernel) and a row-strided view
    q, s = flag_gems.per_token_group_quant_fp8(x.cuda(), 96)
    qr, sr = oracle.per_token_group_quant_fp8(x, 96)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(q, qr)
    xv = x.cuda()[:, :1024]
    q, s = flag_gems.per_token_group_quant_fp8(xv, 128)
    qr, sr = oracle.per_token_group_quant_fp8(x[:, :1024].contiguous(), 128)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(q, qr)


def test_group_quant_golden_and_tiny(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "per_token_group_quant.pt")):
        q, s = flag_gems.per_token_group_quant_fp8(c["x"].cuda(), c["group_size"])
        qr, sr = oracle.per_token_group_quant_fp8(c["x"], c["group_size"])
        assert torch.equal(_bits(s.cpu()), _bits(sr))
        _assert_bytes_equal(q, qr)
        _assert_bytes_equal(q, c["q"])
    x = torch.zeros(4, 256).bfloat16()
    x[1] = 1e-12
    q, s = flag_gems.per_token_group_quant_fp8(x.cuda(), 128)
    qr, sr = oracle.per_token_group_quant_fp8(x, 128)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(q, qr)


def test_group_quant_full_size_scale_roundtrip():
    """Third benchmark configuration's size (M=16384, K=7168): properties that need no CPU oracle pass:
    every scale equals amax/448 of its group computed independently on the device, and
    dequantised values stay within half an FP8 step of the input."""
    torch.manual_seed(3)
    x = torch.randn(16384, 7168, device="cuda").bfloat16()
    q, s = flag_gems.per_token_group_quant_fp8(x, 128)
    amax = x.float().view(16384, 56, 128).abs().amax(-1).clamp(min=1e-10)
    assert torch.equal(s, amax / torch.tensor(448.0, device="cuda"))
    deq = q.float().view(16384, 56, 128) * s.unsqueeze(-1)
    err = (deq - x.float().view(16384, 56, 128)).abs()
    assert bool((err <= amax.unsqueeze(-1) * (0.0625 / 0.875) + 1e-12).all())
    # sampled rows against the CPU oracle, bit for bit
    rows = torch.randint(0, 16384, (64,))
    qr, sr = oracle.per_token_group_quant_fp8(x[rows.cuda()].cpu(), 128)
    assert torch.equal(_bits(s[rows.cuda()].cpu()), _bits(sr))
    _assert_bytes_equal(q[rows.cuda()], qr)


@pytest.mark.parametrize("shape", [(5, 256), (64, 1024), (4096, 4096), (300, 14336), (3, 24576)])
def test_per_token_quant(shape):
    torch.manual_seed(4)
    x = torch.randn(*shape).bfloat16()
    x[0] = 0
    q, s = flag_gems.fused.fused_moe._fp8_quantize(x.cuda(), None, True, None)
    qr, sr = oracle.per_token_quant_fp8(x)
    assert s.shape == sr.shape
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(q, qr)


def test_per_token_quant_golden(golden_dir):
    for c in torch.load(os.path.join(golden_dir, "per_token_quant.pt")):
        q, s = flag_gems.fused.fused_moe._fp8_quantize(c["x"].cuda(), None, True, None)
        assert torch.equal(_bits(s.cpu()), _bits(c["s"]))
        _assert_bytes_equal(q, c["q"])


def test_per_tensor_quant(golden_dir):
    c = torch.load(os.path.join(golden_dir, "fp8_quantize_per_tensor.pt"))
    fq = flag_gems.fused.fused_moe._fp8_quantize
    q, s = fq(c["x"].cuda(), None, False, None)
    assert torch.equal(s.cpu(), c["s_dynamic"])
    _assert_bytes_equal(q, c["q_dynamic"])
    q, s = fq(c["x"].cuda(), c["scale_static"].cuda(), False, None)
    _assert_bytes_equal(q, c["q_static"])
    torch.manual_seed(6)
    x = (torch.randn(777, 2048) * 5).bfloat16()
    q, s = fq(x.cuda(), None, False, None)
    qr, sr = oracle.per_tensor_quant_fp8(x)
    assert torch.equal(_bits(s.cpu()), _bits(sr))
    _assert_bytes_equal(q, qr)


def test_vllm_op_writes_in_place():
    """torch.ops._C.per_token_group_fp8_quant / cutlass_scaled_mm as patch_empty_vllm() defines
    them (in a process of their own: the registrations must not reach later tests)."""
    check_isolated('''
import torch, flag_gems, oracle
flag_gems.patch_empty_vllm()
torch.manual_seed(5)
x = torch.randn(33, 512).bfloat16()
q = torch.empty(33, 512, dtype=torch.float8_e4m3fn, device="cuda")
s = torch.empty(4, 33, dtype=torch.float32, device="cuda").t()
torch.ops._C.per_token_group_fp8_quant(x.cuda(), q, s, 128, 1e-10, -448.0, 448.0, False)
qr, sr = oracle.per_token_group_quant_fp8(x, 128)
assert torch.equal(s.cpu().contiguous().view(torch.int32), sr.view(torch.int32))
assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8))
w = torch.randn(256, 512) * 0.02
wq, sw = oracle.quantize_weight_per_channel(w)
aq, sa = oracle.per_token_quant_fp8(x)
c = torch.empty(33, 256, dtype=torch.bfloat16, device="cuda")
torch.ops._C.cutlass_scaled_mm(c, aq.cuda(), wq.cuda().t(), sa.cuda().view(-1), sw.cuda(), None)
ref = oracle.scaled_mm(aq, wq.t(), sa, sw)
torch.testing.assert_close(c.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
''')


def test_no_device_errors_recorded():
    assert _cabi.device_status() == 0
