"""Two devices driven from ONE process: the library's per-device state (shared-memory opt-ins, cluster
occupancy, SM counts, status words, built-in scratch) must be set up for each device on its first use
there, not once per process.  Needs two visible GPUs; skipped otherwise."""
import pytest
import torch

import flag_gems
import oracle
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
TOL = dict(rtol=1e-2, atol=1e-2)


def _gemm_case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = torch.randn(n, k, generator=g) * 0.02
    aq, sa = oracle.per_token_group_quant_fp8(a, 128)
    wq, sw = oracle.quantize_weight_block(w, 128)
    return aq, sa, wq, sw


def _run_on(dev):
    """Every kernel family once on ``dev`` (which is not made the current device by the caller)."""
    # block-scaled GEMM: wide persistent tile (large dynamic shared memory) and the decode-sized
    # split-K cluster launch (cluster occupancy query)
    for m, n, k in ((256, 512, 1024), (1, 4096, 2048)):
        aq, sa, wq, sw = _gemm_case(m, n, k, seed=m)
        out = flag_gems.w8a8_block_fp8_matmul(aq.to(dev), wq.to(dev), sa.to(dev), sw.to(dev), [128, 128],
                                              output_dtype=torch.bfloat16)
        assert out.device == torch.device(dev)
        ref = oracle.block_scaled_mm(aq, wq, sa, sw, 128, 128, torch.bfloat16)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **TOL)
    # moe_align with more experts than the default shared-memory limit serves
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (2048, 8), generator=g, dtype=torch.int32)
    so, eo, no = flag_gems.moe_align_block_size(ids.to(dev), 64, 512)
    sr, er, nr = oracle.moe_align_block_size(ids, 64, 512)
    assert torch.equal(so.cpu(), sr) and torch.equal(eo.cpu(), er) and torch.equal(no.cpu(), nr)
    # group quantisation (bit-exact)
    x = torch.randn(64, 1024, generator=g).bfloat16()
    q, s = flag_gems.per_token_group_quant_fp8(x.to(dev), 128)
    qr, sr_ = oracle.per_token_group_quant_fp8(x, 128)
    assert torch.equal(q.cpu().view(torch.uint8), qr.view(torch.uint8)) and torch.equal(s.cpu(), sr_)


def test_second_device_after_first_in_one_process():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    _run_on("cuda:0")
    _run_on("cuda:1")
    _run_on("cuda:0")
    assert torch.cuda.current_device() == 0  # the device guards restored the caller's device
    for d in (0, 1):
        with torch.cuda.device(d):
            torch.cuda.synchronize()
            assert _cabi.device_status() == 0
