"""GPU parity: quantising every token once and copying its FP8 row and scales into expert order gives
the same bytes and scales as quantising while gathering (the two orders the MoE layer can take)."""
import pytest
import torch

from flaggems_b200 import _cabi
from flaggems_b200.fused import fused_moe as fm
from flaggems_b200.fused.moe_align_block_size import moe_align_block_size

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("t,e,top_k,hidden", [(512, 8, 2, 512), (300, 16, 4, 1024), (2048, 32, 8, 7168)])
def test_quantise_once_then_gather_equals_gathering_quantiser(t, e, top_k, hidden, dtype):
    g = torch.Generator().manual_seed(t + e)
    x = torch.randn(t, hidden, generator=g).to(dtype).cuda()
    ids = torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(t)]).int().cuda()
    numel = t * top_k
    sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, 128, e)
    rows = sorted_ids.numel() // 128 * 128
    a1, a1s = fm._group_quant_once_then_gather(x, 128, sorted_ids, top_k, numel, post_pad, rows)
    b1, b1s = fm._group_quant(x, 128, sorted_ids, top_k, numel, post_pad, rows)
    torch.cuda.synchronize()
    assert _cabi.device_status() == 0
    n_pad = int(post_pad.item())
    real = (sorted_ids[:n_pad] < numel).cpu()
    assert int(real.sum()) == numel
    assert torch.equal(a1[:n_pad].view(torch.uint8).cpu()[real], b1[:n_pad].view(torch.uint8).cpu()[real])
    assert torch.equal(a1s[:n_pad].cpu()[real], b1s[:n_pad].cpu()[real])
    # padding rows are zero bytes in both
    assert not a1[:n_pad].view(torch.uint8).cpu()[~real].any()
    assert not b1[:n_pad].view(torch.uint8).cpu()[~real].any()
