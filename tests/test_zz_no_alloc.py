"""The allocation-free entry point of the routed-expert pipeline, through the C ABI.

Some embedders cannot let a library allocate: the device's memory was planned up front, or an
allocation at that point would stall the whole device.  For them
``fg_moe_routed_block_fp8_local_noalloc`` keeps its scratch in a fixed array inside the library.
It must give exactly what ``fg_moe_routed_block_fp8_local`` gives with a caller-owned workspace,
also on a second call that finds the first call's leftovers in the array, and it must refuse
problems that do not fit.  (This file sorts last so that a run stopping at the first failure has
already been through every other test.)
"""
import pytest
import torch

import oracle
from flaggems_b200 import _cabi

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
E, H, I = 8, 512, 256


def _weights(seed):
    g = torch.Generator().manual_seed(seed)
    w1 = torch.empty(E, 2 * I, H, dtype=FP8)
    w2 = torch.empty(E, H, I, dtype=FP8)
    s1 = torch.empty(E, 2 * I // 128, H // 128)
    s2 = torch.empty(E, H // 128, I // 128)
    for e in range(E):
        w1[e], s1[e] = oracle.quantize_weight_block(torch.randn(2 * I, H, generator=g) * 0.05)
        w2[e], s2[e] = oracle.quantize_weight_block(torch.randn(H, I, generator=g) * 0.05)
    return [t.cuda() for t in (w1, w2, s1, s2)]


def _inputs(tokens, topk, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(tokens, H, generator=g).bfloat16().cuda()
    tw, ti = torch.topk(torch.softmax(torch.randn(tokens, E, generator=g), -1), topk)
    return hidden, tw.float().contiguous().cuda(), ti.to(torch.int32).contiguous().cuda()


def _with_workspace(hidden, tw, ti, w):
    L = _cabi.lib()
    t, topk = ti.shape
    need = L.fg_moe_routed_workspace_bytes(t * topk, E, H, I)
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    y = torch.full((t * topk, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    _cabi.check(L.fg_moe_routed_block_fp8_local(
        y.data_ptr(), hidden.data_ptr(), 0, ti.data_ptr(), 0, tw.data_ptr(), 2, t, topk,
        w[0].data_ptr(), w[1].data_ptr(), w[2].data_ptr(), w[3].data_ptr(), E, H, I,
        ws.data_ptr(), ws.numel(), _cabi.stream_ptr()))
    return y


def _no_alloc(hidden, tw, ti, w):
    t, topk = ti.shape
    y = torch.full((t * topk, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    _cabi.check(_cabi.lib().fg_moe_routed_block_fp8_local_noalloc(
        y.data_ptr(), hidden.data_ptr(), 0, ti.data_ptr(), 0, tw.data_ptr(), 2, t, topk,
        w[0].data_ptr(), w[1].data_ptr(), w[2].data_ptr(), w[3].data_ptr(), E, H, I, _cabi.stream_ptr()))
    return y


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    w = _weights(0)
    # second call is smaller and differently routed: stale rows of the first stay in the array
    for tokens, topk, seed in ((192, 2, 1), (37, 4, 2)):
        hidden, tw, ti = _inputs(tokens, topk, seed)
        want = _with_workspace(hidden, tw, ti, w)
        got = _no_alloc(hidden, tw, ti, w)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, want)
    assert _cabi.device_status() == 0


def test_oversize_problem_is_refused_with_a_clear_error():
    w = _weights(0)
    hidden, tw, ti = _inputs(16384, 4, 3)  # 65536 routed rows need far more than the built-in scratch
    with pytest.raises(NotImplementedError, match="built-in scratch"):
        _no_alloc(hidden, tw, ti, w)
