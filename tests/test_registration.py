"""enable / only_enable / use_gems and the vLLM op overrides (host logic, no GPU)."""
import torch

import flag_gems


def test_use_gems_registers_and_restores():
    with flag_gems.use_gems():
        assert flag_gems.all_registered_keys() == ["_scaled_mm", "_scaled_mm.out", "_scaled_grouped_mm"]
        assert flag_gems.all_registered_ops() == ["scaled_mm", "scaled_mm_out", "scaled_grouped_mm"]
    with flag_gems.use_gems(exclude=["scaled_mm_out", "scaled_grouped_mm"]):
        assert flag_gems.all_registered_keys() == ["_scaled_mm"]
    with flag_gems.use_gems(include=["scaled_grouped_mm"]):
        assert flag_gems.all_registered_keys() == ["_scaled_grouped_mm"]
    with flag_gems.use_gems(include=["scaled_mm_out"]):
        assert flag_gems.all_registered_keys() == ["_scaled_mm.out"]


def test_record_writes_op_log(tmp_path):
    import logging

    p = tmp_path / "oplist.log"
    with flag_gems.use_gems(record=True, path=str(p)):
        logging.getLogger("flag_gems.ops.scaled_mm").debug("GEMS SCALED_MM")
    text = p.read_text()
    # the reference's tests/test_enable_api.py:72-97 greps "[DEBUG] flag_gems.ops.<op>" prefixes
    assert "[DEBUG] flag_gems.ops.scaled_mm: GEMS SCALED_MM" in text


def test_module_loggers_carry_the_reference_names():
    import importlib

    fm = importlib.import_module("flaggems_b200.fused.fused_moe")
    sm = importlib.import_module("flaggems_b200.ops.scaled_mm")
    gq = importlib.import_module("flaggems_b200.ops.per_token_group_quant_fp8")
    assert sm.logger.name == "flag_gems.ops.scaled_mm"
    assert fm.logger.name == "flag_gems.fused.fused_moe"
    assert gq.logger.name == "flag_gems.ops.per_token_group_quant_fp8"


def test_inplace_outplace_signatures_bind_positionally():
    """Parameter names, order and defaults of src/flag_gems/fused/fused_moe.py:2188-2209 and
    :2241-2262: a custom-op registration passes all 21 arguments by position."""
    import inspect

    names = ["hidden_states", "w1", "w2", "topk_weights", "topk_ids", "activation", "apply_router_weight_on_input",
             "use_fp8_w8a8", "use_int8_w8a8", "use_int8_w8a16", "use_int4_w4a16", "per_channel_quant",
             "global_num_experts", "w1_scale", "w2_scale", "a1_scale", "a2_scale", "block_shape", "w1_bias",
             "w2_bias"]
    defaults = ["silu", False, False, False, False, False, False, -1, None, None, None, None, None, None, None]
    for fn in (flag_gems.inplace_fused_experts, flag_gems.outplace_fused_experts):
        sig = inspect.signature(fn)
        assert list(sig.parameters) == names
        assert [p.default for p in list(sig.parameters.values())[5:]] == defaults
        assert all(p.kind == inspect.Parameter.POSITIONAL_OR_KEYWORD for p in sig.parameters.values())
        bound = sig.bind(*range(len(names)))  # every argument by position
        assert bound.arguments["activation"] == 5 and bound.arguments["w2_bias"] == len(names) - 1
    impl = list(inspect.signature(flag_gems.fused_experts_impl).parameters)
    assert impl[:7] == ["hidden_states", "w1", "w2", "topk_weights", "topk_ids", "inplace", "activation"]
    assert len(impl) == 25


def test_patch_empty_vllm_is_idempotent_and_defines_ops():
    from tests._isolated import check_isolated

    check_isolated('''
import torch, flag_gems
flag_gems.patch_empty_vllm()
flag_gems.patch_empty_vllm()
for ns, op in (("_C", "cutlass_scaled_mm"), ("_C", "per_token_group_fp8_quant"), ("_moe_C", "moe_align_block_size"),
               ("_moe_C", "moe_sum"), ("_moe_C", "topk_softmax"), ("_moe_C", "grouped_topk")):
    assert hasattr(getattr(torch.ops, ns), op), op
''')


def test_api_surface_matches_reference_names():
    for name in ["act_quant_triton", "per_token_group_quant_fp8", "SUPPORTED_FP8_DTYPE", "cutlass_scaled_mm",
                 "scaled_mm", "scaled_mm_out", "w8a8_block_fp8_matmul", "fp8_matmul", "moe_align_block_size",
                 "moe_align_block_size_triton", "fused_experts_impl", "inplace_fused_experts",
                 "outplace_fused_experts", "moe_sum", "silu_and_mul", "silu_and_mul_out", "enable", "only_enable",
                 "use_gems", "all_registered_ops", "all_registered_keys", "patch_empty_vllm",
                 "apply_gems_patches_to_vllm", "device", "vendor_name"]:
        assert hasattr(flag_gems, name), name
    assert flag_gems.device == "cuda" and flag_gems.vendor_name == "nvidia"


def test_unsupported_modes_raise_cleanly():
    import pytest

    h = torch.zeros(2, 128, dtype=torch.bfloat16)
    w1 = torch.zeros(2, 64, 128)
    w2 = torch.zeros(2, 128, 32)
    tw = torch.ones(2, 1)
    ti = torch.zeros(2, 1, dtype=torch.int32)
    with pytest.raises(NotImplementedError):
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti, use_int8_w8a8=True)
    with pytest.raises(NotImplementedError):
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti, ocp_mx_scheme="w_mxfp4_a_bf16")
    with pytest.raises(NotImplementedError):
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti, use_int8_w8a16=True, use_fp8_w8a8=True)
    # the unquantised path exists, and like every path it has no CPU fallback
    from flaggems_b200._cabi import FlagGemsB200Error
    with pytest.raises(FlagGemsB200Error):
        flag_gems.fused_experts_impl(h, w1.bfloat16(), w2.bfloat16(), tw, ti)
    with pytest.raises(AssertionError):
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti, activation="gelu", use_fp8_w8a8=True)


def test_scaled_grouped_mm_argument_checks():
    """Messages of src/flag_gems/ops/scaled_grouped_mm.py:262-366, raised before any device work."""
    import pytest

    fp8 = torch.float8_e4m3fn
    a2, b3 = torch.zeros(9, 32).to(fp8), torch.zeros(3, 32, 16).to(fp8)
    sa, sb = torch.ones(9), torch.ones(3, 16)
    offs = torch.tensor([2, 5, 9], dtype=torch.int32)
    f = flag_gems.scaled_grouped_mm
    with pytest.raises(RuntimeError, match="offs must be provided"):
        f(a2, b3, sa, sb)
    with pytest.raises(RuntimeError, match="offs has to be int32"):
        f(a2, b3, sa, sb, offs.long())
    with pytest.raises(RuntimeError, match="offs length must match the group count"):
        f(a2, b3, sa, sb, offs[:2])
    with pytest.raises(RuntimeError, match="scale_a must be a 1D tensor with length 9"):
        f(a2, b3, sa[:8], sb, offs)
    with pytest.raises(RuntimeError, match="scale_b must have shape"):
        f(a2, b3, sa, sb[:2], offs)
    with pytest.raises(RuntimeError, match="cannot be multiplied"):
        f(a2, torch.zeros(3, 16, 16).to(fp8), sa, sb, offs)
    with pytest.raises(RuntimeError, match="same dtype"):
        f(a2, b3.float(), sa, sb, offs)
    with pytest.raises(RuntimeError, match="scale_result is not supported"):
        f(a2, b3, sa, sb, offs, scale_result=torch.ones(1))
    with pytest.raises(RuntimeError, match="bias must have shape"):
        f(a2, b3, sa, sb, offs, bias=torch.zeros(7))
    with pytest.raises(RuntimeError, match="offs must be None when both inputs are 3D"):
        f(torch.zeros(3, 5, 32).to(fp8), b3, torch.ones(3, 5), sb, offs)
    with pytest.raises(RuntimeError, match="mat_a has to be 2D or 3D"):
        f(a2[0], b3, sa, sb, offs)
    with pytest.raises(Exception, match="CUDA tensors only"):  # valid arguments on the CPU: no fallback
        f(a2, b3, sa, sb, offs)


def test_scaled_grouped_mm_oracle_against_einsum():
    """The oracle of the new op against an independent formulation, all four operand forms."""
    import oracle

    g = torch.Generator().manual_seed(0)
    fp8 = torch.float8_e4m3fn
    a = (torch.randn(3, 5, 32, generator=g) * 0.25).to(fp8)
    b = (torch.randn(3, 32, 16, generator=g) * 0.25).to(fp8)
    sa, sb = torch.rand(3, 5, generator=g) + 0.5, torch.rand(3, 16, generator=g) + 0.5
    ref = torch.einsum("gmk,gkn->gmn", a.float(), b.float()) * sa[:, :, None] * sb[:, None, :]
    out = oracle.scaled_grouped_mm(a, b, sa, sb, out_dtype=torch.float32)
    torch.testing.assert_close(out, ref)
    offs = torch.tensor([5, 10, 15], dtype=torch.int32)
    out2 = oracle.scaled_grouped_mm(a.reshape(15, 32), b, sa.reshape(-1), sb, offs, out_dtype=torch.float32)
    torch.testing.assert_close(out2.reshape(3, 5, 16), ref)
