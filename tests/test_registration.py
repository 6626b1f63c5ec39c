"""enable / only_enable / use_gems and the vLLM op overrides (host logic, no GPU)."""
import torch

import flag_gems


def test_use_gems_registers_and_restores():
    with flag_gems.use_gems():
        assert flag_gems.all_registered_keys() == ["_scaled_mm", "_scaled_mm.out"]
        assert flag_gems.all_registered_ops() == ["scaled_mm", "scaled_mm_out"]
    with flag_gems.use_gems(exclude=["scaled_mm_out"]):
        assert flag_gems.all_registered_keys() == ["_scaled_mm"]
    with flag_gems.use_gems(include=["scaled_mm_out"]):
        assert flag_gems.all_registered_keys() == ["_scaled_mm.out"]


def test_record_writes_op_log(tmp_path):
    import logging

    p = tmp_path / "oplist.log"
    with flag_gems.use_gems(record=True, path=str(p)):
        logging.getLogger("flaggems_b200.ops.scaled_mm").debug("GEMS SCALED_MM")
    assert "GEMS SCALED_MM" in p.read_text()


def test_patch_empty_vllm_is_idempotent_and_defines_ops():
    flag_gems.patch_empty_vllm()
    flag_gems.patch_empty_vllm()
    assert hasattr(torch.ops._C, "cutlass_scaled_mm")
    assert hasattr(torch.ops._C, "per_token_group_fp8_quant")
    assert hasattr(torch.ops._moe_C, "moe_align_block_size")
    assert hasattr(torch.ops._moe_C, "moe_sum")


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
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti)
    with pytest.raises(AssertionError):
        flag_gems.fused_experts_impl(h, w1, w2, tw, ti, activation="gelu", use_fp8_w8a8=True)
