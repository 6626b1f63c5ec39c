"""vLLM custom-op overrides for the hot path.

Mirrors src/flag_gems/patches/patch_util.py:57-163 and
src/flag_gems/patches/patch_vllm_all.py:425-459,617-717 of the reference: the schemas of
``torch.ops._C`` / ``torch.ops._moe_C`` ops are defined when vLLM's own extension has not
defined them, and the CUDA implementations are replaced by this package's functions.
"""
import torch

_VLLM_OPS_SIGNATURES = {
    "_C": {
        "cutlass_scaled_mm": "(Tensor(a!) out, Tensor input, Tensor weight, "
        "Tensor scale_a, Tensor scale_b, Tensor? bias=None) -> ()",
        "per_token_group_fp8_quant": "(Tensor input, Tensor(a!) output_q, "
        "Tensor(b!) output_s, int group_size, float eps, float fp8_min, "
        "float fp8_max, bool scale_ue8m0=False) -> ()",
    },
    "_moe_C": {
        "moe_align_block_size": "(Tensor topk_ids, int num_experts, "
        "int block_size, Tensor(a!) sorted_token_ids, Tensor(b!) experts_ids, "
        "Tensor(c!) num_tokens_post_pad) -> ()",
        "moe_sum": "(Tensor input, Tensor(a!) output) -> ()",
        "topk_softmax": "(Tensor(a!) topk_weights, Tensor(b!) topk_indices, "
        "Tensor(c!) token_expert_indices, Tensor gating_output, bool renormalize=False, "
        "Tensor? e_score_correction_bias=None) -> ()",
        "grouped_topk": "(Tensor gating_output, int n_group, int topk_group, "
        "int topk, bool renormalize, float routed_scaling_factor, Tensor? bias, "
        "int scoring_func=0) -> (Tensor, Tensor)",
    },
}

libs = {}
_flag_ops_registered = False


def _is_op_registered(lib_name, op_name):
    try:
        ns = getattr(torch.ops, lib_name)
        getattr(ns, op_name)
        return True
    except (AttributeError, RuntimeError):
        return False


def custom_per_token_group_fp8_quant(input, output_q, output_s, group_size, eps, fp8_min, fp8_max,
                                     scale_ue8m0=False, dummy_is_scale_transposed=False, dummy_is_tma_aligned=False):
    """Writes straight into the caller's buffers (row- or column-major scales are inferred
    from the strides of ``output_s`` as the reference adapter does).  The two trailing flags exist
    only in newer vLLM schemas, where they are placeholders; the layout is read from the strides."""
    from .. import _cabi

    assert input.dim() == 2 and input.stride(-1) == 1
    assert output_q.is_contiguous() and output_s.dim() == 2 and output_s.dtype == torch.float32
    m, k = input.shape
    with _cabi.device_guard(input):
        _cabi.check(
            _cabi.lib().fg_per_token_group_quant_fp8(
                _cabi.ptr(input), _cabi.DTYPE_CODE[input.dtype], _cabi.ptr(output_q), _cabi.ptr(output_s),
                m, k, group_size, input.stride(0), k, output_s.stride(0), output_s.stride(1), float(eps),
                1 if scale_ue8m0 else 0, _cabi.stream_ptr(input.device),
            )
        )


def custom_cutlass_scaled_mm(output, input, weight, scale_a, scale_b, bias=None):
    from ..fused.cutlass_scaled_mm import cutlass_scaled_mm

    return cutlass_scaled_mm(output, input, weight, scale_a, scale_b, bias)


def custom_moe_align_block_size(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids,
                                num_tokens_post_pad, maybe_expert_map=None):
    from ..fused.moe_align_block_size import moe_align_block_size_triton

    if maybe_expert_map is not None:
        # newer vLLM schemas carry this argument; the reference's op (patch_util.py:78-81) has none
        raise NotImplementedError("moe_align_block_size with maybe_expert_map is not implemented")
    moe_align_block_size_triton(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids,
                                num_tokens_post_pad)


def custom_moe_sum(input, output):
    from ..fused.moe_sum import moe_sum

    moe_sum(input, output)


def custom_topk_softmax(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize=False,
                        e_score_correction_bias=None):
    from ..fused.topk_softmax import topk_softmax

    if e_score_correction_bias is not None:
        # newer vLLM schemas carry this argument; the reference's topk_softmax has no such input
        raise NotImplementedError("topk_softmax with e_score_correction_bias is not implemented")

    topk_softmax(topk_weights, topk_indices, token_expert_indices, gating_output, renormalize)


def custom_moe_grouped_topk(gating_output, n_group, topk_group, topk, renormalize, routed_scaling_factor, bias,
                            scoring_func=0):
    from ..fused.grouped_topk import grouped_topk

    return grouped_topk(scores=gating_output, n_group=n_group, topk_group=topk_group, topk=topk,
                        renormalize=renormalize, routed_scaling_factor=routed_scaling_factor, bias=bias,
                        scoring_func=scoring_func)


_VLLM_OPS_IMPLS = {
    "_C": {
        "cutlass_scaled_mm": custom_cutlass_scaled_mm,
        "per_token_group_fp8_quant": custom_per_token_group_fp8_quant,
    },
    "_moe_C": {
        "moe_align_block_size": custom_moe_align_block_size,
        "moe_sum": custom_moe_sum,
        "topk_softmax": custom_topk_softmax,
        "grouped_topk": custom_moe_grouped_topk,
    },
}


def init_vllm_libraries():
    global libs
    for lib_name, ops in _VLLM_OPS_SIGNATURES.items():
        for op_name, sig in ops.items():
            if not _is_op_registered(lib_name, op_name):
                torch.library.define(f"{lib_name}::{op_name}", sig)
    libs = {name: torch.library.Library(name, "IMPL") for name in _VLLM_OPS_SIGNATURES}


def patch_vllm_lib(lib_name, fn_name, fn, key, verbose=True):
    if lib_name not in libs:
        raise ValueError(f"Library {lib_name} is not recognized.")
    libs[lib_name].impl(fn_name, fn, key)
    if verbose:
        print(f"Patched torch.ops.{lib_name}.{fn_name} with FLAGGEMS {fn.__name__}")


def _patch_all(verbose):
    init_vllm_libraries()
    for lib_name, ops in _VLLM_OPS_IMPLS.items():
        for op_name, fn in ops.items():
            patch_vllm_lib(lib_name, op_name, fn, "CUDA", verbose)


def patch_empty_vllm() -> None:
    """Define (if absent) and implement the hot-path vLLM ops; idempotent."""
    global _flag_ops_registered
    if _flag_ops_registered:
        return
    _flag_ops_registered = True
    _patch_all(verbose=False)


def apply_gems_patches_to_vllm(verbose=True):
    """Override vLLM's own CUDA kernels for the hot-path ops with this package's."""
    import vllm  # noqa: F401
    import vllm._custom_ops  # noqa: F401

    global _flag_ops_registered
    _flag_ops_registered = True
    _patch_all(verbose)
