"""CPU oracle for the FP8 quantized-inference hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
``--impl reference`` legs do, and there only as the checker or as the timed
CPU arm, never as the product path.

Every function restates, in plain torch on the CPU (fp32 arithmetic unless the
reference says otherwise), one function of the reference FlagGems code base and
cites the file:line it follows.  The restatements are pinned by
``tests/golden/*.pt``: fixtures produced by executing the reference's own golden
functions (loaded from the reference's test files, see
``tests/golden/make_golden.py``) on seeded inputs.

Parity status: pinned for act_quant, per_token_group_quant_fp8,
moe_align_block_size, the block-scaled matmul and the block-fp8 fused MoE.  The
per-token x per-channel FP8 fused MoE has no test in the reference at all
("parity unpinned"): its oracle is restated from the kernel source only.  The router functions
(topk_softmax, grouped_topk) are likewise unpinned by goldens: the reference tests them only against
vLLM's CUDA ops at run time, which the GPU tests here repeat when those ops load.
"""
from .quant import (  # noqa: F401
    act_quant,
    per_token_group_quant_fp8,
    per_token_quant_fp8,
    per_tensor_quant_fp8,
    per_token_quant_int8,
    quantize_weight_per_channel,
    quantize_weight_block,
)
from .gemm import scaled_mm, block_scaled_mm, scaled_grouped_mm  # noqa: F401
from .router import topk_softmax, grouped_topk  # noqa: F401
from .moe import (  # noqa: F401
    moe_align_block_size,
    silu_and_mul,
    moe_sum,
    expert_rows_block_fp8,
    expert_rows_per_channel_fp8,
    fused_moe_block_fp8,
    fused_moe_per_channel_fp8,
    fused_moe_per_channel_int8,
    fused_moe_16bit,
    fused_moe_per_tensor_fp8,
    dense_block_fp8_mlp,
)
