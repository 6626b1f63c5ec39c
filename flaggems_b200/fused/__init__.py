from .act_quant import act_quant_triton  # noqa: F401
from .cutlass_scaled_mm import cutlass_scaled_mm  # noqa: F401
from .fused_moe import (  # noqa: F401
    MoEActivation,
    dispatch_fused_moe_kernel,
    invoke_fused_moe_triton_kernel,
    fused_experts_impl,
    inplace_fused_experts,
    moe_kernel_quantize_input,
    outplace_fused_experts,
)
from .grouped_topk import grouped_topk  # noqa: F401
from .moe_align_block_size import moe_align_block_size, moe_align_block_size_triton  # noqa: F401
from .moe_sum import moe_sum  # noqa: F401
from .silu_and_mul import silu_and_mul, silu_and_mul_out  # noqa: F401
from .topk_softmax import topk_softmax  # noqa: F401
