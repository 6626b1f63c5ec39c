from .fp8_matmul import fp8_matmul  # noqa: F401
from .per_token_group_quant_fp8 import SUPPORTED_FP8_DTYPE, per_token_group_quant_fp8  # noqa: F401
from .scaled_grouped_mm import scaled_grouped_mm  # noqa: F401
from .scaled_mm import scaled_mm, scaled_mm_out  # noqa: F401
from .w8a8_block_fp8_matmul import w8a8_block_fp8_matmul  # noqa: F401
from .w8a8_block_fp8_bmm import fp8_einsum, w8a8_block_fp8_bmm  # noqa: F401
