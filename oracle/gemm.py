"""CPU oracle: scaled FP8 matrix products (test infrastructure only)."""
from typing import Optional

import torch


def _bcast_scale(s: torch.Tensor, n: int, axis: int) -> torch.Tensor:
    s = s.float().reshape(-1)
    assert s.numel() in (1, n), f"scale numel {s.numel()} must be 1 or {n}"
    if axis == 0:
        return s.reshape(-1, 1) if s.numel() == n else s.reshape(1, 1)
    return s.reshape(1, -1) if s.numel() == n else s.reshape(1, 1)


def scaled_mm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    bias_after_round: bool = True,
) -> torch.Tensor:
    """c = out_dtype(b_scale[n] * (a_scale[m] * sum_k a[m,k] b[k,n])) (+ bias).

    a: [M,K] fp8, b: [K,N] fp8 (any strides), scales numel 1 / M / N.
    Follows the kernel epilogue src/flag_gems/fused/cutlass_scaled_mm.py:288-305
    (a_scale first, then b_scale, cast, then ``c += bias`` in the output dtype);
    ``bias_after_round=False`` gives the aten ``_scaled_mm`` variant of
    src/flag_gems/ops/scaled_mm.py:116-136 where the bias joins in fp32 before
    the cast.  tests/test_cutlass_scaled_mm.py:154-187 is the reference's golden
    of the same contract (it scales the operands first; equal up to fp32
    rounding).
    """
    m, k = a.shape
    n = b.shape[1]
    acc = torch.mm(a.float(), b.float())
    acc = _bcast_scale(a_scale, m, 0) * acc
    acc = _bcast_scale(b_scale, n, 1) * acc
    if bias is not None and not bias_after_round:
        acc = acc + bias.float().reshape(1, -1)
    if out_dtype == torch.float8_e4m3fn:
        # aten _scaled_mm with out_dtype=None stores the fp32 tile through an fp8 pointer
        # (src/flag_gems/ops/scaled_mm.py:134-136, :214-220): round to nearest even, saturating
        # at +-448 (the NVIDIA fp32 -> e4m3 conversion; torch's CPU cast would give NaN above 464)
        acc = acc.clamp(-448.0, 448.0)
    c = acc.to(out_dtype)
    if bias is not None and bias_after_round:
        c = c + bias.to(out_dtype).reshape(1, -1)
    return c


def block_scaled_mm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_s: torch.Tensor,
    b_s: torch.Tensor,
    block_n: int = 128,
    block_k: int = 128,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """C[m,n] = sum_kb (A[m,kb] . B[n,kb]) * As[m,kb] * Bs[n//block_n, kb].

    a: [..., K] fp8, b: [N, K] fp8, a_s: [..., ceil(K/bk)], b_s: [ceil(N/bn), ceil(K/bk)].
    Follows the kernel loop src/flag_gems/ops/w8a8_block_fp8_matmul.py:99-116
    and the reference's golden tests/test_fused_experts_impl.py:531-579.
    """
    k = a.shape[-1]
    m = a.numel() // k
    n = b.shape[0]
    af = a.reshape(m, k).float()
    bf = b.float()
    a_s = a_s.reshape(m, -1).float()
    kt = (k + block_k - 1) // block_k
    nt = (n + block_n - 1) // block_n
    assert a_s.shape[1] == kt and tuple(b_s.shape) == (nt, kt)
    bs_cols = b_s.float().repeat_interleave(block_n, dim=0)[:n]  # [N, kt]
    c = torch.zeros(m, n, dtype=torch.float32)
    for i in range(kt):
        ks = slice(i * block_k, min((i + 1) * block_k, k))
        part = torch.mm(af[:, ks], bf[:, ks].t())
        c += part * a_s[:, i : i + 1] * bs_cols[:, i].reshape(1, -1)
    return c.reshape(a.shape[:-1] + (n,)).to(out_dtype)


def scaled_grouped_mm(mat_a, mat_b, scale_a, scale_b, offs=None, bias=None, out_dtype=torch.bfloat16):
    """aten _scaled_grouped_mm in fp32 on the CPU: ``(chunk_a @ chunk_b) * scale_a * scale_b (+ bias)`` per group,
    cast to out_dtype, for the four operand forms (A 2-D / B 3-D rows grouped by offs; both 3-D; A 3-D / B 2-D
    columns grouped; both 2-D with the K range split).

    Follows the reference's own statement of the op, src/flag_gems/ops/scaled_grouped_mm.py:379-467
    (``_scaled_grouped_mm_fallback``), which is also the golden of tests/test_scaled_grouped_mm.py:129-215.
    """
    a_is_2d, b_is_2d = mat_a.dim() == 2, mat_b.dim() == 2
    a, b = mat_a.float(), mat_b.float()
    sa, sb = scale_a.float(), scale_b.float()
    bias = None if bias is None else bias.float()
    starts = [0] + ([] if offs is None else offs.tolist())

    def finish(chunk, s_a, s_b, bi):
        chunk = chunk * s_a.reshape(-1, 1) * s_b.reshape(1, -1)
        if bi is not None:
            chunk = chunk + bi
        return chunk.to(out_dtype)

    chunks = []
    if a_is_2d and not b_is_2d:
        for g in range(b.shape[0]):
            lo, hi = starts[g], starts[g + 1]
            bi = None if bias is None else (bias if bias.dim() == 1 else bias[g])
            chunks.append(finish(a[lo:hi] @ b[g], sa[lo:hi], sb[g], bi))
        return torch.cat(chunks, 0)
    if not a_is_2d and b_is_2d:
        for g in range(a.shape[0]):
            lo, hi = starts[g], starts[g + 1]
            chunks.append(finish(a[g] @ b[:, lo:hi], sa[g], sb[lo:hi], None if bias is None else bias[lo:hi]))
        return torch.cat(chunks, 1)
    if a_is_2d and b_is_2d:
        groups = len(starts) - 1
        sa, sb = sa.reshape(groups, a.shape[0]), sb.reshape(groups, b.shape[1])
        for g in range(groups):
            lo, hi = starts[g], starts[g + 1]
            bi = None if bias is None else (bias if bias.dim() == 1 else bias[g])
            chunks.append(finish(a[:, lo:hi] @ b[lo:hi], sa[g], sb[g], bi))
        return torch.stack(chunks, 0)
    for g in range(a.shape[0]):
        bi = None if bias is None else (bias if bias.dim() == 1 else bias[g])
        chunks.append(finish(a[g] @ b[g], sa[g], sb[g], bi))
    return torch.stack(chunks, 0)
