"""CPU oracle: FP8 e4m3 quantization functions (test infrastructure only).

All arithmetic is IEEE fp32 on the CPU; the FP8 cast is torch's
round-to-nearest-even ``.to(torch.float8_e4m3fn)`` applied after clamping to
+-448 (an unclamped cast turns |v| >= 480 into NaN).
"""
from typing import Optional, Tuple

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
FP8_MIN = -448.0


def act_quant(
    x: torch.Tensor, block_size: int = 128, scale_fmt: Optional[str] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block-wise activation quantization.

    Follows tests/test_act_quant.py:48-98 (the reference's golden for
    src/flag_gems/fused/act_quant.py:45-108):
      amax = max|x| per block in fp32, clamped to >= 1e-4        (:68-69, kernel :81-82)
      scale = amax * fp32(1/448)                                  (:84,   kernel :95)
      scale_fmt != None: scale = 2^ceil(log2(scale)) by the exponent/mantissa
        bit test                                                  (:71-82, kernel :22-41)
      y = clamp(x * (1/scale), +-448) -> e4m3                     (:87-91)
    """
    assert x.is_contiguous(), "Input tensor must be contiguous"
    assert x.size(-1) % block_size == 0
    n = x.size(-1)
    x2 = x.reshape(-1, n)
    m = x2.size(0)
    nb = n // block_size
    xb = x2.reshape(m, nb, block_size).float()
    amax = xb.abs().amax(dim=-1).clamp(min=1e-4)
    inv448 = torch.tensor(1.0 / 448.0, dtype=torch.float32)
    scale = amax * inv448
    if scale_fmt is not None:
        bits = scale.view(torch.int32)
        exp = (bits >> 23) & 0xFF
        man = bits & ((1 << 23) - 1)
        e = (exp - 127 + (man != 0).int()).int()
        scale = ((e + 127) << 23).view(torch.float32)
    y = xb * (1.0 / scale.unsqueeze(-1))
    y = y.clamp(FP8_MIN, FP8_MAX).reshape(m, n).to(FP8).reshape(x.shape)
    s = scale.to(torch.float32).reshape(*x.shape[:-1], nb)
    return y, s


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    column_major_scales: bool = False,
    scale_ue8m0: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token-group quantization with vLLM semantics.

    Follows the kernel src/flag_gems/ops/per_token_group_quant_fp8.py:58-68 and
    the torch goldens src/flag_gems/fused/fused_moe.py:660-671 and
    tests/test_fused_experts_impl.py:582-601:
      s = max(amax, eps) / 448          (IEEE divide, :62-63)
      ue8m0: s = exp2(ceil(log2(max(|s|, 1e-10))))   (:65-66)
      q = clamp(x / s, +-448) -> e4m3   (:68)
    The reference's other golden (tests/test_per_token_group_quant_fp8.py:40)
    multiplies by fp32(1/448) instead; that differs by 1 ulp in about half of
    the scales and is deliberately not followed.
    column_major_scales: same values, stored with shape
      (K/g,) + x.shape[:-1] and returned permuted (-1,-2)  (:250-252).
    """
    assert x.shape[-1] % group_size == 0
    g = x.numel() // group_size
    xr = x.reshape(g, group_size).float()
    amax = xr.abs().amax(dim=-1, keepdim=True).clamp(min=eps)
    s = amax / FP8_MAX
    if scale_ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(torch.maximum(s.abs(), torch.tensor(1e-10)))))
    q = (xr / s).clamp(FP8_MIN, FP8_MAX).to(FP8).reshape(x.shape)
    s = s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))
    if column_major_scales:
        shape = (x.shape[-1] // group_size,) + x.shape[:-1]
        buf = torch.empty(shape, dtype=torch.float32).permute(-1, -2)
        buf.copy_(s)
        s = buf
    return q, s


def per_token_quant_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic per-token (per-row) quantization used by the per-channel MoE mode.

    Follows src/flag_gems/fused/fused_moe.py:673-684:
      s = max(rowamax, 1e-10) / 448; s = max(s, 1/(448*512)); q = clamp(x.float()/s)
    Scale shape: x.shape[:-1] + (1,).
    """
    xf = x.reshape(-1, x.size(-1))
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10).to(torch.float32)
    s = amax / FP8_MAX
    s = s.clamp(min=torch.tensor(1.0 / (FP8_MAX * 512.0), dtype=torch.float32))
    q = (xf.float() / s).clamp(FP8_MIN, FP8_MAX).to(FP8).reshape(x.shape)
    return q, s.reshape(x.shape[:-1] + (1,))


def per_tensor_quant_fp8(x: torch.Tensor, scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor quantisation, static or dynamic.

    Follows src/flag_gems/fused/fused_moe.py:686-698: with a given scale ``q = clamp(x.float() / scale)``;
    otherwise ``scale = max(max|x|, 1e-10) / 448`` and ``q = clamp(x.float() * (1 / scale))``.
    """
    if scale is not None:
        s = scale.float().reshape(-1)[:1]
        q = (x.float() / s).clamp(FP8_MIN, FP8_MAX).to(FP8)
        return q, s
    amax = x.abs().amax().clamp(min=1e-10).to(torch.float32)
    s = amax / FP8_MAX
    q = (x.float() * (1.0 / s)).clamp(FP8_MIN, FP8_MAX).to(FP8)
    return q, s.reshape(1)


def quantize_weight_per_channel(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Synthetic-weight helper: per-output-channel scales for W[..., N, K] fp32.

    s[n] = max(max|W[n,:]|, 1e-10)/448, Wq = RNE(clamp(W/s)).  Not a reference
    function; it manufactures FP8 weights for the benchmark configurations.
    """
    amax = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10).float()
    s = amax / FP8_MAX
    q = (w.float() / s).clamp(FP8_MIN, FP8_MAX).to(FP8)
    return q, s.squeeze(-1)


def quantize_weight_block(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Synthetic-weight helper: block x block scales for W[N, K] fp32.

    Bs[i,j] = max(max|W[block i, block j]|, 1e-10)/448 with shape
    [ceil(N/block), ceil(K/block)]; ragged edge blocks use the elements present.
    """
    n, k = w.shape
    nb, kb = (n + block - 1) // block, (k + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32)
    wp[:n, :k] = w.float()
    tiles = wp.reshape(nb, block, kb, block)
    amax = tiles.abs().amax(dim=(1, 3)).clamp(min=1e-10)
    s = amax / FP8_MAX
    q = (tiles / s[:, None, :, None]).clamp(FP8_MIN, FP8_MAX).reshape(nb * block, kb * block)
    return q[:n, :k].contiguous().to(FP8), s


def per_token_quant_int8(x: torch.Tensor):
    """Per-row INT8 quantisation: s = max(rowamax, 1e-10) / 127, q = clamp(round(x / s), -128, 127).

    Follows the per-token branch of ``_int8_quantize``, src/flag_gems/fused/fused_moe.py:732-739
    (``torch.round`` rounds halves to even)."""
    flat = x.reshape(-1, x.shape[-1])
    amax = flat.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10).to(torch.float32)
    scale = amax / 127.0
    q = (flat.float() / scale).round().clamp(-128, 127).to(torch.int8)
    return q.reshape(x.shape), scale.reshape(x.shape[:-1] + (1,))
