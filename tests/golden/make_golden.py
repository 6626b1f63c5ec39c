"""Regenerate tests/golden/*.pt from the reference's own golden functions.

Run where a checkout of the reference (FlagGems) is at hand and point
FLAGGEMS_REFERENCE at its root:

    FLAGGEMS_REFERENCE=<path to the FlagGems checkout> python tests/golden/make_golden.py

The reference package cannot be imported without an accelerator, so the pure
torch golden functions are lifted out of the reference's files by name (their
``def`` blocks are parsed with ``ast`` and executed in a namespace that holds
only torch/typing), run here on seeded CPU inputs, and their inputs and outputs
saved.  No reference source is written into this repository: only tensors.
tests/test_oracle_golden.py then checks the restatements in ``oracle/`` against
these files, bit for bit where the domain is integer/FP8 bytes.
"""
import ast
import os
import sys
from typing import Optional, Tuple  # noqa: F401  (names used by lifted code)

import torch

REF = os.environ.get("FLAGGEMS_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set FLAGGEMS_REFERENCE to the root of a FlagGems checkout")
OUT = os.path.dirname(os.path.abspath(__file__))


def lift(relpath, names):
    """Return {name: function} for top-level (or class-level static) defs."""
    src = open(os.path.join(REF, relpath)).read()
    tree = ast.parse(src)
    ns = {"torch": torch, "Optional": Optional, "Tuple": Tuple}
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, relpath, "exec"), ns)
            found[node.name] = ns[node.name]
    missing = set(names) - set(found)
    assert not missing, f"{relpath}: {missing} not found"
    return found


def save(name, obj):
    path = os.path.join(OUT, name + ".pt")
    torch.save(obj, path)
    print(f"{name}.pt  {os.path.getsize(path)} bytes")


def main():
    torch.set_num_threads(1)

    # ---- act_quant: tests/test_act_quant.py:48-98
    f = lift("tests/test_act_quant.py", ["torch_act_quant"])["torch_act_quant"]
    cases = []
    g = torch.Generator().manual_seed(0)
    for (m, n, bs, fmt, kind) in [
        (1, 128, 128, None, "randn"),
        (40, 896, 64, None, "randn"),
        (33, 2048, 128, "ue8m0", "randn"),
        (17, 256, 128, None, "tiny"),
        (8, 512, 512, None, "randn"),
        (5, 256, 64, "ue8m0", "wide"),
    ]:
        x = torch.randn(m, n, generator=g)
        if kind == "tiny":
            x = x * 1e-6
            x[0] = 0.0
        if kind == "wide":
            x = x * torch.logspace(-6, 4, n).unsqueeze(0)
        x = x.bfloat16()
        y, s = f(x, bs, fmt)
        cases.append(dict(x=x, block_size=bs, scale_fmt=fmt, y=y.view(torch.uint8), s=s))
    save("act_quant", cases)

    # ---- per-token-group quant: tests/test_fused_experts_impl.py:582-601 (divide by 448)
    fe = lift(
        "tests/test_fused_experts_impl.py",
        ["torch_per_token_group_quant_fp8", "torch_w8a8_block_matmul", "torch_w8a8_block_fp8_moe"],
    )
    # torch_w8a8_block_fp8_moe calls the other two by global name
    fe["torch_w8a8_block_fp8_moe"].__globals__.update(fe)
    cases = []
    for (m, k, gs, kind, dt) in [
        (7, 512, 128, "rand", torch.bfloat16),
        (83, 1024, 64, "randn", torch.bfloat16),
        (9, 1024, 256, "randn", torch.float16),
        (4, 256, 128, "tiny", torch.bfloat16),
        (6, 384, 128, "randn", torch.float32),
    ]:
        x = torch.rand(m, k, generator=g) if kind == "rand" else torch.randn(m, k, generator=g)
        if kind == "tiny":
            x = x * 1e-8
            x[0] = 0.0
        x = x.to(dt)
        q, s = fe["torch_per_token_group_quant_fp8"](x, gs)
        cases.append(dict(x=x, group_size=gs, q=q.view(torch.uint8), s=s))
    save("per_token_group_quant", cases)

    # the diverging golden (multiplies by fp32(1/448)): kept to document the 1-ulp gap
    fn = lift("tests/test_per_token_group_quant_fp8.py", ["native_per_token_group_quant_fp8"])[
        "native_per_token_group_quant_fp8"
    ]
    x = torch.rand(83, 512, generator=g).bfloat16()
    q, s = fn(x, 128, dtype=torch.float8_e4m3fn)
    q2, s2 = fn(x, 128, dtype=torch.float8_e4m3fn, scale_ue8m0=True)
    save("per_token_group_quant_native", dict(x=x, group_size=128, q=q.view(torch.uint8), s=s,
                                              q_ue8m0=q2.view(torch.uint8), s_ue8m0=s2))

    # ---- per-token quant: src/flag_gems/fused/fused_moe.py:629-698 (torch-eager branches)
    fq = lift("src/flag_gems/fused/fused_moe.py", ["_fp8_quantize"])["_fp8_quantize"]
    cases = []
    for (m, k, kind) in [(5, 256, "randn"), (64, 1024, "randn"), (3, 128, "tiny")]:
        x = torch.randn(m, k, generator=g)
        if kind == "tiny":
            x = x * 1e-7
            x[1] = 0
        x = x.bfloat16()
        q, s = fq(x, None, True, None)
        cases.append(dict(x=x, q=q.view(torch.uint8), s=s))
    save("per_token_quant", cases)
    # block branch, 3-D input so that the torch-eager code (not the Triton op) runs (:660-671)
    x = torch.randn(2, 6, 512, generator=g).bfloat16()
    q, s = fq(x, None, False, [128, 128])
    save("fp8_quantize_block3d", dict(x=x, q=q.view(torch.uint8), s=s))

    # per-tensor branches (:686-698): dynamic scale, then a given scale
    x = torch.randn(33, 512, generator=g).bfloat16()
    q_dyn, s_dyn = fq(x, None, False, None)
    given = torch.tensor([0.0123])
    q_st, _ = fq(x, given, False, None)
    save("fp8_quantize_per_tensor", dict(x=x, q_dynamic=q_dyn.view(torch.uint8), s_dynamic=s_dyn,
                                         scale_static=given, q_static=q_st.view(torch.uint8)))

    # ---- moe_align_block_size: tests/test_moe_align_block_size.py:28-123
    fa = lift("tests/test_moe_align_block_size.py", ["torch_moe_align_block_size"])[
        "torch_moe_align_block_size"
    ]
    cases = []
    for (t, topk, e, bs) in [(1, 2, 8, 8), (4, 2, 8, 8), (33, 2, 8, 64), (64, 8, 256, 64),
                             (1024, 10, 10, 16), (257, 6, 128, 32), (100, 4, 250, 16)]:
        if (t, topk) == (1, 2):
            ids = torch.tensor([[1, 3]], dtype=torch.int32)
        elif (t, topk) == (4, 2):
            ids = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]], dtype=torch.int32)
        else:
            ids = torch.randint(0, e, (t, topk), generator=g, dtype=torch.int32)
        max_pad = ids.numel() + e * (bs - 1)
        so = torch.empty(max_pad, dtype=torch.int32)
        eo = torch.empty(max_pad // bs, dtype=torch.int32)
        no = torch.empty(1, dtype=torch.int32)
        fa(ids, e, bs, so, eo, no)
        cases.append(dict(topk_ids=ids, num_experts=e, block_size=bs,
                          sorted_ids=so, expert_ids=eo, num_post_pad=no))
    save("moe_align", cases)

    # ---- block-scaled matmul: tests/test_fused_experts_impl.py:531-579
    cases = []
    for (m, n, k) in [(64, 128, 128), (33, 200, 384), (5, 256, 512)]:
        a = torch.randn(m, k, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
        b = torch.randn(n, k, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
        a_s = 0.01 * torch.rand(m, (k + 127) // 128, generator=g) + 0.005
        b_s = 0.01 * torch.rand((n + 127) // 128, (k + 127) // 128, generator=g) + 0.005
        c = fe["torch_w8a8_block_matmul"](a, b, a_s, b_s, [128, 128], torch.float32)
        cases.append(dict(a=a.view(torch.uint8), b=b.view(torch.uint8), a_s=a_s, b_s=b_s, c=c))
    save("block_scaled_mm", cases)

    # ---- scaled mm: tests/test_cutlass_scaled_mm.py:52-56,154-187
    fs = lift("tests/test_cutlass_scaled_mm.py", ["to_fp8", "baseline_scaled_mm"])
    cases = []
    for (m, n, k, pa, pb, bias) in [(1, 256, 128, False, False, False), (33, 256, 496, True, True, True),
                                    (64, 128, 256, True, False, True), (16, 48, 128, False, True, False)]:
        a = fs["to_fp8"](torch.randn(m, k, generator=g))
        b = fs["to_fp8"](torch.randn(n, k, generator=g)).t()
        sa = torch.randn(m if pa else 1, 1, generator=g)
        sb = torch.randn(1, n if pb else 1, generator=g)
        bi = torch.rand(n, generator=g).bfloat16() * 10 if bias else None
        c = fs["baseline_scaled_mm"](a, b, sa, sb, torch.float32, None)
        cases.append(dict(a=a.view(torch.uint8), b_nk=b.t().contiguous().view(torch.uint8),
                          sa=sa, sb=sb, bias=bi, c_f32_nobias=c))
    save("scaled_mm", cases)

    # ---- block-fp8 fused MoE: tests/test_fused_experts_impl.py:604-662
    t, h, i, e, topk = 24, 256, 128, 8, 2
    hidden = (torch.randn(t, h, generator=g) / 4).bfloat16()
    w1 = torch.randn(e, 2 * i, h, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
    w2 = torch.randn(e, h, i, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
    w1s = 0.01 * torch.rand(e, 2 * i // 128, h // 128, generator=g) + 0.002
    w2s = 0.01 * torch.rand(e, h // 128, i // 128, generator=g) + 0.002
    logits = torch.randn(t, e, generator=g)
    tw, ti = torch.topk(torch.softmax(logits, -1), topk)
    tw = (tw / tw.sum(-1, keepdim=True)).bfloat16()
    out = fe["torch_w8a8_block_fp8_moe"](hidden, w1, w2, w1s, w2s, tw, ti, [128, 128])
    save("fused_moe_block_fp8", dict(hidden=hidden, w1=w1.view(torch.uint8), w2=w2.view(torch.uint8),
                                     w1_scale=w1s, w2_scale=w2s, topk_weights=tw, topk_ids=ti, out=out))

    # ---- per-row fake-quantised FP8 MoE: tests/test_fused_experts_impl.py:465-528, on the input
    # recipe of test_accuracy_fused_moe_fp8 (:375-462): weights quantised per tensor (one scale per
    # expert), dequantised to bf16 for the golden.  A second set of cases quantises the weights
    # per output channel instead: the golden takes dequantised weights, so the same function
    # bounds the per-token x per-channel mode as well.
    fm = lift("tests/test_fused_experts_impl.py", ["_fake_quantize_fp8", "_fake_quantize_int8",
                                                   "torch_fused_moe_quantized_reference"])
    fm["torch_fused_moe_quantized_reference"].__globals__.update(fm)
    g2 = torch.Generator().manual_seed(0)
    cases = []
    for granularity in ("per_tensor", "per_channel"):
        for (t, e, h, i, topk) in [(4, 8, 128, 256, 2), (32, 4, 128, 128, 4)]:
            hidden = torch.randn(t, h, generator=g2).bfloat16()
            w1f = torch.randn(e, 2 * i, h, generator=g2) * (1.0 / h ** 0.5)
            w2f = torch.randn(e, h, i, generator=g2) * (1.0 / i ** 0.5)
            quant = []
            for w in (w1f, w2f):
                if granularity == "per_tensor":
                    sc = w.abs().amax(dim=(1, 2)).clamp(min=1e-10) / 448.0  # [E]
                    q = (w / sc[:, None, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
                    deq = (q.float() * sc[:, None, None]).bfloat16()
                else:
                    sc = w.abs().amax(dim=2).clamp(min=1e-10) / 448.0  # [E, N]
                    q = (w / sc[:, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
                    deq = (q.float() * sc[:, :, None]).bfloat16()
                quant.append((q, sc, deq))
            gating = torch.randn(t, e, generator=g2)
            tw, ti = torch.topk(torch.softmax(gating, -1), topk)
            tw = (tw / tw.sum(-1, keepdim=True)).bfloat16()
            out = fm["torch_fused_moe_quantized_reference"](hidden, quant[0][2], quant[1][2], tw, ti, quant_mode="fp8")
            cases.append(dict(granularity=granularity, hidden=hidden, w1=quant[0][0].view(torch.uint8),
                              w2=quant[1][0].view(torch.uint8), w1_scale=quant[0][1], w2_scale=quant[1][1],
                              topk_weights=tw, topk_ids=ti, out=out))
    save("fused_moe_fake_quant_fp8", cases)

    # ---- the same golden in its int8 mode, on the input recipe of test_fused_moe_int8 (:765-835):
    # weights quantised per output channel to int8 (scale amax / 127), dequantised to bf16 for the golden.
    g3 = torch.Generator().manual_seed(0)
    cases = []
    for (t, e, h, i, topk) in [(4, 8, 128, 256, 2), (32, 4, 128, 128, 4)]:
        hidden = torch.randn(t, h, generator=g3).bfloat16()
        quant = []
        for w in (torch.randn(e, 2 * i, h, generator=g3) * (1.0 / h ** 0.5),
                  torch.randn(e, h, i, generator=g3) * (1.0 / i ** 0.5)):
            sc = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / 127.0
            q = (w / sc).round().clamp(-128, 127).to(torch.int8)
            quant.append((q, sc.squeeze(-1), (q.float() * sc).bfloat16()))
        gating = torch.randn(t, e, generator=g3)
        tw, ti = torch.topk(torch.softmax(gating, -1), topk)
        tw = (tw / tw.sum(-1, keepdim=True)).bfloat16()
        out = fm["torch_fused_moe_quantized_reference"](hidden, quant[0][2], quant[1][2], tw, ti, quant_mode="int8")
        cases.append(dict(hidden=hidden, w1=quant[0][0], w2=quant[1][0], w1_scale=quant[0][1], w2_scale=quant[1][1],
                          topk_weights=tw, topk_ids=ti, out=out))
    save("fused_moe_fake_quant_int8", cases)

    # ---- weight-only golden (torch_fused_moe_weight_only_reference, :837-872) on the recipes of
    # test_fused_moe_int8_w8a16 (:880-950) and test_fused_moe_int4_w4a16 (:958-1030, int4 values in int8
    # containers): per-channel symmetric weights, bf16 activations, everything in fp32.
    wo = lift("tests/test_fused_experts_impl.py", ["torch_fused_moe_weight_only_reference"])
    g4 = torch.Generator().manual_seed(0)
    cases = []
    for bits, (t, e, h, i, topk) in ((8, (4, 8, 128, 256, 2)), (8, (32, 4, 128, 128, 4)), (4, (16, 4, 128, 128, 2))):
        qmax, qmin = (127, -128) if bits == 8 else (7, -8)
        hidden = torch.randn(t, h, generator=g4).bfloat16()
        quant = []
        for w in (torch.randn(e, 2 * i, h, generator=g4) * (1.0 / h ** 0.5),
                  torch.randn(e, h, i, generator=g4) * (1.0 / i ** 0.5)):
            sc = w.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10) / qmax
            quant.append(((w / sc).round().clamp(qmin, qmax).to(torch.int8), sc.squeeze(-1)))
        gating = torch.randn(t, e, generator=g4)
        tw, ti = torch.topk(torch.softmax(gating, -1), topk)
        tw = (tw / tw.sum(-1, keepdim=True)).bfloat16()
        out = wo["torch_fused_moe_weight_only_reference"](hidden, quant[0][0], quant[1][0], quant[0][1], quant[1][1],
                                                          tw, ti)
        cases.append(dict(bits=bits, hidden=hidden, w1=quant[0][0], w2=quant[1][0], w1_scale=quant[0][1],
                          w2_scale=quant[1][1], topk_weights=tw, topk_ids=ti, out=out))
    save("fused_moe_weight_only", cases)


if __name__ == "__main__":
    if not os.path.isdir(REF):
        sys.exit(f"reference checkout not found at {REF}")
    main()
